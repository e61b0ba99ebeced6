// tcgen05 (5th-generation tensor core) building blocks for sm_100a: shared-memory
// matrix descriptors, the instruction descriptor for int8 x int8 -> int32,
// TMEM allocation, MMA issue, commit, and TMEM loads. One thread issues an MMA
// for the whole CTA; accumulators live in tensor memory (128 lanes x 512
// 32-bit columns per SM) and come back to registers with tcgen05.ld.
//
// Operand tiles sit in shared memory in the K-major "no swizzle" canonical
// layout: 8-row x 16-byte core matrices, each 128 contiguous bytes. For a tile
// of R rows x 32 bytes of K (one quantization block of int8):
//     offset(row, kbyte) = (kbyte / 16) * (R / 8) * 128 + (row / 8) * 128 + (row % 8) * 16 + kbyte % 16
// so SBO (stride between 8-row groups) = 128 bytes and LBO (stride between the
// two 16-byte K halves) = R * 16 bytes. Global memory holds the tiles in
// exactly this order, so one bulk copy brings a tile in ready for the MMA.
#pragma once

#include <stdint.h>

namespace tc {
namespace umma {

// 64-bit shared-memory matrix descriptor (K-major, no swizzle).
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr >> 4) & 0x3FFFu);         // start address, 16-byte units
    d |= uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16;   // leading (K) byte offset
    d |= uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32;   // stride (row-group) byte offset
    d |= uint64_t(1) << 46;                            // descriptor version for sm_100
    return d;                                          // base offset 0, layout type 0 = no swizzle
}

// Instruction descriptor: D s32, A and B signed 8-bit, both K-major, dense.
__host__ __device__ constexpr uint32_t idesc_s8(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     uint32_t(__cvta_generic_to_shared(dst_smem))),
                 "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, one K = 32 step; issued by ONE thread.
__device__ __forceinline__ void mma_s8(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

// Arrives on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     uint32_t(__cvta_generic_to_shared(bar)))
                 : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes (this warp's quadrant) x 32 consecutive 32-bit columns: thread i gets lane i's 32 values.
__device__ __forceinline__ void ld_32x32(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

// The same for 16 columns.
__device__ __forceinline__ void ld_32x16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

// Waits for this thread's TMEM loads. The values pass through the statement so
// that no use of them can be scheduled above the wait.
__device__ __forceinline__ void wait_ld(int (&v)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                   "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]),
                   "+r"(v[15])
                 :
                 : "memory");
}

// Byte offset of (row, kbyte) inside a tile of `rows` rows x 32 K-bytes.
__host__ __device__ constexpr uint32_t tile_offset(uint32_t rows, uint32_t row, uint32_t kbyte) {
    return (kbyte / 16) * (rows / 8) * 128 + (row / 8) * 128 + (row % 8) * 16 + kbyte % 16;
}

}  // namespace umma
}  // namespace tc
