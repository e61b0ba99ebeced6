// Self-check of the tcgen05 building blocks: one 128 x N x 32 int8 MMA from
// shared memory into tensor memory, read back to global memory. Used by the
// test-suite (through tc_umma_selftest) to pin the descriptor encodings and the
// tile layout before the grouped kernels rely on them. Every wait is bounded.
#include "experts_common.cuh"
#include "umma.cuh"

namespace tc {

namespace {

template <int N>
__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const int8_t* __restrict__ a_tile, const int8_t* __restrict__ b_tile, int* __restrict__ d_out,
                  int* __restrict__ status) {
    __shared__ __align__(128) uint8_t s_a[128 * 32];
    __shared__ __align__(128) uint8_t s_b[N * 32];
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Tiles are already in the canonical order in global memory: plain copy.
    for (int i = tid; i < 128 * 32 / 16; i += 128)
        reinterpret_cast<uint4*>(s_a)[i] = reinterpret_cast<const uint4*>(a_tile)[i];
    for (int i = tid; i < N * 32 / 16; i += 128)
        reinterpret_cast<uint4*>(s_b)[i] = reinterpret_cast<const uint4*>(b_tile)[i];
    if (tid == 0) {
        mbar_init(&s_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Generic-proxy writes above must be visible to the tensor core's async-proxy reads.
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        umma::tmem_alloc(&s_tmem, 64 < N ? 128 : 64);
        umma::tmem_relinquish();
    }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = s_tmem;
    if (warp == 0 && lane == 0) {
        const uint64_t da = umma::smem_desc(smem_addr(s_a), 128 * 16, 128);
        const uint64_t db = umma::smem_desc(smem_addr(s_b), N * 16, 128);
        umma::mma_s8(tmem, da, db, umma::idesc_s8(128, N), 0u);
        umma::commit(&s_bar);
    }
    const bool landed = mbar_wait_bounded(&s_bar, 0);
    umma::fence_after_sync();
    if (landed) {
#pragma unroll
        for (int c0 = 0; c0 < N; c0 += 32) {
            int v[32];
            umma::ld_32x32(tmem + (uint32_t(warp * 32) << 16) + c0, v);
            umma::wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j++) d_out[(warp * 32 + lane) * N + c0 + j] = v[j];
        }
    } else if (tid == 0) {
        atomicExch(status, ERR_COPY_WAIT_TIMEOUT);
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 64 < N ? 128 : 64);
}

}  // namespace

// a_tile: 128 x 32 int8, b_tile: n x 32 int8, both in the canonical tile order;
// d_out: 128 x n int32 row-major. n is 64 or 128.
int launch_umma_selftest(const int8_t* a_tile, const int8_t* b_tile, int n, int* d_out, int* status,
                      cudaStream_t stream) {
    if (n == 64)
        umma_selftest_kernel<64><<<1, 128, 0, stream>>>(a_tile, b_tile, d_out, status);
    else if (n == 128)
        umma_selftest_kernel<128><<<1, 128, 0, stream>>>(a_tile, b_tile, d_out, status);
    else
        return -1;
    return 1;
}

}  // namespace tc
