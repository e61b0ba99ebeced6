// The dense int8 rate of the 5th-generation tensor cores, measured: every SM issues
// tcgen05.mma.kind::i8 (M 128 x N 256 x K 32, accumulating in tensor memory) back to back
// from operand tiles that stay in shared memory, for a requested number of instructions.
// No global memory traffic, no epilogue: the figure the prefill-size expert kernels'
// tensor-pipe fraction is stated against. (Tachyon has nothing like it; its Metal
// backend quotes no peak.)
//
// One CTA per SM; one thread issues. Two accumulators of 256 columns alternate, a batch
// of instructions per commit; the issuer waits (bounded) for the batch before the
// previous one, so the pipe always has a batch queued behind the one it runs. Tensor
// memory is freed on every path.
#include "experts_common.cuh"
#include "umma.cuh"

namespace tc {

namespace {

constexpr int PK_M = 128, PK_N = 256, PK_BATCH = 32;

__global__ void __launch_bounds__(128, 1) int8_peak_kernel(int batches, int* status) {
    __shared__ __align__(128) uint8_t s_a[PK_M * 32];
    __shared__ __align__(128) uint8_t s_b[PK_N * 32];
    __shared__ __align__(8) uint64_t s_bar[2];
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < PK_M * 32 / 4; i += 128) reinterpret_cast<uint32_t*>(s_a)[i] = 0x01010101u;
    for (int i = tid; i < PK_N * 32 / 4; i += 128) reinterpret_cast<uint32_t*>(s_b)[i] = 0x01010101u;
    if (tid == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        umma::tmem_alloc(&s_tmem, 2 * PK_N);
        umma::tmem_relinquish();
    }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = s_tmem;
    if (tid == 0) {
        const uint64_t da = umma::smem_desc(smem_addr(s_a), PK_M * 16, 128);
        const uint64_t db = umma::smem_desc(smem_addr(s_b), PK_N * 16, 128);
        const uint32_t idesc = umma::idesc_s8(PK_M, PK_N);
        bool ok = true;
        for (int b = 0; b < batches && ok; b++) {
            const int buf = b & 1;
            // This accumulator's previous batch (b - 2) must be done before it is restarted.
            if (b >= 2) ok = mbar_wait_bounded(&s_bar[buf], ((b - 2) >> 1) & 1);
            if (!ok) break;
            for (int i = 0; i < PK_BATCH; i++)
                umma::mma_s8(tmem + buf * PK_N, da, db, idesc, i ? 1u : 0u);
            umma::commit(&s_bar[buf]);
        }
        // Everything issued has completed before tensor memory is released.
        for (int b = max(0, batches - 2); b < batches; b++)
            if (!mbar_wait_bounded(&s_bar[b & 1], (b >> 1) & 1)) ok = false;
        if (!ok) atomicExch(status, ERR_COPY_WAIT_TIMEOUT);
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 2 * PK_N);
}

}  // namespace

// Enqueues the measurement: `batches` batches of PK_BATCH instructions on each of `sms`
// SMs. Returns the integer operations (multiply and add counted separately) it performs.
double launch_int8_peak(int sms, int batches, int* status, cudaStream_t stream) {
    int8_peak_kernel<<<sms, 128, 0, stream>>>(batches, status);
    return 2.0 * PK_M * PK_N * 32.0 * double(PK_BATCH) * double(batches) * double(sms);
}

}  // namespace tc
