// Token -> expert dispatch: per-expert histogram, prefix scan, and the stable
// permutation of the t*k (token, pick) slots into expert-contiguous order.
//
// The CPU path pushes each token's picks onto per-expert lists while walking
// tokens in order (src/model.rs:474-482), so within an expert the slots are in
// ascending token order and counts[e] is the list length. This file produces
// the same lists without a serial walk. A CTA owns 256 consecutive tokens, a
// thread per token. Each thread sets one bit per pick in a shared bit matrix
// (expert x token); a token's rank among the CTA's earlier tokens that picked
// the same expert is then a popcount of that expert's row below its own bit.
// Per-CTA histograms (row popcounts) are scanned across CTAs for the CTA's
// base, and a warp-shuffle exclusive scan over experts gives each expert's
// first slot.
//
// Outputs: counts[E], offsets[E+1], perm[sorted slot] = token*k + j,
// pos[token*k + j] = sorted slot.
#include "common.cuh"

namespace tc {

namespace {

constexpr int DISPATCH_THREADS = 256;
constexpr int DISPATCH_WARPS = DISPATCH_THREADS / 32;

// Sets this token's bits and returns with bits[e][w] complete (after a CTA barrier).
__device__ __forceinline__ void mark_picks(uint32_t (*bits)[DISPATCH_WARPS], const uint32_t* ids,
                                           int token, int t, int experts, int topk) {
    const int tid = threadIdx.x;
    for (int i = tid; i < experts * DISPATCH_WARPS; i += DISPATCH_THREADS) (&bits[0][0])[i] = 0;
    __syncthreads();
    if (token < t) {
        const int warp = tid >> 5, lane = tid & 31;
        for (int q = 0; q < topk; q++)
            atomicOr(&bits[ids[size_t(token) * topk + q]][warp], 1u << lane);
    }
    __syncthreads();
}

__device__ __forceinline__ uint32_t row_count(const uint32_t (*bits)[DISPATCH_WARPS], int e) {
    uint32_t n = 0;
#pragma unroll
    for (int w = 0; w < DISPATCH_WARPS; w++) n += __popc(bits[e][w]);
    return n;
}

// Tokens of this CTA before `tid` that picked expert e.
__device__ __forceinline__ uint32_t rank_in_cta(const uint32_t (*bits)[DISPATCH_WARPS], int e, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    uint32_t n = __popc(bits[e][warp] & ((1u << lane) - 1u));
#pragma unroll
    for (int w = 0; w < DISPATCH_WARPS; w++)
        if (w < warp) n += __popc(bits[e][w]);
    return n;
}

// Exclusive scan of counts[0..experts) into offsets[0..experts], by one warp:
// each lane sums a contiguous run of experts, the runs are scanned with
// shuffles, then each lane writes its run.
__device__ __forceinline__ void scan_experts(const uint32_t* counts, uint32_t* offsets, int experts,
                                             int lane) {
    const int per = (experts + 31) / 32;
    uint32_t local = 0;
    for (int i = 0; i < per; i++) {
        int e = lane * per + i;
        if (e < experts) local += counts[e];
    }
    uint32_t incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    uint32_t run = incl - local;
    for (int i = 0; i < per; i++) {
        int e = lane * per + i;
        if (e < experts) {
            offsets[e] = run;
            run += counts[e];
        }
    }
    if (lane == 31) offsets[experts] = incl;
}

// Small batches (t <= DISPATCH_THREADS): the whole dispatch in one CTA.
__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_small_kernel(const uint32_t* __restrict__ ids, int t, int experts, int topk,
                      uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets,
                      uint32_t* __restrict__ perm, uint32_t* __restrict__ pos) {
    __shared__ uint32_t bits[MAX_EXPERTS][DISPATCH_WARPS];
    __shared__ uint32_t scount[MAX_EXPERTS];
    __shared__ uint32_t soff[MAX_EXPERTS + 1];
    const int tid = threadIdx.x;
    mark_picks(bits, ids, tid, t, experts, topk);
    for (int e = tid; e < experts; e += DISPATCH_THREADS) {
        const uint32_t n = row_count(bits, e);
        scount[e] = n;
        counts[e] = n;
    }
    __syncthreads();
    if (tid < 32) scan_experts(scount, soff, experts, tid);
    __syncthreads();
    for (int e = tid; e <= experts; e += DISPATCH_THREADS) offsets[e] = soff[e];
    if (tid < t) {
        for (int q = 0; q < topk; q++) {
            const uint32_t slot = uint32_t(tid) * topk + q;
            const int e = ids[slot];
            const uint32_t p = soff[e] + rank_in_cta(bits, e, tid);
            perm[p] = slot;
            pos[slot] = p;
        }
    }
}

// Large batches, pass 1: each CTA's histogram of its DISPATCH_THREADS tokens.
__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_count_kernel(const uint32_t* __restrict__ ids, int t, int experts, int topk,
                      uint32_t* __restrict__ block_hist) {
    __shared__ uint32_t bits[MAX_EXPERTS][DISPATCH_WARPS];
    const int tid = threadIdx.x;
    mark_picks(bits, ids, blockIdx.x * DISPATCH_THREADS + tid, t, experts, topk);
    for (int e = tid; e < experts; e += DISPATCH_THREADS)
        block_hist[size_t(blockIdx.x) * experts + e] = row_count(bits, e);
}

// Pass 2 (one CTA): per expert, scan the CTA histograms into CTA bases; then
// the exclusive scan over experts.
__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_scan_kernel(uint32_t* __restrict__ block_hist, int blocks, int experts,
                     uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets) {
    __shared__ uint32_t scount[MAX_EXPERTS];
    __shared__ uint32_t soff[MAX_EXPERTS + 1];
    const int tid = threadIdx.x;
    for (int e = tid; e < experts; e += DISPATCH_THREADS) {
        uint32_t run = 0;
        for (int b = 0; b < blocks; b++) {
            uint32_t c = block_hist[size_t(b) * experts + e];
            block_hist[size_t(b) * experts + e] = run;
            run += c;
        }
        scount[e] = run;
        counts[e] = run;
    }
    __syncthreads();
    if (tid < 32) scan_experts(scount, soff, experts, tid);
    __syncthreads();
    for (int e = tid; e <= experts; e += DISPATCH_THREADS) offsets[e] = soff[e];
}

// Pass 3: every slot's sorted position.
__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_permute_kernel(const uint32_t* __restrict__ ids, int t, int experts, int topk,
                        const uint32_t* __restrict__ block_base,
                        const uint32_t* __restrict__ offsets, uint32_t* __restrict__ perm,
                        uint32_t* __restrict__ pos) {
    __shared__ uint32_t bits[MAX_EXPERTS][DISPATCH_WARPS];
    const int tid = threadIdx.x;
    const int token = blockIdx.x * DISPATCH_THREADS + tid;
    mark_picks(bits, ids, token, t, experts, topk);
    if (token < t) {
        for (int q = 0; q < topk; q++) {
            const uint32_t slot = uint32_t(token) * topk + q;
            const int e = ids[slot];
            const uint32_t p = offsets[e] + block_base[size_t(blockIdx.x) * experts + e] +
                               rank_in_cta(bits, e, tid);
            perm[p] = slot;
            pos[slot] = p;
        }
    }
}

}  // namespace

int launch_dispatch(const MoeDims& d, int t, Workspace& ws, cudaStream_t stream) {
    if (t <= DISPATCH_THREADS) {
        dispatch_small_kernel<<<1, DISPATCH_THREADS, 0, stream>>>(ws.ids, t, d.experts, d.topk,
                                                                  ws.counts, ws.offsets, ws.perm,
                                                                  ws.pos);
        return 1;
    }
    const int blocks = (t + DISPATCH_THREADS - 1) / DISPATCH_THREADS;
    dispatch_count_kernel<<<blocks, DISPATCH_THREADS, 0, stream>>>(ws.ids, t, d.experts, d.topk,
                                                                   ws.block_hist);
    dispatch_scan_kernel<<<1, DISPATCH_THREADS, 0, stream>>>(ws.block_hist, blocks, d.experts,
                                                             ws.counts, ws.offsets);
    dispatch_permute_kernel<<<blocks, DISPATCH_THREADS, 0, stream>>>(
        ws.ids, t, d.experts, d.topk, ws.block_hist, ws.offsets, ws.perm, ws.pos);
    return 3;
}

}  // namespace tc
