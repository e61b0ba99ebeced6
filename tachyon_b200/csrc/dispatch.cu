// Token -> expert dispatch: per-expert histogram, prefix scan, and the stable
// permutation of the t*k (token, pick) slots into expert-contiguous order.
//
// The CPU path pushes each token's picks onto per-expert lists while walking
// tokens in order (src/model.rs:474-482), so within an expert the slots are in
// ascending token order and counts[e] is the list length. This file produces
// the same lists without a serial walk: a thread per token, a warp ballot per
// expert for the rank of a token among the earlier tokens of its CTA that
// picked the same expert, per-CTA histograms scanned across CTAs for the base,
// and a warp-shuffle exclusive scan over experts for each expert's first slot.
//
// Outputs: counts[E], offsets[E+1], perm[sorted slot] = token*k + j,
// pos[token*k + j] = sorted slot.
#include "common.cuh"

namespace tc {

namespace {

constexpr int DISPATCH_THREADS = 256;
constexpr int DISPATCH_WARPS = DISPATCH_THREADS / 32;

// Ballot pass over every expert. Each thread owns one token (or none) with its
// k picks in `mine`. For expert e the warp learns which lanes picked it;
// `on_expert(e, ballot, j)` runs on every lane, with j = the lane's pick index
// for e or -1.
template <class F>
__device__ __forceinline__ void for_each_expert(int experts, int topk, const uint32_t* mine,
                                                bool has_token, F on_expert) {
    for (int e = 0; e < experts; e++) {
        int j = -1;
        if (has_token) {
            for (int q = 0; q < topk; q++)
                if (mine[q] == uint32_t(e)) j = q;
        }
        unsigned ballot = __ballot_sync(0xffffffffu, j >= 0);
        on_expert(e, ballot, j);
    }
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
    __shared__ uint32_t wcount[DISPATCH_WARPS][MAX_EXPERTS];  // per-warp counts, then bases
    __shared__ uint32_t scount[MAX_EXPERTS];
    __shared__ uint32_t soff[MAX_EXPERTS + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool has = tid < t;
    uint32_t mine[MAX_TOPK];
    if (has)
        for (int q = 0; q < topk; q++) mine[q] = ids[size_t(tid) * topk + q];
    for_each_expert(experts, topk, mine, has, [&](int e, unsigned ballot, int) {
        if (lane == 0) wcount[warp][e] = __popc(ballot);
    });
    __syncthreads();
    for (int e = tid; e < experts; e += DISPATCH_THREADS) {
        uint32_t run = 0;
        for (int w = 0; w < DISPATCH_WARPS; w++) {
            uint32_t c = wcount[w][e];
            wcount[w][e] = run;
            run += c;
        }
        scount[e] = run;
        counts[e] = run;
    }
    __syncthreads();
    if (warp == 0) scan_experts(scount, soff, experts, lane);
    __syncthreads();
    for (int e = tid; e <= experts; e += DISPATCH_THREADS) offsets[e] = soff[e];
    const unsigned lt = (1u << lane) - 1u;
    for_each_expert(experts, topk, mine, has, [&](int e, unsigned ballot, int j) {
        if (j >= 0) {
            uint32_t p = soff[e] + wcount[warp][e] + __popc(ballot & lt);
            uint32_t slot = uint32_t(tid) * topk + j;
            perm[p] = slot;
            pos[slot] = p;
        }
    });
}

// Large batches, pass 1: each CTA's histogram of its DISPATCH_THREADS tokens.
__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_count_kernel(const uint32_t* __restrict__ ids, int t, int experts, int topk,
                      uint32_t* __restrict__ block_hist) {
    __shared__ uint32_t wcount[DISPATCH_WARPS][MAX_EXPERTS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int token = blockIdx.x * DISPATCH_THREADS + tid;
    const bool has = token < t;
    uint32_t mine[MAX_TOPK];
    if (has)
        for (int q = 0; q < topk; q++) mine[q] = ids[size_t(token) * topk + q];
    for_each_expert(experts, topk, mine, has, [&](int e, unsigned ballot, int) {
        if (lane == 0) wcount[warp][e] = __popc(ballot);
    });
    __syncthreads();
    for (int e = tid; e < experts; e += DISPATCH_THREADS) {
        uint32_t run = 0;
        for (int w = 0; w < DISPATCH_WARPS; w++) run += wcount[w][e];
        block_hist[size_t(blockIdx.x) * experts + e] = run;
    }
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
    __shared__ uint32_t wcount[DISPATCH_WARPS][MAX_EXPERTS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int token = blockIdx.x * DISPATCH_THREADS + tid;
    const bool has = token < t;
    uint32_t mine[MAX_TOPK];
    if (has)
        for (int q = 0; q < topk; q++) mine[q] = ids[size_t(token) * topk + q];
    for_each_expert(experts, topk, mine, has, [&](int e, unsigned ballot, int) {
        if (lane == 0) wcount[warp][e] = __popc(ballot);
    });
    __syncthreads();
    for (int e = tid; e < experts; e += DISPATCH_THREADS) {
        uint32_t run = offsets[e] + block_base[size_t(blockIdx.x) * experts + e];
        for (int w = 0; w < DISPATCH_WARPS; w++) {
            uint32_t c = wcount[w][e];
            wcount[w][e] = run;
            run += c;
        }
    }
    __syncthreads();
    const unsigned lt = (1u << lane) - 1u;
    for_each_expert(experts, topk, mine, has, [&](int e, unsigned ballot, int j) {
        if (j >= 0) {
            uint32_t p = wcount[warp][e] + __popc(ballot & lt);
            uint32_t slot = uint32_t(token) * topk + j;
            perm[p] = slot;
            pos[slot] = p;
        }
    });
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
