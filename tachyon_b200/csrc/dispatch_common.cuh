// Device-side pieces of the token -> expert dispatch, shared by the stand-alone
// dispatch kernels and by the router kernel, whose last CTA runs the
// single-CTA dispatch itself when the batch fits one CTA.
#pragma once

#include "common.cuh"

namespace tc {

constexpr int DISPATCH_THREADS = 256;
constexpr int DISPATCH_WARPS = DISPATCH_THREADS / 32;

// Sets this token's bits and returns with bits[e][w] complete (after a CTA barrier).
// An id outside [0, experts) or an expert named twice by one token is not marked:
// the slot is left out of the dispatch and *status is set to ERR_BAD_EXPERT_ID.
__device__ __forceinline__ void mark_picks(uint32_t (*bits)[DISPATCH_WARPS], const uint32_t* ids,
                                           int token, int t, int experts, int topk, int* status) {
    const int tid = threadIdx.x;
    for (int i = tid; i < experts * DISPATCH_WARPS; i += DISPATCH_THREADS) (&bits[0][0])[i] = 0;
    __syncthreads();
    if (token < t) {
        const int warp = tid >> 5, lane = tid & 31;
        for (int q = 0; q < topk; q++) {
            const uint32_t e = ids[size_t(token) * topk + q];
            const bool bad = e >= uint32_t(experts) || ((atomicOr(&bits[e][warp], 1u << lane) >> lane) & 1u);
            if (bad && status) atomicExch(status, ERR_BAD_EXPERT_ID);
        }
    }
    __syncthreads();
}

// True for a pick the dispatch places: a valid expert id, and the first of the token's
// picks to name that expert.
__device__ __forceinline__ bool pick_is_placed(const uint32_t* ids, int token, int q, int experts, int topk) {
    const uint32_t e = ids[size_t(token) * topk + q];
    if (e >= uint32_t(experts)) return false;
    for (int p = 0; p < q; p++)
        if (ids[size_t(token) * topk + p] == e) return false;
    return true;
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

// The experts with tokens, ascending, by one warp; active[experts] = their number.
__device__ __forceinline__ void list_active(const uint32_t* counts, int experts, int* active, int lane) {
    int n = 0;
    for (int e0 = 0; e0 < experts; e0 += 32) {
        const int e = e0 + lane;
        const bool on = e < experts && counts[e] > 0;
        const unsigned ballot = __ballot_sync(0xffffffffu, on);
        if (on) active[n + __popc(ballot & ((1u << lane) - 1u))] = e;
        n += __popc(ballot);
    }
    if (lane == 0) active[experts] = n;
}

// Shared memory of the single-CTA dispatch.
struct DispatchSmem {
    uint32_t bits[MAX_EXPERTS][DISPATCH_WARPS];
    uint32_t scount[MAX_EXPERTS];
    uint32_t soff[MAX_EXPERTS + 1];
};

// Small batches (t <= DISPATCH_THREADS): the whole dispatch by one CTA of
// DISPATCH_THREADS threads.
__device__ __forceinline__ void dispatch_small_body(DispatchSmem& sm, const uint32_t* ids, int t, int experts,
                                                    int topk, uint32_t* counts, uint32_t* offsets,
                                                    uint32_t* perm, uint32_t* pos, uint32_t* slot_token,
                                                    int* active, int* status) {
    uint32_t (*bits)[DISPATCH_WARPS] = sm.bits;
    uint32_t* scount = sm.scount;
    uint32_t* soff = sm.soff;
    const int tid = threadIdx.x;
    mark_picks(bits, ids, tid, t, experts, topk, status);
    for (int e = tid; e < experts; e += DISPATCH_THREADS) {
        const uint32_t n = row_count(bits, e);
        scount[e] = n;
        counts[e] = n;
    }
    __syncthreads();
    if (tid < 32) scan_experts(scount, soff, experts, tid);
    if (tid >= 32 && tid < 64) list_active(scount, experts, active, tid - 32);
    __syncthreads();
    for (int e = tid; e <= experts; e += DISPATCH_THREADS) offsets[e] = soff[e];
    if (tid < t) {
        for (int q = 0; q < topk; q++) {
            const uint32_t slot = uint32_t(tid) * topk + q;
            if (!pick_is_placed(ids, tid, q, experts, topk)) continue;
            const int e = ids[slot];
            const uint32_t p = soff[e] + rank_in_cta(bits, e, tid);
            perm[p] = slot;
            slot_token[p] = tid;
            pos[slot] = p;
        }
    }
}

}  // namespace tc
