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
// slot_token[sorted slot] = token, pos[token*k + j] = sorted slot, and the
// ascending list of experts that have tokens (active[0..n), active[E] = n),
// which the expert kernels cut into equal shares.
#include <atomic>

#include <atomic>

#include "dispatch_common.cuh"

namespace tc {

namespace {

// `ids` carries no __restrict__ in the kernels that may wait for other ranks: in the
// peer-memory exchange other GPUs store the ids while the kernel is already resident,
// so the loads must not be treated as reads of memory that never changes.
__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_small_kernel(const uint32_t* ids, int t, int experts, int topk,
                      uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets,
                      uint32_t* __restrict__ perm, uint32_t* __restrict__ pos,
                      uint32_t* __restrict__ slot_token, int* __restrict__ active, const PeerWait pw,
                      int* status) {
    __shared__ DispatchSmem sm;
    if (pw.flags) {  // the ids come from other ranks: all of them have signalled this block
        if (int(threadIdx.x) < pw.ranks) peer_wait(pw, threadIdx.x);
        __syncthreads();
    }
    dispatch_small_body(sm, ids, t, experts, topk, counts, offsets, perm, pos, slot_token, active, status);
}

// Large batches, pass 1: each CTA's histogram of its DISPATCH_THREADS tokens.
__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_count_kernel(const uint32_t* ids, int t, int experts, int topk,
                      uint32_t* __restrict__ block_hist, const PeerWait pw, int* status) {
    __shared__ uint32_t bits[MAX_EXPERTS][DISPATCH_WARPS];
    const int tid = threadIdx.x;
    if (pw.flags) {
        if (tid < pw.ranks) peer_wait(pw, tid);
        __syncthreads();
    }
    mark_picks(bits, ids, blockIdx.x * DISPATCH_THREADS + tid, t, experts, topk, status);
    for (int e = tid; e < experts; e += DISPATCH_THREADS)
        block_hist[size_t(blockIdx.x) * experts + e] = row_count(bits, e);
}

// Pass 2 (one CTA): per expert, scan the CTA histograms into CTA bases; then
// the exclusive scan over experts.
__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_scan_kernel(uint32_t* __restrict__ block_hist, int blocks, int experts,
                     uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets,
                     int* __restrict__ active) {
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
    if (tid >= 32 && tid < 64) list_active(scount, experts, active, tid - 32);
    __syncthreads();
    for (int e = tid; e <= experts; e += DISPATCH_THREADS) offsets[e] = soff[e];
}

// Pass 3: every slot's sorted position. (Bad ids were reported by pass 1.)
__global__ void __launch_bounds__(DISPATCH_THREADS)
dispatch_permute_kernel(const uint32_t* __restrict__ ids, int t, int experts, int topk,
                        const uint32_t* __restrict__ block_base,
                        const uint32_t* __restrict__ offsets, uint32_t* __restrict__ perm,
                        uint32_t* __restrict__ pos, uint32_t* __restrict__ slot_token) {
    __shared__ uint32_t bits[MAX_EXPERTS][DISPATCH_WARPS];
    const int tid = threadIdx.x;
    const int token = blockIdx.x * DISPATCH_THREADS + tid;
    mark_picks(bits, ids, token, t, experts, topk, nullptr);
    if (token < t) {
        for (int q = 0; q < topk; q++) {
            const uint32_t slot = uint32_t(token) * topk + q;
            if (!pick_is_placed(ids, token, q, experts, topk)) continue;
            const int e = ids[slot];
            const uint32_t p = offsets[e] + block_base[size_t(blockIdx.x) * experts + e] +
                               rank_in_cta(bits, e, tid);
            perm[p] = slot;
            slot_token[p] = token;
            pos[slot] = p;
        }
    }
}

}  // namespace

int launch_dispatch(const MoeDims& d, int t, Workspace& ws, cudaStream_t stream) {
    if (t <= DISPATCH_THREADS) {
        dispatch_small_kernel<<<1, DISPATCH_THREADS, 0, stream>>>(ws.ids, t, d.experts, d.topk,
                                                                  ws.counts, ws.offsets, ws.perm,
                                                                  ws.pos, ws.slot_token, ws.active,
                                                                  ws.dispatch_wait, ws.status);
        return 1;
    }
    const int blocks = (t + DISPATCH_THREADS - 1) / DISPATCH_THREADS;
    dispatch_count_kernel<<<blocks, DISPATCH_THREADS, 0, stream>>>(ws.ids, t, d.experts, d.topk,
                                                                   ws.block_hist, ws.dispatch_wait,
                                                                   ws.status);
    dispatch_scan_kernel<<<1, DISPATCH_THREADS, 0, stream>>>(ws.block_hist, blocks, d.experts,
                                                             ws.counts, ws.offsets, ws.active);
    dispatch_permute_kernel<<<blocks, DISPATCH_THREADS, 0, stream>>>(
        ws.ids, t, d.experts, d.topk, ws.block_hist, ws.offsets, ws.perm, ws.pos, ws.slot_token);
    return 3;
}

// ---------------------------------------------------------------------------
// Dispatch for callers that must not allocate.
//
// The three-pass dispatch above needs one piece of scratch besides its inputs
// and outputs: the per-CTA histograms (block_hist). launch_dispatch() takes it
// from the workspace a layer allocates when it is created. The entry point
// below instead keeps it in the array that follows, which lives in the
// library's image: every GPU that loads the library holds these 64 KiB until
// the process exits, and no call ever allocates or frees anything.
//
// Limits that follow from the array's size: at most STATIC_MAX_TOKENS tokens
// (64 CTAs of 256) and MAX_EXPERTS experts per call.
//
// The array is shared by every call on a device and keeps whatever the last
// call left in it. Nothing in it has to start at zero: pass 1 overwrites every
// entry that passes 2 and 3 read. Two calls whose kernels overlap on the GPU
// (different streams, or different contexts on one device) would race on it.
//
// What the caller must guarantee about ids: every value below `experts`, and no
// expert named twice by one token. A value that breaks this is not placed (its
// slot is missing from counts, perm and pos) and the next tc_sync reports it.
constexpr int STATIC_MAX_BLOCKS = 64;
constexpr int STATIC_MAX_TOKENS = STATIC_MAX_BLOCKS * DISPATCH_THREADS;
static __device__ __align__(256) uint32_t g_static_block_hist[STATIC_MAX_BLOCKS * MAX_EXPERTS];
// Where the kernels of this entry point report an expert id they refused to place
// (ERR_BAD_EXPERT_ID). Also part of the library's image, for the same reason.
static __device__ int g_static_status;

namespace {
// In host code the arrays' names are only stand-ins; the device addresses come from
// the runtime, once per device. Each slot is written once (to the same value by
// whoever gets there first) and only read afterwards.
constexpr int MAX_DEVICES = 64;
struct StaticAddresses {
    std::atomic<uint32_t*> block_hist{nullptr};
    std::atomic<int*> status{nullptr};
};
StaticAddresses g_static_dev[MAX_DEVICES];
}  // namespace

const char* dispatch_static(int device, const uint32_t* ids, int t, int experts, int topk,
                            uint32_t* counts, uint32_t* offsets, uint32_t* perm, uint32_t* pos,
                            uint32_t* slot_token, int* active, cudaStream_t stream, int** status_word) {
    if (device < 0 || device >= MAX_DEVICES) return "device ordinal out of range";
    if (!ids || !counts || !offsets || !perm || !pos || !slot_token || !active)
        return "an input or output pointer is null";
    if (experts < 1 || experts > MAX_EXPERTS) return "between 1 and 256 experts";
    if (topk < 1 || topk > MAX_TOPK || topk > experts) return "between 1 and min(32, experts) experts per token";
    if (t < 1) return "empty batch";
    if (t > STATIC_MAX_TOKENS) return "more than 16384 tokens: beyond the built-in scratch array";
    // The context's device is made current on every call (and stays current): the launches
    // below and the symbol look-up both act on the current device.
    if (cudaSetDevice(device) != cudaSuccess) return "cudaSetDevice failed";
    StaticAddresses& sa = g_static_dev[device];
    uint32_t* block_hist = sa.block_hist.load(std::memory_order_acquire);
    int* status = sa.status.load(std::memory_order_acquire);
    if (!block_hist || !status) {
        // First call on this device (make it before any stream capture): look the
        // arrays' device addresses up, with this device current.
        void *p = nullptr, *q = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_block_hist) != cudaSuccess || !p)
            return "cudaGetSymbolAddress failed for the built-in scratch array";
        if (cudaGetSymbolAddress(&q, g_static_status) != cudaSuccess || !q)
            return "cudaGetSymbolAddress failed for the built-in status word";
        block_hist = static_cast<uint32_t*>(p);
        status = static_cast<int*>(q);
        sa.block_hist.store(block_hist, std::memory_order_release);
        sa.status.store(status, std::memory_order_release);
    }
    if (status_word) *status_word = status;
    const int blocks = (t + DISPATCH_THREADS - 1) / DISPATCH_THREADS;
    dispatch_count_kernel<<<blocks, DISPATCH_THREADS, 0, stream>>>(ids, t, experts, topk, block_hist, PeerWait{},
                                                                   status);
    dispatch_scan_kernel<<<1, DISPATCH_THREADS, 0, stream>>>(block_hist, blocks, experts, counts, offsets, active);
    dispatch_permute_kernel<<<blocks, DISPATCH_THREADS, 0, stream>>>(ids, t, experts, topk, block_hist, offsets,
                                                                     perm, pos, slot_token);
    return cudaGetLastError() == cudaSuccess ? nullptr : "a dispatch kernel failed to launch";
}

}  // namespace tc
