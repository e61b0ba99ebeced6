// Per-token front end of the MoE block, one CTA per token: (optional) RMSNorm,
// router GEMV, top-k, gating softmax, 8-bit quantization of the row, and - when
// the whole batch fits one CTA's dispatch - the token -> expert dispatch, run by
// whichever CTA finishes last.
//
// Reproduces, value for value:
//   rmsnorm        - src/kernels.rs:522-528 with dot_f32's AVX2 order
//                    (src/kernels_x86.rs:132-154), applied as src/model.rs:662-667;
//   router logits  - Matrix::matmul's bf16 arm (src/weights.rs:230-240) with
//                    the AVX2 dot bf16s (src/kernels_x86.rs:157-171): two
//                    8-lane fma accumulators over 16-element strides, summed
//                    lane-wise, then the fixed hsum tree (33-38);
//   top-k + gates  - route() (src/model.rs:448-457): order by total_cmp
//                    descending, ties to the lower expert, softmax over the k
//                    kept with max = the top score, sum taken in that order;
//   quantization   - quantize_q8 (src/kernels.rs:84-98) per 32-block, as
//                    quantize_input applies it per token (src/weights.rs:652-664).
// The softmax exponential is evaluated in double precision and rounded to
// float; the CPU path calls libm's expf. The two agree except where expf
// itself is not correctly rounded, hence the 1e-5 tolerance on gates.
#include "dispatch_common.cuh"
#include "experts_common.cuh"
#include "route_common.cuh"

namespace tc {

namespace {

constexpr size_t ROUTE_SMEM_LIMIT = 200 * 1024;
constexpr int ROUTE_THREADS = DISPATCH_THREADS;  // the last CTA runs the dispatch with the same threads

struct RouteArgs {
    const uint16_t* router;
    const float* bias;
    const float* x;        // [t, hidden]: the normed input, or the residual stream when norm_w is set
    const float* norm_w;   // RMSNorm weight, or null when x is already normed
    float eps;
    int t, hidden, experts, topk;
    float* logits;
    uint32_t* ids;
    float* gates;
    int8_t* xq;
    float* xs;
    float* xsum;
    // dispatch outputs, used when fused
    int fuse_dispatch;
    int stage_router;      // the router matrix fits in shared memory beside the row: stage it with bulk copies
    int* ticket;
    int* status;
    uint32_t *counts, *offsets, *perm, *pos, *slot_token;
    int* active;
    PeerPlan scatter;      // ranks > 0: the last CTA sends the rows to every rank instead of dispatching
};

__global__ void __launch_bounds__(ROUTE_THREADS) route_kernel(const RouteArgs a) {
    extern __shared__ __align__(128) float smem[];
    float* xrow = smem;                 // [hidden] the block's input row (after the norm)
    float* slog = smem + a.hidden;      // [experts]
    __shared__ float s_inv;
    __shared__ int s_last;
    __shared__ __align__(8) uint64_t s_wbar;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hidden = a.hidden, experts = a.experts, topk = a.topk;
    grid_launch_dependents();
    // The router matrix, one bulk copy per row, into rows padded by 32 bytes (so the four-thread
    // groups of a half-warp read distinct banks). Issued first: it lands while the row is normed.
    const int wstride = 2 * hidden + 32;
    uint8_t* wsm = reinterpret_cast<uint8_t*>(smem) + (size_t(hidden + experts) * 4 + 127) / 128 * 128;
    if (a.stage_router) {
        if (tid == 0) {
            mbar_init(&s_wbar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(&s_wbar, uint32_t(experts) * 2u * uint32_t(hidden));
        }
        __syncthreads();
        if (warp == 0)
            for (int e = lane; e < experts; e += 32)
                bulk_copy(wsm + size_t(e) * wstride, a.router + size_t(e) * hidden, 2 * hidden, &s_wbar);
    }
    // The router matrix is a constant: it streams in while the kernel in front of this
    // one (the previous block's combine) finishes. Everything below reads its output.
    grid_dependency_wait();
    // A CTA walks tokens blockIdx.x, blockIdx.x + gridDim.x, ...: one each for batches of up to a few
    // CTAs per SM, several for prefill-size batches (the staged router matrix is then read once per
    // CTA instead of once per token). The next token's row is requested before this one is worked on.
    bool w_landed = true;
    constexpr int ROW_VEC = 4;  // float4 per thread held ahead: rows of up to 4096 floats
    float4 ahead[ROW_VEC];
    auto request_row = [&](int token) {
#pragma unroll
        for (int i = 0; i < ROW_VEC; i++) {
            const int c = (tid + i * ROUTE_THREADS) * 4;
            if (token < a.t && c < hidden)
                ahead[i] = *reinterpret_cast<const float4*>(a.x + size_t(token) * hidden + c);
        }
    };
    const bool rows_ahead = hidden <= ROW_VEC * ROUTE_THREADS * 4;
    if (rows_ahead) request_row(blockIdx.x);
    for (int token = blockIdx.x; token < a.t; token += gridDim.x) {
        if (token != int(blockIdx.x)) __syncthreads();  // the previous token's row and logits are no longer read
        if (rows_ahead) {
#pragma unroll
            for (int i = 0; i < ROW_VEC; i++) {
                const int c = (tid + i * ROUTE_THREADS) * 4;
                if (c < hidden) *reinterpret_cast<float4*>(xrow + c) = ahead[i];
            }
            request_row(token + gridDim.x);
        } else {
            const float* xin = a.x + size_t(token) * hidden;
            for (int c = tid * 4; c < hidden; c += ROUTE_THREADS * 4)
                *reinterpret_cast<float4*>(xrow + c) = *reinterpret_cast<const float4*>(xin + c);
        }
        __syncthreads();
        if (a.norm_w) route_norm_row(xrow, hidden, a.norm_w, a.eps, &s_inv, tid, ROUTE_THREADS);

        if (a.stage_router && token == int(blockIdx.x)) w_landed = mbar_wait_bounded(&s_wbar, 0);
        route_logits(a.router, a.stage_router && w_landed ? wsm : nullptr, wstride, xrow, a.bias, hidden, 0, experts,
                     slog, a.logits ? a.logits + size_t(token) * experts : nullptr, tid, ROUTE_THREADS);
        __syncthreads();

        // Warp 0 ranks the logits while warps 1.. quantize the row (the two do not depend on each other).
        if (warp == 0)
            route_topk_gates(slog, experts, topk, a.ids + size_t(token) * topk, a.gates + size_t(token) * topk, lane);
        const int padded = (hidden / QK + SUPER - 1) / SUPER * SUPER;
        route_quantize_row(xrow, hidden, a.xq + size_t(token) * hidden, a.xs + size_t(token) * padded,
                           a.xsum + size_t(token) * padded, warp, lane, 1, ROUTE_THREADS / 32 - 1);
    }  // tokens of this CTA

    // ---- the dispatch, by the last CTA to get here (batches of up to one CTA's worth of tokens).
    if (a.stage_router && !w_landed) {
        // The staged copy did not arrive within the spin limit (the logits came from
        // global memory instead). Report it, and give the copy a last bounded chance to
        // land before this shared memory is reused or released.
        if (tid == 0) atomicExch(a.status, ERR_COPY_WAIT_TIMEOUT);
        mbar_wait_bounded(&s_wbar, 0);
    }
    if (a.fuse_dispatch) {
        __threadfence();  // this CTA's ids are visible before its ticket
        __syncthreads();
        if (tid == 0) s_last = atomicAdd(a.ticket, 1) == a.t - 1;
        __syncthreads();
        if (s_last) {
            __threadfence();
            if (a.scatter.ranks) {
                // Expert parallelism over peer memory: the dispatch runs over every rank's
                // tokens, after this CTA has stored this rank's rows into every window.
                __shared__ uint32_t s_epoch;
                peer_scatter_signal(a.scatter, &s_epoch);
            } else {
                DispatchSmem& sm = *reinterpret_cast<DispatchSmem*>(smem);
                dispatch_small_body(sm, a.ids, a.t, experts, topk, a.counts, a.offsets, a.perm, a.pos,
                                    a.slot_token, a.active, a.status);
            }
            if (tid == 0) *a.ticket = 0;  // ready for the next launch on this stream
        }
    }
}

// One warp per row.
__global__ void rmsnorm_kernel(const float* x, const float* __restrict__ w, float eps, int t, int n,
                               float* out) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= t) return;
    const float* xr = x + size_t(row) * n;
    const float ss = __fdiv_rn(sum_squares_avx_order(xr, n, lane), float(n));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(ss + eps));
    float* o = out + size_t(row) * n;
#pragma unroll 8
    for (int c = lane; c < n; c += 32) o[c] = xr[c] * inv * w[c];
}

}  // namespace

void init_kernels_route() {
    cudaFuncSetAttribute(route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ROUTE_SMEM_LIMIT));
}

int launch_route(const MoeDims& d, const uint16_t* router, const float* bias, const float* x,
                 const float* norm_w, float eps, int t, Workspace& ws, cudaStream_t stream) {
    RouteArgs a{};
    a.router = router;
    a.bias = bias;
    a.x = x;
    a.norm_w = norm_w;
    a.eps = eps;
    a.t = t;
    a.hidden = d.hidden;
    a.experts = d.experts;
    a.topk = d.topk;
    a.logits = ws.logits;
    a.ids = ws.ids;
    a.gates = ws.gates;
    a.xq = ws.xq;
    a.xs = ws.xs;
    a.xsum = ws.xsum;
    a.fuse_dispatch = t <= DISPATCH_THREADS;
    a.ticket = ws.ticket;
    a.status = ws.status;
    a.counts = ws.counts;
    a.offsets = ws.offsets;
    a.perm = ws.perm;
    a.pos = ws.pos;
    a.slot_token = ws.slot_token;
    a.active = ws.active;
    if (a.fuse_dispatch) a.scatter = ws.route_scatter;
    size_t smem = (size_t(d.hidden + d.experts) * sizeof(float) + 127) / 128 * 128;
    const size_t staged = smem + size_t(d.experts) * (2 * size_t(d.hidden) + 32);
    a.stage_router = staged <= ROUTE_SMEM_LIMIT;
    if (a.stage_router) smem = staged;
    if (smem < sizeof(DispatchSmem)) smem = sizeof(DispatchSmem);
    // One CTA per token while that is at most three CTAs per SM (short CTAs overlap best);
    // beyond that a fixed grid whose CTAs walk several tokens each, so that a prefill-size
    // batch stages the router matrix a few hundred times instead of once per token.
    const int sms = ws.sms > 0 ? ws.sms : 148;
    const int grid = a.fuse_dispatch || t <= 3 * sms ? t : 3 * sms;
    launch_overlapped(route_kernel, dim3(grid), dim3(ROUTE_THREADS), smem, stream, a);
    int launched = 1;
    if (!a.fuse_dispatch) launched += launch_dispatch(d, t, ws, stream);
    return launched;
}

int launch_rmsnorm(const float* x, const float* w, float eps, int t, int n, float* out,
                   cudaStream_t stream) {
    const int warps = 4;
    rmsnorm_kernel<<<(t + warps - 1) / warps, warps * 32, 0, stream>>>(x, w, eps, t, n, out);
    return 1;
}

}  // namespace tc

