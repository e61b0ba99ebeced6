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
#include <algorithm>

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

// Prefill-size batches: a CTA takes ROUTE_TILE tokens at a time (walking tiles blockIdx.x,
// blockIdx.x + gridDim.x, ...), so that every warp has work in every step: a warp per token for
// the norm, the ranking and the quantization, four threads per (token, expert) pair for the
// logits, with the router matrix staged once per CTA. Same arithmetic per token as route_kernel.
constexpr int ROUTE_TILE = 8;

// Shared memory of the tile kernel before the staged router matrix: padded rows, logits, norm weight.
__host__ __device__ inline size_t route_tile_bytes(int hidden, int experts) {
    return (size_t(ROUTE_TILE) * (hidden / QK * ROW_PAD_BLOCK + experts) * 4 + size_t(hidden) * 4 + 127) / 128 * 128;
}

__global__ void __launch_bounds__(ROUTE_THREADS) route_tile_kernel(const RouteArgs a) {
    extern __shared__ __align__(128) float smem[];
    const int hidden = a.hidden, experts = a.experts, topk = a.topk;
    const int rstride = hidden / QK * ROW_PAD_BLOCK;  // floats per padded row
    float* xrows = smem;                              // [ROUTE_TILE] padded rows
    float* slog = xrows + ROUTE_TILE * rstride;       // [ROUTE_TILE][experts]
    float* snw = slog + ROUTE_TILE * experts;         // [hidden] the norm's weight
    __shared__ __align__(8) uint64_t s_wbar;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    grid_launch_dependents();
    const int wstride = 2 * hidden + 32;
    uint8_t* wsm = reinterpret_cast<uint8_t*>(smem) + route_tile_bytes(hidden, experts);
    if (a.norm_w)
        for (int c = tid; c < hidden; c += ROUTE_THREADS) snw[c] = a.norm_w[c];  // (a constant: before the wait)
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
    grid_dependency_wait();
    bool w_landed = true, w_waited = false;
    const int padded = (hidden / QK + SUPER - 1) / SUPER * SUPER;
    const int tiles = (a.t + ROUTE_TILE - 1) / ROUTE_TILE;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int t0 = tile * ROUTE_TILE, nt = min(ROUTE_TILE, a.t - t0);
        __syncthreads();  // the previous tile's rows and logits are no longer read
        const int vec_per_row = hidden / 4;
        for (int k = 0; k < nt; k++) {
            const float4* src = reinterpret_cast<const float4*>(a.x + size_t(t0 + k) * hidden);
            for (int i = tid; i < vec_per_row; i += ROUTE_THREADS)
                *reinterpret_cast<float4*>(xrows + k * rstride + padded_at(4 * i)) = src[i];
        }
        __syncthreads();
        if (a.norm_w && warp < nt) {  // a warp per token
            float* xr = xrows + warp * rstride;
            const float ss = __fdiv_rn(sum_squares_padded_row(xr, hidden, lane), float(hidden));
            const float inv = __fdiv_rn(1.0f, __fsqrt_rn(ss + a.eps));
            __syncwarp();
#pragma unroll 4
            for (int k = 0; k < hidden / QK; k++)
                xr[k * ROW_PAD_BLOCK + lane] = xr[k * ROW_PAD_BLOCK + lane] * inv * snw[k * QK + lane];
        }
        if (a.stage_router && !w_waited) {
            w_landed = mbar_wait_bounded(&s_wbar, 0);
            w_waited = true;
        }
        __syncthreads();
        // Logits: four threads per (expert, group of ROUTE_TG tokens): the expert's row is read from
        // shared memory once for the group's tokens (the row reads, distinct per expert, are what
        // the shared-memory pipe is busy with; the tokens' reads are broadcasts). Each (token,
        // expert) logit keeps its own accumulators: the same sums as one token at a time.
        constexpr int ROUTE_TG = 4;
        const int groups = (nt + ROUTE_TG - 1) / ROUTE_TG, tasks = groups * experts;
        for (int p0 = 0; p0 < tasks; p0 += ROUTE_THREADS / 4) {
            const int p = p0 + (tid >> 2), q = tid & 3;
            const bool valid = p < tasks;
            const int grp = valid ? p / experts : 0, e = valid ? p - grp * experts : 0;
            float acc[ROUTE_TG][4];
#pragma unroll
            for (int k = 0; k < ROUTE_TG; k++) acc[k][0] = acc[k][1] = acc[k][2] = acc[k][3] = 0.0f;
            if (p0 + ((tid >> 5) << 3) < tasks) {  // (a warp without work skips the loop)
                const bool staged = a.stage_router && w_landed;
                const uint8_t* ws = wsm + size_t(e) * wstride + q * 8;
                const uint16_t* wg = a.router + size_t(e) * hidden + q * 4;
                const float* xr = xrows + size_t(grp * ROUTE_TG) * rstride + q * 4;
#pragma unroll 2
                for (int c = 0; c < hidden; c += 16) {
                    const uint2 wv = staged ? *reinterpret_cast<const uint2*>(ws + 2 * c)
                                            : __ldg(reinterpret_cast<const uint2*>(wg + c));
                    const float w0 = bf16_lo(wv.x), w1 = bf16_hi(wv.x), w2 = bf16_lo(wv.y), w3 = bf16_hi(wv.y);
#pragma unroll
                    for (int k = 0; k < ROUTE_TG; k++) {
                        if (grp * ROUTE_TG + k < nt) {
                            const float4 xv = *reinterpret_cast<const float4*>(xr + k * rstride + padded_at(c));
                            acc[k][0] = fmaf(w0, xv.x, acc[k][0]);
                            acc[k][1] = fmaf(w1, xv.y, acc[k][1]);
                            acc[k][2] = fmaf(w2, xv.z, acc[k][2]);
                            acc[k][3] = fmaf(w3, xv.w, acc[k][3]);
                        }
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < ROUTE_TG; k++) {
                // As route_dot_quad: the two 8-lane accumulators added lane-wise, then the hsum tree.
                float v[4], sv[4];
#pragma unroll
                for (int l = 0; l < 4; l++) v[l] = acc[k][l] + __shfl_xor_sync(0xffffffffu, acc[k][l], 2);
#pragma unroll
                for (int l = 0; l < 4; l++) sv[l] = v[l] + __shfl_xor_sync(0xffffffffu, v[l], 1);
                float y = (sv[0] + sv[2]) + (sv[1] + sv[3]);
                y = y + 0.0f;  // the dot's scalar tail is an empty sum
                const int token = grp * ROUTE_TG + k;
                if (valid && q == 0 && token < nt) {
                    if (a.bias) y = y + a.bias[e];
                    slog[token * experts + e] = y;
                    if (a.logits) a.logits[size_t(t0 + token) * experts + e] = y;
                }
            }
        }
        __syncthreads();
        if (warp < nt) {  // a warp per token: ranking and gates, then the row's 8-bit blocks
            const size_t token = size_t(t0 + warp);
            route_topk_gates(slog + warp * experts, experts, topk, a.ids + token * topk, a.gates + token * topk, lane);
            route_quantize_padded_row(xrows + warp * rstride, hidden, a.xq + token * hidden, a.xs + token * padded,
                                      a.xsum + token * padded, lane);
        }
    }
    if (a.stage_router && (!w_waited || !w_landed)) {
        // Not waited for (a CTA without tiles) or not arrived in time: a last bounded chance for the
        // copy to land before this shared memory is released; a late copy is reported.
        const bool late = w_waited && !w_landed;
        mbar_wait_bounded(&s_wbar, 0);
        if (late && tid == 0) atomicExch(a.status, ERR_COPY_WAIT_TIMEOUT);
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
    cudaFuncSetAttribute(route_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ROUTE_SMEM_LIMIT));
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
    const int sms = ws.sms > 0 ? ws.sms : 148;
    if (a.fuse_dispatch) {
        // Up to one CTA's worth of tokens: a CTA per token; the last one to finish runs the dispatch.
        launch_overlapped(route_kernel, dim3(t), dim3(ROUTE_THREADS), smem, stream, a);
    } else {
        // Larger batches: CTAs that walk tiles of ROUTE_TILE tokens with every warp busy, as many as
        // stay resident (the staged router matrix is then read a few hundred times, not once per token).
        size_t tsmem = route_tile_bytes(d.hidden, d.experts);
        const size_t tstaged = tsmem + size_t(d.experts) * (2 * size_t(d.hidden) + 32);
        a.stage_router = tstaged <= ROUTE_SMEM_LIMIT;
        if (a.stage_router) tsmem = tstaged;
        const int per_sm = int(std::max<size_t>(1, std::min<size_t>(4, (220 * 1024) / (tsmem + 1024))));
        const int tiles = (t + ROUTE_TILE - 1) / ROUTE_TILE;
        launch_overlapped(route_tile_kernel, dim3(std::min(tiles, per_sm * sms)), dim3(ROUTE_THREADS), tsmem, stream, a);
    }
    int launched = 1;
    // (Expert parallel over peer windows: the dispatch runs later, over every rank's tokens.)
    if (!a.fuse_dispatch && ws.route_scatter.ranks == 0) launched += launch_dispatch(d, t, ws, stream);
    return launched;
}

int launch_rmsnorm(const float* x, const float* w, float eps, int t, int n, float* out,
                   cudaStream_t stream) {
    const int warps = 4;
    rmsnorm_kernel<<<(t + warps - 1) / warps, warps * 32, 0, stream>>>(x, w, eps, t, n, out);
    return 1;
}

}  // namespace tc

