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

namespace tc {

namespace {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// f32::total_cmp as an integer key (larger key = later in total order).
__device__ __forceinline__ int total_key(float v) {
    int b = __float_as_int(v);
    return b ^ int(unsigned(b >> 31) >> 1);
}

// The hsum tree of src/kernels_x86.rs:33-38 over 8 values held by lanes
// j..j+7 of an aligned 8-lane group: (v0+v4, v1+v5, v2+v6, v3+v7) ->
// (s0+s2, s1+s3) -> s0+s1. Lane j%8==0 ends with the sum.
__device__ __forceinline__ float hsum8(float v, unsigned mask) {
    v = v + __shfl_down_sync(mask, v, 4, 8);
    v = v + __shfl_down_sync(mask, v, 2, 8);
    v = v + __shfl_down_sync(mask, v, 1, 8);
    return v;
}

// Sum of squares of a row in dot_f32's order, by one warp: lane L owns the
// elements L, L+32, ... (the four 8-lane accumulators of the main loop side by
// side); leftover groups of eight go to the first accumulator; then
// (acc0+acc1)+(acc2+acc3) lane-wise, the hsum tree, and the scalar tail.
__device__ __forceinline__ float sum_squares_avx_order(const float* xr, int n, int lane) {
    float acc = 0.0f;
    int i = 0;
#pragma unroll 8
    for (; i + 32 <= n; i += 32) {
        const float v = xr[i + lane];
        acc = fmaf(v, v, acc);
    }
    for (; i + 8 <= n; i += 8) {
        if (lane < 8) {
            const float v = xr[i + lane];
            acc = fmaf(v, v, acc);
        }
    }
    float s = acc + __shfl_down_sync(0xffffffffu, acc, 8);  // lanes 0-7: a0+a1; 16-23: a2+a3
    s = s + __shfl_down_sync(0xffffffffu, s, 16);           // lanes 0-7: the four summed
    s = hsum8(s, 0xffffffffu);
    float tail = 0.0f;
    for (int j = i; j < n; j++) tail = tail + xr[j] * xr[j];
    s = s + tail;
    return __shfl_sync(0xffffffffu, s, 0);
}

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
    // A CTA walks tokens blockIdx.x, blockIdx.x + gridDim.x, ...: one each as launched today.
    bool w_landed = true;
    for (int token = blockIdx.x; token < a.t; token += gridDim.x) {
    if (token != int(blockIdx.x)) __syncthreads();  // the previous token's row and logits are no longer read
    const float* xin = a.x + size_t(token) * hidden;
    for (int c = tid * 4; c < hidden; c += ROUTE_THREADS * 4)
        *reinterpret_cast<float4*>(xrow + c) = *reinterpret_cast<const float4*>(xin + c);
    __syncthreads();

    if (a.norm_w) {
        if (warp == 0) {
            const float ss = __fdiv_rn(sum_squares_avx_order(xrow, hidden, lane), float(hidden));
            if (lane == 0) s_inv = __fdiv_rn(1.0f, __fsqrt_rn(ss + a.eps));
        }
        __syncthreads();
        const float inv = s_inv;
        for (int c = tid; c < hidden; c += ROUTE_THREADS) xrow[c] = xrow[c] * inv * a.norm_w[c];
        __syncthreads();
    }

    // ---- logits. Four threads per expert, each holding four of the dot's
    // sixteen float lanes: thread q owns elements 16j+4q..16j+4q+3, so q = 0,1
    // hold the first 8-lane accumulator and q = 2,3 the second. The weights of
    // a whole batch of steps are requested before the chains run, so the loads
    // overlap instead of each waiting for the previous fma.
    constexpr int BATCH = 16;
    if (a.stage_router && token == int(blockIdx.x)) w_landed = mbar_wait_bounded(&s_wbar, 0);
    for (int e0 = 0; e0 < experts; e0 += ROUTE_THREADS / 4) {
        const int e = e0 + (tid >> 2), q = tid & 3;
        const bool valid = e < experts;
        const uint16_t* w = a.router + size_t(valid ? e : 0) * hidden + q * 4;
        const float* xr = xrow + q * 4;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (a.stage_router && w_landed) {
            const uint8_t* ws = wsm + size_t(valid ? e : 0) * wstride + q * 8;
#pragma unroll 8
            for (int c = 0; c < hidden; c += 16) {
                const uint2 wv = *reinterpret_cast<const uint2*>(ws + 2 * c);
                const float4 xv = *reinterpret_cast<const float4*>(xr + c);
                acc[0] = fmaf(bf16_lo(wv.x), xv.x, acc[0]);
                acc[1] = fmaf(bf16_hi(wv.x), xv.y, acc[1]);
                acc[2] = fmaf(bf16_lo(wv.y), xv.z, acc[2]);
                acc[3] = fmaf(bf16_hi(wv.y), xv.w, acc[3]);
            }
        } else
        for (int c0 = 0; c0 < hidden; c0 += 16 * BATCH) {
            uint2 wv[BATCH];
#pragma unroll
            for (int u = 0; u < BATCH; u++)
                wv[u] = c0 + 16 * u < hidden ? __ldg(reinterpret_cast<const uint2*>(w + c0 + 16 * u))
                                             : make_uint2(0u, 0u);
#pragma unroll
            for (int u = 0; u < BATCH; u++) {
                if (c0 + 16 * u < hidden) {
                    const float4 xv = *reinterpret_cast<const float4*>(xr + c0 + 16 * u);
                    acc[0] = fmaf(bf16_lo(wv[u].x), xv.x, acc[0]);
                    acc[1] = fmaf(bf16_hi(wv[u].x), xv.y, acc[1]);
                    acc[2] = fmaf(bf16_lo(wv[u].y), xv.z, acc[2]);
                    acc[3] = fmaf(bf16_hi(wv[u].y), xv.w, acc[3]);
                }
            }
        }
        // acc0 + acc1 lane-wise: lane l of the first accumulator (q = l/4) plus
        // lane l of the second (q = 2 + l/4): the thread two to the right.
        float v[4];
#pragma unroll
        for (int l = 0; l < 4; l++) v[l] = acc[l] + __shfl_xor_sync(0xffffffffu, acc[l], 2);
        // Now q = 0 holds v0..v3 and q = 1 holds v4..v7 (q = 2,3 hold copies).
        // hsum: (v0+v4, v1+v5, v2+v6, v3+v7) -> (s0+s2, s1+s3) -> sum.
        float sv[4];
#pragma unroll
        for (int l = 0; l < 4; l++) sv[l] = v[l] + __shfl_xor_sync(0xffffffffu, v[l], 1);
        float y = (sv[0] + sv[2]) + (sv[1] + sv[3]);
        if (valid && q == 0) {
            // The dot's scalar tail is an empty sum (hidden is a multiple of 32): hsum + 0.0.
            y = y + 0.0f;
            if (a.bias) y = y + a.bias[e];
            slog[e] = y;
            if (a.logits) a.logits[size_t(token) * experts + e] = y;
        }
    }
    __syncthreads();

    // ---- top-k and gates: warp 0. Lane l holds experts l, l+32, ...
    if (warp == 0) {
        constexpr int SLOTS = MAX_EXPERTS / 32;
        const int nslots = (experts + 31) >> 5;
        unsigned ukeys[SLOTS];  // order-preserving unsigned keys; 0 = not a candidate
        unsigned taken = 0;
#pragma unroll
        for (int s = 0; s < SLOTS; s++) {
            const int e = lane + 32 * s;
            // total_key is a signed order; flipping the sign bit makes it unsigned. +1 keeps 0 free
            // (the all-ones key, -NaN's neighbour in this order, cannot occur: it would be key 2^32).
            ukeys[s] = (s < nslots && e < experts) ? (unsigned(total_key(slog[e])) ^ 0x80000000u) : 0u;
            if (!(s < nslots && e < experts)) taken |= 1u << s;
        }
        int my_id = 0;
        float my_val = 0.0f;
        for (int j = 0; j < topk; j++) {
            unsigned best_key = 0;
            int best_idx = 0x7fffffff;
#pragma unroll
            for (int s = 0; s < SLOTS; s++) {
                if (s < nslots && !((taken >> s) & 1u)) {
                    if (best_idx == 0x7fffffff || ukeys[s] > best_key) {
                        best_key = ukeys[s];
                        best_idx = lane + 32 * s;
                    }
                }
            }
            // The largest key in the warp, then the lowest expert index among its holders.
            const bool have = best_idx != 0x7fffffff;
            const unsigned all_have = __ballot_sync(0xffffffffu, have);
            const unsigned wmax = __reduce_max_sync(0xffffffffu, have ? best_key : 0u);
            const bool tie = have && best_key == wmax;
            const unsigned widx = __reduce_min_sync(0xffffffffu, tie ? unsigned(best_idx) : 0xffffffffu);
            (void)all_have;
            const int win = int(widx);
            if ((win & 31) == lane) taken |= 1u << (win >> 5);
            if (lane == j) {
                my_id = win;
                my_val = slog[win];
            }
        }
        const float mx = __shfl_sync(0xffffffffu, my_val, 0);
        float ej = 0.0f;
        if (lane < topk) ej = float(exp(double(my_val - mx)));
        float sum = 0.0f;
        for (int j = 0; j < topk; j++) sum = sum + __shfl_sync(0xffffffffu, ej, j);
        if (lane < topk) {
            a.ids[size_t(token) * topk + lane] = uint32_t(my_id);
            a.gates[size_t(token) * topk + lane] = __fdiv_rn(ej, sum);
        }
    }

    // ---- 8-bit quantization of the row, a warp per 32-block.
    const int nb = hidden / QK;
    const int padded = (nb + SUPER - 1) / SUPER * SUPER;
    // Warps 1.. take the blocks while warp 0 is still ranking the logits above (the two do
    // not depend on each other); a single-warp launch would do both in turn.
    constexpr int QWARPS = ROUTE_THREADS / 32 - 1;
    for (int b = warp - 1; warp > 0 && b < padded; b += QWARPS) {
        if (b >= nb) {  // zero padding up to whole super-blocks
            if (lane == 0) {
                a.xs[size_t(token) * padded + b] = 0.0f;
                a.xsum[size_t(token) * padded + b] = 0.0f;
            }
            continue;
        }
        const float v = xrow[b * QK + lane];
        float amax = fabsf(v);
        // f32::max drops NaN operands, as fmaxf does.
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        float r = roundf(v * id);
        int q = (r != r) ? 0 : int(fminf(127.0f, fmaxf(-128.0f, r)));
        a.xq[size_t(token) * hidden + b * QK + lane] = int8_t(q);
        int qsum = q;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
        if (lane == 0) {
            a.xs[size_t(token) * padded + b] = d;
            a.xsum[size_t(token) * padded + b] = d * float(qsum);
        }
    }

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
    // One CTA per token at every batch size: measured faster than fewer CTAs that walk several
    // tokens each (which the kernel's token loop would allow), since short CTAs overlap better.
    launch_overlapped(route_kernel, dim3(t), dim3(ROUTE_THREADS), smem, stream, a);
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

