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
    int* ticket;
    uint32_t *counts, *offsets, *perm, *pos, *slot_token;
    int* active;
};

__global__ void __launch_bounds__(ROUTE_THREADS) route_kernel(const RouteArgs a) {
    extern __shared__ __align__(16) float smem[];
    float* xrow = smem;                 // [hidden] the block's input row (after the norm)
    float* slog = smem + a.hidden;      // [experts]
    __shared__ float s_inv;
    __shared__ int s_last;
    const int token = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hidden = a.hidden, experts = a.experts, topk = a.topk;
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

    // ---- logits. Two threads per expert: one holds the dot's first 8-lane
    // accumulator (elements 16j..16j+7), the other the second (16j+8..16j+15).
    for (int e0 = 0; e0 < experts; e0 += ROUTE_THREADS / 2) {
        const int e = e0 + (tid >> 1), half = tid & 1;
        const bool valid = e < experts;
        const uint16_t* w = a.router + size_t(valid ? e : 0) * hidden + half * 8;
        const float* xr = xrow + half * 8;
        float acc[8];
#pragma unroll
        for (int l = 0; l < 8; l++) acc[l] = 0.0f;
#pragma unroll 4
        for (int c = 0; c + 16 <= hidden; c += 16) {
            const uint4 wv = *reinterpret_cast<const uint4*>(w + c);
            const float4 x0 = *reinterpret_cast<const float4*>(xr + c);
            const float4 x1 = *reinterpret_cast<const float4*>(xr + c + 4);
            acc[0] = fmaf(bf16_lo(wv.x), x0.x, acc[0]);
            acc[1] = fmaf(bf16_hi(wv.x), x0.y, acc[1]);
            acc[2] = fmaf(bf16_lo(wv.y), x0.z, acc[2]);
            acc[3] = fmaf(bf16_hi(wv.y), x0.w, acc[3]);
            acc[4] = fmaf(bf16_lo(wv.z), x1.x, acc[4]);
            acc[5] = fmaf(bf16_hi(wv.z), x1.y, acc[5]);
            acc[6] = fmaf(bf16_lo(wv.w), x1.z, acc[6]);
            acc[7] = fmaf(bf16_hi(wv.w), x1.w, acc[7]);
        }
        // acc0 + acc1 lane-wise, then the hsum tree: (v0+v4, ...) -> (s0+s2, s1+s3) -> sum.
        float v[8];
#pragma unroll
        for (int l = 0; l < 8; l++) v[l] = acc[l] + __shfl_xor_sync(0xffffffffu, acc[l], 1);
        const float s0 = v[0] + v[4], s1 = v[1] + v[5], s2 = v[2] + v[6], s3 = v[3] + v[7];
        float y = (s0 + s2) + (s1 + s3);
        if (valid && half == 0) {
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
        int keys[SLOTS];
        unsigned taken = 0;
#pragma unroll
        for (int s = 0; s < SLOTS; s++) {
            int e = lane + 32 * s;
            keys[s] = e < experts ? total_key(slog[e]) : 0;
            if (e >= experts) taken |= 1u << s;
        }
        int my_id = 0;
        float my_val = 0.0f;
        for (int j = 0; j < topk; j++) {
            int best_key = 0, best_idx = 0x7fffffff;
#pragma unroll
            for (int s = 0; s < SLOTS; s++) {
                if (!((taken >> s) & 1u)) {
                    int idx = lane + 32 * s;
                    if (best_idx == 0x7fffffff || keys[s] > best_key) {
                        best_key = keys[s];
                        best_idx = idx;
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                int ok = __shfl_xor_sync(0xffffffffu, best_key, o);
                int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
                bool other_better = (oi != 0x7fffffff) &&
                                    (best_idx == 0x7fffffff || ok > best_key ||
                                     (ok == best_key && oi < best_idx));
                if (other_better) {
                    best_key = ok;
                    best_idx = oi;
                }
            }
            if ((best_idx & 31) == lane) taken |= 1u << (best_idx >> 5);
            if (lane == j) {
                my_id = best_idx;
                my_val = slog[best_idx];
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
    for (int b = warp; b < padded; b += ROUTE_THREADS / 32) {
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

    // ---- the dispatch, by the last CTA to get here (batches of up to one CTA's worth of tokens).
    if (a.fuse_dispatch) {
        __threadfence();  // this CTA's ids are visible before its ticket
        __syncthreads();
        if (tid == 0) s_last = atomicAdd(a.ticket, 1) == a.t - 1;
        __syncthreads();
        if (s_last) {
            __threadfence();
            DispatchSmem& sm = *reinterpret_cast<DispatchSmem*>(smem);
            dispatch_small_body(sm, a.ids, a.t, experts, topk, a.counts, a.offsets, a.perm, a.pos,
                                a.slot_token, a.active);
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
    a.counts = ws.counts;
    a.offsets = ws.offsets;
    a.perm = ws.perm;
    a.pos = ws.pos;
    a.slot_token = ws.slot_token;
    a.active = ws.active;
    size_t smem = size_t(d.hidden + d.experts) * sizeof(float);
    if (smem < sizeof(DispatchSmem)) smem = sizeof(DispatchSmem);
    route_kernel<<<t, ROUTE_THREADS, smem, stream>>>(a);
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
