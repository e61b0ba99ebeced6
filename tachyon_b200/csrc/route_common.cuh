// The per-token front end of the MoE block as device functions, shared by the
// stand-alone router kernel (route.cu) and the one-kernel decode block
// (moe_decode.cu): RMSNorm, router logits, top-k with gating softmax, and the
// 8-bit quantization of the token's row.
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
// The softmax exponential is evaluated in double precision (a short polynomial of
// this file, accurate to about 1e-16) and rounded to float; the CPU path calls libm's
// expf. The two agree except where expf itself is not correctly rounded, hence the
// 1e-5 tolerance on gates.
#pragma once

#include "common.cuh"

namespace tc {

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

// xrow[0..hidden) (shared memory, already loaded) becomes rmsnorm(xrow) * norm_w. Called
// by every thread of the CTA; s_inv is one shared float. Ends with a CTA barrier.
__device__ __forceinline__ void route_norm_row(float* xrow, int hidden, const float* norm_w, float eps,
                                               float* s_inv, int tid, int nthreads) {
    if ((tid >> 5) == 0) {
        const float ss = __fdiv_rn(sum_squares_avx_order(xrow, hidden, tid & 31), float(hidden));
        if (tid == 0) *s_inv = __fdiv_rn(1.0f, __fsqrt_rn(ss + eps));
    }
    __syncthreads();
    const float inv = *s_inv;
    for (int c = tid; c < hidden; c += nthreads) xrow[c] = xrow[c] * inv * norm_w[c];
    __syncthreads();
}

// One router logit: dot(bf16 row of expert e, xrow) by FOUR threads (q = 0..3 of an aligned
// quad), each holding four of the dot's sixteen float lanes: thread q owns elements
// 16j+4q..16j+4q+3, so q = 0,1 hold the first 8-lane accumulator of the AVX2 dot and q = 2,3
// the second. `staged`: the router matrix in shared memory with rows `wstride` bytes apart (row
// index e_staged), or null to read expert e's row from global memory (a whole batch of steps
// is requested before the chains run, so the loads overlap instead of each waiting for the
// previous fma). A warp none of whose quads has work passes busy = false and skips the loop (it
// would only take shared-memory bandwidth from the warps that have work) but still takes part
// in the shuffles. The value is complete in every thread of the quad.
__device__ __forceinline__ float route_dot_quad(const uint16_t* router, const uint8_t* staged, int wstride,
                                                const float* xrow, int hidden, int e, int q, bool busy,
                                                int e_staged = -1) {
    constexpr int BATCH = 8;
    const uint16_t* w = router + size_t(e) * hidden + q * 4;
    const float* xr = xrow + q * 4;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (!busy) {
    } else if (staged) {
        const uint8_t* ws = staged + size_t(e_staged >= 0 ? e_staged : e) * wstride + q * 8;
#pragma unroll 8
        for (int c = 0; c < hidden; c += 16) {
            const uint2 wv = *reinterpret_cast<const uint2*>(ws + 2 * c);
            const float4 xv = *reinterpret_cast<const float4*>(xr + c);
            acc[0] = fmaf(bf16_lo(wv.x), xv.x, acc[0]);
            acc[1] = fmaf(bf16_hi(wv.x), xv.y, acc[1]);
            acc[2] = fmaf(bf16_lo(wv.y), xv.z, acc[2]);
            acc[3] = fmaf(bf16_hi(wv.y), xv.w, acc[3]);
        }
    } else {
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
    const float y = (sv[0] + sv[2]) + (sv[1] + sv[3]);
    // The dot's scalar tail is an empty sum (hidden is a multiple of 32): hsum + 0.0.
    return y + 0.0f;
}

// Router logits of one token, experts e_lo..e_hi-1, into slog[e] (and, when given, a global
// row), by every thread of the CTA, four per expert. `staged`: rows e_lo.. of the router
// matrix in shared memory, or null. The caller puts a CTA barrier after it.
__device__ __forceinline__ void route_logits(const uint16_t* router, const uint8_t* staged, int wstride,
                                             const float* xrow, const float* bias, int hidden, int e_lo, int e_hi,
                                             float* slog, float* logits_row, int tid, int nthreads) {
    for (int e0 = e_lo; e0 < e_hi; e0 += nthreads / 4) {
        const int e = e0 + (tid >> 2);
        const bool valid = e < e_hi;
        float y = route_dot_quad(router, staged, wstride, xrow, hidden, valid ? e : e_lo, tid & 3,
                                 e0 + ((tid >> 5) << 3) < e_hi, valid ? e - e_lo : 0);
        if (valid && (tid & 3) == 0) {
            if (bias) y = y + bias[e];
            slog[e] = y;
            if (logits_row) logits_row[e] = y;
        }
    }
}

// exp(x) for x <= 0 in double precision, rounded to float: what the gating softmax needs
// (its arguments are score - max score). Argument reduction by ln 2 in two parts, a
// degree-13 Taylor polynomial on |r| <= ln(2)/2 (truncation error below 1e-17), and the
// power of two put into the exponent. Results below the smallest float flush to zero as
// the conversion would make them.
__device__ __forceinline__ float exp_nonpositive_f64(float xf) {
    if (xf != xf) return xf;
    if (xf < -104.0f) return 0.0f;
    const double x = double(xf);
    const double n = rint(x * 1.4426950408889634);
    double r = fma(-n, 6.93147180369123816490e-01, x);
    r = fma(-n, 1.90821492927058770002e-10, r);
    double p = 1.0 / 6227020800.0;
    p = fma(p, r, 1.0 / 479001600.0);
    p = fma(p, r, 1.0 / 39916800.0);
    p = fma(p, r, 1.0 / 3628800.0);
    p = fma(p, r, 1.0 / 362880.0);
    p = fma(p, r, 1.0 / 40320.0);
    p = fma(p, r, 1.0 / 5040.0);
    p = fma(p, r, 1.0 / 720.0);
    p = fma(p, r, 1.0 / 120.0);
    p = fma(p, r, 1.0 / 24.0);
    p = fma(p, r, 1.0 / 6.0);
    p = fma(p, r, 0.5);
    p = fma(p, r, 1.0);
    p = fma(p, r, 1.0);
    const long long bits = __double_as_longlong(p) + (static_cast<long long>(n) << 52);
    return float(__longlong_as_double(bits));
}

// Top-k and gates of one token, by ONE warp: lane l holds experts l, l+32, ...; after the
// k rounds lane j < k holds the j-th pick and writes ids_row[j] / gates_row[j].
__device__ __forceinline__ void route_topk_gates(const float* slog, int experts, int topk, uint32_t* ids_row,
                                                 float* gates_row, int lane) {
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
    if (experts <= 32) {
        // One expert per lane: each lane counts the experts that come before its own in the
        // order (larger key first, lower index first among equals), all 32 comparisons
        // independent of one another; the lane of rank j is the j-th pick. Same picks as the
        // rounds below, without their chain of dependent steps.
        const unsigned key = ukeys[0];
        int rank = 0;
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const unsigned kj = __shfl_sync(0xffffffffu, key, j);
            rank += (j < experts && (kj > key || (kj == key && j < lane))) ? 1 : 0;
        }
        if (lane >= experts) rank = 0x7fffffff;
        for (int j = 0; j < topk; j++) {
            const int win = __ffs(__ballot_sync(0xffffffffu, rank == j)) - 1;
            if (lane == j) {
                my_id = win;
                my_val = slog[win];
            }
        }
    } else
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
        const unsigned wmax = __reduce_max_sync(0xffffffffu, have ? best_key : 0u);
        const bool tie = have && best_key == wmax;
        const unsigned widx = __reduce_min_sync(0xffffffffu, tie ? unsigned(best_idx) : 0xffffffffu);
        const int win = int(widx);
        if ((win & 31) == lane) taken |= 1u << (win >> 5);
        if (lane == j) {
            my_id = win;
            my_val = slog[win];
        }
    }
    const float mx = __shfl_sync(0xffffffffu, my_val, 0);
    float ej = 0.0f;
    if (lane < topk) ej = exp_nonpositive_f64(my_val - mx);
    float sum = 0.0f;
    for (int j = 0; j < topk; j++) sum = sum + __shfl_sync(0xffffffffu, ej, j);
    if (lane < topk) {
        ids_row[lane] = uint32_t(my_id);
        gates_row[lane] = __fdiv_rn(ej, sum);
    }
}

// 8-bit quantization of one token's row, a warp per 32-block: warps first_warp ..
// first_warp + nq - 1 of the CTA take the blocks (and the zero padding up to whole
// super-blocks of the scale rows) in turn.
__device__ __forceinline__ void route_quantize_row(const float* xrow, int hidden, int8_t* xq_row, float* xs_row,
                                                   float* xsum_row, int warp, int lane, int first_warp, int nq) {
    const int nb = hidden / QK;
    const int padded = (nb + SUPER - 1) / SUPER * SUPER;
    for (int b = warp - first_warp; warp >= first_warp && b < padded; b += nq) {
        if (b >= nb) {
            if (lane == 0) {
                xs_row[b] = 0.0f;
                xsum_row[b] = 0.0f;
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
        xq_row[b * QK + lane] = int8_t(q);
        int qsum = q;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
        if (lane == 0) {
            xs_row[b] = d;
            xsum_row[b] = d * float(qsum);
        }
    }
}

// Rows kept in shared memory with four floats of padding after every 32-element block
// (element c at c + 4 * (c / 32)): lanes that each walk their own block then spread over the
// banks instead of all hitting the same one, and 16-byte vector accesses stay aligned.
constexpr int ROW_PAD_BLOCK = QK + 4;
__device__ __forceinline__ int padded_at(int c) { return c + ((c >> 5) << 2); }

// sum_squares_avx_order over such a padded row (n a multiple of 32): lane L owns elements
// L, L + 32, ... as there; the same additions in the same order.
__device__ __forceinline__ float sum_squares_padded_row(const float* xr, int n, int lane) {
    float acc = 0.0f;
#pragma unroll 8
    for (int k = 0; k < n / QK; k++) {
        const float v = xr[k * ROW_PAD_BLOCK + lane];
        acc = fmaf(v, v, acc);
    }
    float s = acc + __shfl_down_sync(0xffffffffu, acc, 8);
    s = s + __shfl_down_sync(0xffffffffu, s, 16);
    s = hsum8(s, 0xffffffffu);
    s = s + 0.0f;  // the scalar tail is an empty sum
    return __shfl_sync(0xffffffffu, s, 0);
}

// The row quantization by ONE warp with a lane per 32-block (32 blocks at a time) over a
// padded row: each lane runs its block's 32 elements itself, so the warp spends a few
// hundred instructions on the row instead of a shuffle reduction per block. Same values:
// the maximum does not depend on the order, the sum of the quants is an integer.
__device__ __forceinline__ void route_quantize_padded_row(const float* xrow, int hidden, int8_t* xq_row, float* xs_row,
                                                          float* xsum_row, int lane) {
    const int nb = hidden / QK;
    const int padded = (nb + SUPER - 1) / SUPER * SUPER;
    for (int b0 = 0; b0 < padded; b0 += 32) {
        const int b = b0 + lane;
        if (b >= padded) continue;
        if (b >= nb) {  // zero padding up to whole super-blocks
            xs_row[b] = 0.0f;
            xsum_row[b] = 0.0f;
            continue;
        }
        const float4* xb = reinterpret_cast<const float4*>(xrow + b * ROW_PAD_BLOCK);
        float4 v[QK / 4];
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < QK / 4; i++) {
            v[i] = xb[i];
            amax = fmaxf(fmaxf(fmaxf(fmaxf(amax, fabsf(v[i].x)), fabsf(v[i].y)), fabsf(v[i].z)), fabsf(v[i].w));
        }
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        auto q8 = [&](float x) {
            const float r = roundf(x * id);
            return (r != r) ? 0 : int(fminf(127.0f, fmaxf(-128.0f, r)));
        };
        int qsum = 0;
        uint32_t words[QK / 4];
#pragma unroll
        for (int i = 0; i < QK / 4; i++) {
            const int q0 = q8(v[i].x), q1 = q8(v[i].y), q2 = q8(v[i].z), q3 = q8(v[i].w);
            qsum += q0 + q1 + q2 + q3;
            words[i] = uint32_t(q0 & 0xFF) | (uint32_t(q1 & 0xFF) << 8) | (uint32_t(q2 & 0xFF) << 16) |
                       (uint32_t(q3 & 0xFF) << 24);
        }
        uint4* dst = reinterpret_cast<uint4*>(xq_row + b * QK);
        dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
        dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
        xs_row[b] = d;
        xsum_row[b] = d * float(qsum);
    }
}

}  // namespace tc
