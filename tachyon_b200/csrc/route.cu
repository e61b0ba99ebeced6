// Router GEMV + top-k + gating softmax + activation quantization, one CTA per
// token; and the row RMSNorm that produces the block's input.
//
// Reproduces, value for value:
//   router logits  - Matrix::matmul's bf16 arm (src/weights.rs:230-240) with
//                    the AVX2 dot bf16s (src/kernels_x86.rs:157-171): two
//                    8-lane fma accumulators over 16-element strides, summed
//                    lane-wise, then the fixed hsum tree (33-38);
//   top-k + gates  - route() (src/model.rs:448-457): order by total_cmp
//                    descending, ties to the lower expert, softmax over the k
//                    kept with max = the top score, sum taken in that order;
//   quantization   - quantize_q8 (src/kernels.rs:84-98) per 32-block, as
//                    quantize_input applies it per token (src/weights.rs:652-664);
//   rmsnorm        - src/kernels.rs:522-528 with dot_f32's AVX2 order
//                    (src/kernels_x86.rs:132-154).
// The softmax exponential is evaluated in double precision and rounded to
// float; the CPU path calls libm's expf. The two agree except where expf
// itself is not correctly rounded, hence the 1e-5 tolerance on gates.
#include "common.cuh"

namespace tc {

namespace {

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
    return __uint_as_float(uint32_t(b) << 16);
}

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

constexpr int ROUTE_THREADS = 512;

__global__ void __launch_bounds__(ROUTE_THREADS)
route_quant_kernel(const uint16_t* __restrict__ router, const float* __restrict__ bias,
                   const float* __restrict__ x, int hidden, int experts, int topk,
                   float* __restrict__ logits_out, uint32_t* __restrict__ ids_out,
                   float* __restrict__ gates_out, int8_t* __restrict__ xq, float* __restrict__ xs,
                   float* __restrict__ xsum) {
    extern __shared__ float smem[];
    float* xrow = smem;              // [hidden]
    float* slog = smem + hidden;     // [experts]
    const int token = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* xin = x + size_t(token) * hidden;
    for (int c = tid * 4; c < hidden; c += ROUTE_THREADS * 4)
        *reinterpret_cast<float4*>(xrow + c) = *reinterpret_cast<const float4*>(xin + c);
    __syncthreads();

    // ---- logits: 16 lanes per expert; lane L owns elements L, L+16, L+32, ...
    {
        const int groups = ROUTE_THREADS / 16;
        const int g = tid >> 4, L = tid & 15;
        for (int e0 = 0; e0 < experts; e0 += groups) {
            const int e = e0 + g;
            const bool valid = e < experts;
            const uint16_t* w = router + size_t(valid ? e : 0) * hidden;
            float acc = 0.0f;
#pragma unroll 16
            for (int c = L; c < hidden; c += 16) acc = fmaf(bf16_bits_to_f32(w[c]), xrow[c], acc);
            // acc0 + acc1 lane-wise (lanes L and L+8), then the hsum tree.
            float v = acc + __shfl_down_sync(0xffffffffu, acc, 8, 16);
            v = hsum8(v, 0xffffffffu);
            if (valid && L == 0) {
                // The dot's scalar tail is an empty sum: hsum + 0.0.
                v = v + 0.0f;
                if (bias) v = v + bias[e];
                slog[e] = v;
                if (logits_out) logits_out[size_t(token) * experts + e] = v;
            }
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
            ids_out[size_t(token) * topk + lane] = uint32_t(my_id);
            gates_out[size_t(token) * topk + lane] = __fdiv_rn(ej, sum);
        }
    }

    // ---- 8-bit quantization of the row, a warp per 32-block.
    const int nb = hidden / QK;
    const int padded = (nb + SUPER - 1) / SUPER * SUPER;
    for (int b = warp; b < padded; b += ROUTE_THREADS / 32) {
        if (b >= nb) {  // zero padding up to whole super-blocks
            if (lane == 0) {
                xs[size_t(token) * padded + b] = 0.0f;
                xsum[size_t(token) * padded + b] = 0.0f;
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
        xq[size_t(token) * hidden + b * QK + lane] = int8_t(q);
        int qsum = q;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
        if (lane == 0) {
            xs[size_t(token) * padded + b] = d;
            xsum[size_t(token) * padded + b] = d * float(qsum);
        }
    }
}

// One warp per row. Lane L owns elements L, L+32, ...: the four 8-lane
// accumulators of dot_f32's main loop side by side.
__global__ void rmsnorm_kernel(const float* x, const float* __restrict__ w, float eps, int t, int n,
                               float* out) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= t) return;
    const float* xr = x + size_t(row) * n;
    float acc = 0.0f;
    int i = 0;
#pragma unroll 16
    for (; i + 32 <= n; i += 32) {
        float v = xr[i + lane];
        acc = fmaf(v, v, acc);
    }
    // Leftover groups of eight go to the first accumulator, one after another.
    for (; i + 8 <= n; i += 8) {
        if (lane < 8) {
            float v = xr[i + lane];
            acc = fmaf(v, v, acc);
        }
    }
    // (acc0 + acc1) + (acc2 + acc3), lane-wise over j = lane % 8.
    float s = acc + __shfl_down_sync(0xffffffffu, acc, 8);   // lanes 0-7: a0+a1; 16-23: a2+a3
    s = s + __shfl_down_sync(0xffffffffu, s, 16);            // lanes 0-7: the four summed
    s = hsum8(s, 0xffffffffu);
    float tail = 0.0f;
    for (int j = i; j < n; j++) tail = tail + xr[j] * xr[j];
    s = s + tail;
    s = __shfl_sync(0xffffffffu, s, 0);
    const float ss = __fdiv_rn(s, float(n));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(ss + eps));
    float* o = out + size_t(row) * n;
#pragma unroll 8
    for (int c = lane; c < n; c += 32) o[c] = xr[c] * inv * w[c];
}

}  // namespace

int launch_route(const MoeDims& d, const uint16_t* router, const float* bias, const float* x, int t,
                 Workspace& ws, cudaStream_t stream) {
    size_t smem = size_t(d.hidden + d.experts) * sizeof(float);
    route_quant_kernel<<<t, ROUTE_THREADS, smem, stream>>>(router, bias, x, d.hidden, d.experts,
                                                           d.topk, ws.logits, ws.ids, ws.gates,
                                                           ws.xq, ws.xs, ws.xsum);
    return 1;
}

int launch_rmsnorm(const float* x, const float* w, float eps, int t, int n, float* out,
                   cudaStream_t stream) {
    const int warps = 4;
    rmsnorm_kernel<<<(t + warps - 1) / warps, warps * 32, 0, stream>>>(x, w, eps, t, n, out);
    return 1;
}

}  // namespace tc
