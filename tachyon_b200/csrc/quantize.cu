// Tachyon's weight quantizers on the device: what Matrix::from_f32 (src/weights.rs:82-105)
// does on the host when a checkpoint is loaded, producing the same bytes.
//
//   bf16  - f32_to_bf16 (src/kernels.rs:21-28): round to nearest even, NaN -> 0x7FC0.
//   8-bit - quantize_q8_weights (src/kernels.rs:135-149): per 32 weights the scale
//           f16(amax / 127), values rounded (half away from zero) against the
//           f16 scale read back with f16_finite, clamped to +-127.
//   4-bit - quantize_q4_packed (src/kernels.rs:180-242) with fit_q4_offset
//           (438-495), no importance matrix: per block a weighted least-squares
//           fit of (scale, offset) over 21 candidate level assignments, then per
//           super-block of 8 blocks two f16 steps and, per block, the best of the
//           four roundings of (scale, offset) onto the 8-bit grid with the levels
//           refitted.
//
// Every float operation is the reference's, in its order: sums run left to right
// from zero, products are rounded before they are added (the library is compiled
// without fused multiply-add contraction), divisions and square roots are the
// IEEE ones. The per-block work is independent, so it maps to a thread per block
// (fit) and a thread per super-block (packing); only the row's mean square is a
// serial sum, done by one warp per row.
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"

namespace tc {

namespace {

__device__ __forceinline__ float f16_finite_bits(uint16_t h) {  // src/kernels.rs:127-130
    const uint32_t v = uint32_t(h) & 0x7FFFu, sign = (uint32_t(h) & 0x8000u) << 16;
    return __uint_as_float(sign | (v << 13)) * __uint_as_float(0x77800000u);
}

__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) {  // src/kernels.rs:31-60: nearest even
    return __half_as_ushort(__float2half_rn(f));
}

__global__ void bf16_kernel(const float* __restrict__ x, size_t n, uint16_t* __restrict__ out) {
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
        const float f = x[i];
        const uint32_t bits = __float_as_uint(f);
        out[i] = f != f ? uint16_t(0x7FC0) : uint16_t((bits + (0x7FFFu + ((bits >> 16) & 1u))) >> 16);
    }
}

// A warp per 32-weight block.
__global__ void q8_kernel(const float* __restrict__ x, size_t nblocks, uint16_t* __restrict__ scales,
                          int8_t* __restrict__ qs) {
    const int lane = threadIdx.x & 31;
    const size_t warp = size_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const size_t nwarps = size_t(gridDim.x) * (blockDim.x >> 5);
    for (size_t b = warp; b < nblocks; b += nwarps) {
        const float v = x[b * QK + lane];
        float amax = fabsf(v);  // f32::max drops NaN operands, as fmaxf does
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const uint16_t h = f32_to_f16_bits(__fdiv_rn(amax, 127.0f));
        const float d = f16_finite_bits(h);
        const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        const float r = roundf(v * id);
        qs[b * QK + lane] = int8_t(r != r ? 0 : int(fminf(127.0f, fmaxf(-127.0f, r))));
        if (lane == 0) scales[b] = h;
    }
}

// sigma2[row] = (sum of squares, left to right) / cols. A warp per row: the lanes load 32
// elements at a time and every lane adds them in order.
__global__ void q4_sigma_kernel(const float* __restrict__ x, size_t rows, int cols, float* __restrict__ sigma2) {
    const int lane = threadIdx.x & 31;
    const size_t warp = size_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const size_t nwarps = size_t(gridDim.x) * (blockDim.x >> 5);
    for (size_t r = warp; r < rows; r += nwarps) {
        const float* row = x + r * cols;
        float acc = 0.0f;
        for (int c0 = 0; c0 < cols; c0 += 32) {
            const float v = c0 + lane < cols ? row[c0 + lane] : 0.0f;
            const float sq = v * v;
            const int n = min(32, cols - c0);
            for (int j = 0; j < n; j++) acc = acc + __shfl_sync(0xffffffffu, sq, j);
        }
        if (lane == 0) sigma2[r] = __fdiv_rn(acc, float(cols));
    }
}

__device__ __forceinline__ float level_of(float v, float lo, float iscale) {
    return fminf(15.0f, fmaxf(0.0f, roundf((v - lo) * iscale)));
}

// fit_q4_offset for one block (a thread per block): the free (scale, offset) fit.
__global__ void q4_fit_kernel(const float* __restrict__ xall, const float* __restrict__ sigma2, size_t nblocks,
                              int nb, float* __restrict__ d_out, float* __restrict__ c_out) {
    const size_t blk = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (blk >= nblocks) return;
    const float s2 = sigma2[blk / nb];
    float x[QK], w[QK];
    const float4* src = reinterpret_cast<const float4*>(xall + blk * QK);
#pragma unroll
    for (int i = 0; i < QK / 4; i++) {
        const float4 v = src[i];
        x[4 * i] = v.x, x[4 * i + 1] = v.y, x[4 * i + 2] = v.z, x[4 * i + 3] = v.w;
    }
    float lo = __int_as_float(0x7f800000), hi = __int_as_float(0xff800000);
#pragma unroll
    for (int j = 0; j < QK; j++) {
        w[j] = __fsqrt_rn(s2 + x[j] * x[j]);
        lo = fminf(lo, x[j]);
        hi = fmaxf(hi, x[j]);
    }
    if (hi <= lo) {  // a constant block: all offset
        d_out[blk] = 0.0f;
        c_out[blk] = lo;
        return;
    }
    const float range = hi - lo;
    auto err = [&](float a, float m, float iscale) {
        float e = 0.0f;
#pragma unroll
        for (int j = 0; j < QK; j++) {
            const float r = x[j] - a * level_of(x[j], lo, iscale) - m;
            e = e + w[j] * (r * r);
        }
        return e;
    };
    // The plain choice: the block's range in 15 steps from its minimum.
    float best_a = __fdiv_rn(range, 15.0f), best_m = lo;
    float best_e = err(best_a, best_m, __fdiv_rn(15.0f, range));
#pragma unroll 1
    for (int step = -10; step <= 10; step++) {
        const float iscale = __fdiv_rn(15.0f + 0.1f * float(step), range);
        // weighted least squares for x = a * level + m
        float sw = 0.0f, sl = 0.0f, sll = 0.0f, sx = 0.0f, slx = 0.0f;
#pragma unroll
        for (int j = 0; j < QK; j++) {
            const float l = level_of(x[j], lo, iscale);
            sw = sw + w[j];
            sl = sl + w[j] * l;
            sll = sll + w[j] * l * l;
            sx = sx + w[j] * x[j];
            slx = slx + w[j] * l * x[j];
        }
        const float det = sw * sll - sl * sl;
        if (det <= 0.0f) continue;
        const float a = __fdiv_rn(sw * slx - sl * sx, det);
        const float m = __fdiv_rn(sll * sx - sl * slx, det);
        const float e = err(a, m, iscale);
        if (e < best_e) best_a = a, best_m = m, best_e = e;
    }
    // value = a * level + m = a * (level - 8) + (m + 8 a)
    d_out[blk] = fmaxf(best_a, 0.0f);
    c_out[blk] = best_m + 8.0f * best_a;
}

// One super-block (up to 8 blocks of a row) per thread: the two f16 steps, then per block the
// best of the four grid roundings with its levels refitted; packs the five words and the nibbles.
__global__ void q4_pack_kernel(const float* __restrict__ xall, const float* __restrict__ sigma2,
                               const float* __restrict__ d_fit, const float* __restrict__ c_fit, size_t rows, int nb,
                               uint32_t* __restrict__ packed, uint8_t* __restrict__ qs) {
    const int supers = (nb + SUPER - 1) / SUPER;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= rows * supers) return;
    const size_t row = idx / supers;
    const int k = int(idx - row * supers);
    const int b0 = k * SUPER, b1 = min(nb, b0 + SUPER);
    const float s2 = sigma2[row];
    float dmax = 0.0f, cmax = 0.0f;
    for (int b = b0; b < b1; b++) {
        dmax = fmaxf(dmax, d_fit[row * nb + b]);
        cmax = fmaxf(cmax, fabsf(c_fit[row * nb + b]));
    }
    const uint16_t dh = f32_to_f16_bits(__fdiv_rn(dmax, 255.0f)), mh = f32_to_f16_bits(__fdiv_rn(cmax, 127.0f));
    const float step_d = f16_finite_bits(dh), step_c = f16_finite_bits(mh);
    uint32_t words[SUPER_WORDS] = {uint32_t(dh) | (uint32_t(mh) << 16), 0u, 0u, 0u, 0u};
    for (int b = b0; b < b1; b++) {
        const int j = b - b0;
        const float* xb = xall + (row * nb + b) * QK;
        const float d = d_fit[row * nb + b], c = c_fit[row * nb + b];
        float x[QK], w[QK];
#pragma unroll
        for (int i = 0; i < QK; i++) {
            x[i] = xb[i];
            w[i] = __fsqrt_rn(s2 + x[i] * x[i]);
        }
        const float fs = step_d > 0.0f ? floorf(__fdiv_rn(d, step_d)) : 0.0f;
        const float fo = step_c > 0.0f ? floorf(__fdiv_rn(c, step_c)) : 0.0f;
        float best_err = __int_as_float(0x7f800000);
        uint32_t best_s = 0, best_o = 0;
        uint32_t best_nib[4] = {0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u};  // level 8 everywhere
#pragma unroll 1
        for (int opt = 0; opt < 4; opt++) {
            const float s = fminf(255.0f, fmaxf(0.0f, fs + float(opt >> 1)));
            const float o = fminf(127.0f, fmaxf(-128.0f, fo + float(opt & 1)));
            const float dq = step_d * s, cq = step_c * o;
            const float id = dq > 0.0f ? __fdiv_rn(1.0f, dq) : 0.0f;
            float e = 0.0f;
            uint32_t nib[4] = {0u, 0u, 0u, 0u};  // byte i of the block = level i | level (i + 16) << 4
#pragma unroll
            for (int i = 0; i < QK; i++) {
                const float l = fminf(15.0f, fmaxf(0.0f, roundf((x[i] - cq) * id + 8.0f)));
                const float r = x[i] - dq * (l - 8.0f) - cq;
                e = e + w[i] * (r * r);
                const uint32_t li = uint32_t(l != l ? 0.0f : l);
                const int byte = i & 15;
                nib[byte >> 2] |= (i < 16 ? li : li << 4) << (8 * (byte & 3));
            }
            if (e < best_err) {
                best_err = e;
                best_s = uint32_t(s);
                best_o = uint32_t(uint8_t(int8_t(int(o))));
#pragma unroll
                for (int q = 0; q < 4; q++) best_nib[q] = nib[q];
            }
        }
        words[1 + j / 4] |= best_s << (8 * (j % 4));
        words[3 + j / 4] |= best_o << (8 * (j % 4));
        uint32_t* dst = reinterpret_cast<uint32_t*>(qs + (row * nb + b) * (QK / 2));
#pragma unroll
        for (int q = 0; q < 4; q++) dst[q] = best_nib[q];
    }
    uint32_t* wp = packed + (row * supers + k) * SUPER_WORDS;
#pragma unroll
    for (int q = 0; q < SUPER_WORDS; q++) wp[q] = words[q];
}

}  // namespace

// Quantizes x[rows, cols] (device, f32) into the buffers of a Matrix of `kind`. `scratch` holds
// rows * (1 + 2 * cols / 32) floats for the 4-bit fit (unused otherwise). Returns kernels launched.
int launch_quantize(int kind, const float* x, size_t rows, size_t cols, void* scales, void* data, float* scratch,
                    cudaStream_t stream) {
    const size_t n = rows * cols, nblocks = n / QK;
    const int nb = int(cols / QK);
    auto grid_for = [](size_t work, int per_block) {
        return unsigned(std::min<size_t>((work + per_block - 1) / per_block, 148 * 64));
    };
    if (kind == 0) {
        bf16_kernel<<<grid_for(n, 256), 256, 0, stream>>>(x, n, static_cast<uint16_t*>(data));
        return 1;
    }
    if (kind == 1) {
        q8_kernel<<<grid_for(nblocks, 8), 256, 0, stream>>>(x, nblocks, static_cast<uint16_t*>(scales),
                                                           static_cast<int8_t*>(data));
        return 1;
    }
    float* sigma2 = scratch;
    float* d_fit = scratch + rows;
    float* c_fit = d_fit + nblocks;
    q4_sigma_kernel<<<grid_for(rows, 8), 256, 0, stream>>>(x, rows, int(cols), sigma2);
    q4_fit_kernel<<<unsigned((nblocks + 127) / 128), 128, 0, stream>>>(x, sigma2, nblocks, nb, d_fit, c_fit);
    const size_t supers = rows * ((nb + SUPER - 1) / SUPER);
    q4_pack_kernel<<<unsigned((supers + 127) / 128), 128, 0, stream>>>(x, sigma2, d_fit, c_fit, rows, nb,
                                                                       static_cast<uint32_t*>(scales),
                                                                       static_cast<uint8_t*>(data));
    return 3;
}

}  // namespace tc
