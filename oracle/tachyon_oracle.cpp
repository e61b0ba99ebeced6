// CPU oracle for the Granite mixture-of-experts block: TEST INFRASTRUCTURE ONLY.
//
// A restatement, in C++ with AVX2/FMA intrinsics, of the arithmetic Tachyon's
// x86-64 CPU path performs for one MoE block. It is the checker the CUDA path
// is compared against, and the CPU baseline that is timed beside it. Nothing
// in the shipped library links, loads or calls this file.
//
// Every function names the reference source it follows (paths are relative to
// the Tachyon project root). The restatement keeps the reference's operation
// ORDER (which value is multiplied or added to which, where an fma is used
// and where it is not), because float results depend on it; it does not keep
// the reference's code structure.
//
// Build: g++ -O2 -mavx2 -mfma -mf16c -ffp-contract=off -fno-fast-math
//   -ffp-contract=off matters: Rust never contracts a*b+c into an fma unless
//   the source says mul_add, so neither may this file.
//
// Parity pinning: the known-answer and property tests Tachyon keeps beside
// this code (src/model.rs:790-798, src/kernels.rs:1523-1810,
// src/weights.rs:685-731) are restated in tests/ and run against this file.

#include <immintrin.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace {

constexpr int QK = 32;          // src/kernels.rs:13
constexpr int SUPER = 8;        // src/kernels.rs:165
constexpr int SUPER_WORDS = 5;  // src/kernels.rs:167

inline float bits_f32(uint32_t b) {
    float f;
    std::memcpy(&f, &b, 4);
    return f;
}
inline uint32_t f32_bits(float f) {
    uint32_t b;
    std::memcpy(&b, &f, 4);
    return b;
}

// ---------------------------------------------------------------- conversions

// src/kernels.rs:16-18
inline float bf16_to_f32(uint16_t b) { return bits_f32(uint32_t(b) << 16); }

// src/kernels.rs:21-28 (round to nearest even; NaN -> 0x7FC0)
uint16_t f32_to_bf16(float f) {
    if (std::isnan(f)) return 0x7FC0;
    uint32_t bits = f32_bits(f);
    uint32_t round = 0x7FFFu + ((bits >> 16) & 1u);
    return uint16_t((bits + round) >> 16);
}

// src/kernels.rs:31-60 (round to nearest even, subnormals, overflow to inf)
uint16_t f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint16_t sign = uint16_t((x >> 16) & 0x8000u);
    int exp = int((x >> 23) & 0xFFu);
    uint32_t mant = x & 0x7FFFFFu;
    if (exp == 0xFF) return uint16_t(sign | 0x7C00u | (mant ? 0x200u : 0u));
    int e = exp - 127 + 15;
    if (e >= 0x1F) return uint16_t(sign | 0x7C00u);
    uint32_t full, shift, base;
    if (e > 0) {
        full = mant;
        shift = 13;
        base = uint32_t(e) << 10;
    } else {
        full = mant | 0x800000u;
        shift = uint32_t(14 - e);
        base = 0;
    }
    if (shift > 25) return sign;
    uint32_t h = base | (full >> shift);
    uint32_t rem = full & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1u))) h += 1;
    return uint16_t(sign | uint16_t(h));
}

// src/kernels.rs:62-81
float f16_to_f32(uint16_t h) {
    uint32_t sign = uint32_t(h >> 15) << 31;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t frac = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0 && frac == 0) {
        bits = sign;
    } else if (exp == 0) {
        uint32_t e = 127 - 15 + 1;
        while ((frac & 0x400u) == 0) {
            frac <<= 1;
            e -= 1;
        }
        bits = sign | (e << 23) | ((frac & 0x3FFu) << 13);
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (frac << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (frac << 13);
    }
    return bits_f32(bits);
}

// src/kernels.rs:127-130 (finite halves only: shift into place, times 2^112)
inline float f16_finite(uint16_t h) {
    uint32_t v = uint32_t(h) & 0x7FFFu, sign = (uint32_t(h) & 0x8000u) << 16;
    return bits_f32(sign | (v << 13)) * bits_f32(0x77800000u);
}

// Rust's f32::round: half away from zero. C's roundf has the same rule.
inline float round_away(float v) { return std::roundf(v); }

// Rust's `as i8` from f32: saturating, NaN -> 0.
inline int8_t sat_i8(float v) {
    if (std::isnan(v)) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return int8_t(int(v));
}

// ---------------------------------------------------------------- quantizers

// src/kernels.rs:84-98: activations, f32 scale per block.
void quantize_q8(const float* x, size_t n, float* scales, int8_t* qs) {
    for (size_t b = 0; b < n / QK; b++) {
        const float* blk = x + b * QK;
        float amax = 0.0f;
        for (int j = 0; j < QK; j++) amax = std::max(amax, std::fabs(blk[j]));
        float d = amax / 127.0f;
        float id = d > 0.0f ? 1.0f / d : 0.0f;
        for (int j = 0; j < QK; j++) qs[b * QK + j] = sat_i8(round_away(blk[j] * id));
        scales[b] = d;
    }
}

// src/kernels.rs:103-121: symmetric 4-bit (used by the reference's kernel tests).
void quantize_q4(const float* x, size_t n, float* scales, uint8_t* qs) {
    for (size_t b = 0; b < n / QK; b++) {
        const float* blk = x + b * QK;
        float mx = 0.0f;
        for (int j = 0; j < QK; j++)
            if (std::fabs(blk[j]) > std::fabs(mx)) mx = blk[j];
        float d = mx / -8.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        auto nibble = [&](float v) -> uint8_t {
            // `as i32` truncates toward zero (saturating); then clamp 0..15.
            float f = v * id + 8.5f;
            int i = std::isnan(f) ? 0 : (f >= 2147483648.0f ? INT32_MAX : (f <= -2147483648.0f ? INT32_MIN : int(f)));
            return uint8_t(std::min(15, std::max(0, i)));
        };
        for (int j = 0; j < QK / 2; j++)
            qs[b * (QK / 2) + j] = uint8_t(nibble(blk[j]) | (nibble(blk[j + QK / 2]) << 4));
        scales[b] = d;
    }
}

// src/kernels.rs:135-149: weights, f16 scale per block, rounded against it.
void quantize_q8_weights(const float* x, size_t n, uint16_t* scales, int8_t* qs) {
    for (size_t b = 0; b < n / QK; b++) {
        const float* blk = x + b * QK;
        float amax = 0.0f;
        for (int j = 0; j < QK; j++) amax = std::max(amax, std::fabs(blk[j]));
        scales[b] = f32_to_f16(amax / 127.0f);
        float d = f16_finite(scales[b]);
        float id = d > 0.0f ? 1.0f / d : 0.0f;
        for (int j = 0; j < QK; j++) {
            float r = round_away(blk[j] * id);
            r = std::min(127.0f, std::max(-127.0f, r));
            qs[b * QK + j] = sat_i8(r);
        }
    }
}

inline float powi2(float v) { return v * v; }

// src/kernels.rs:438-495: weighted least-squares fit of one block to
// value = d*(level-8) + c, trying 21 roundings around the plain one.
void fit_q4_offset(const float* x, const float* w, float* d_out, float* c_out) {
    float lo = INFINITY, hi = -INFINITY;
    for (int j = 0; j < QK; j++) {
        lo = std::min(lo, x[j]);
        hi = std::max(hi, x[j]);
    }
    if (hi <= lo) {
        *d_out = 0.0f;
        *c_out = lo;
        return;
    }
    uint8_t l[QK];
    auto levels_for = [&](float iscale) {
        for (int j = 0; j < QK; j++) {
            float r = round_away((x[j] - lo) * iscale);
            r = std::min(15.0f, std::max(0.0f, r));
            l[j] = uint8_t(r);
        }
    };
    auto err = [&](float a, float m) {
        float s = 0.0f;
        for (int j = 0; j < QK; j++) s += w[j] * powi2(x[j] - a * float(l[j]) - m);
        return s;
    };
    levels_for(15.0f / (hi - lo));
    float best_a = (hi - lo) / 15.0f, best_m = lo;
    float best_e = err(best_a, best_m);
    for (int step = -10; step <= 10; step++) {
        levels_for((15.0f + 0.1f * float(step)) / (hi - lo));
        float sw = 0, sl = 0, sll = 0, sx = 0, slx = 0;
        for (int j = 0; j < QK; j++) {
            float lj = float(l[j]);
            sw += w[j];
            sl += w[j] * lj;
            sll += w[j] * lj * lj;
            sx += w[j] * x[j];
            slx += w[j] * lj * x[j];
        }
        float det = sw * sll - sl * sl;
        if (det <= 0.0f) continue;
        float a = (sw * slx - sl * sx) / det;
        float m = (sll * sx - sl * slx) / det;
        float e = err(a, m);
        if (e < best_e) {
            best_a = a;
            best_m = m;
            best_e = e;
        }
    }
    *d_out = best_a;
    *c_out = best_m + 8.0f * best_a;
}

// src/kernels.rs:180-242: one row to packed 4-bit. `packed` holds
// ceil(nb/8)*5 words, `qs` cols/2 bytes. importance may be null.
void quantize_q4_packed(const float* row, size_t cols, const float* importance, uint32_t* packed,
                        uint8_t* qs) {
    float ss = 0.0f;
    for (size_t i = 0; i < cols; i++) ss += row[i] * row[i];
    float sigma2 = ss / float(cols);
    size_t nb = cols / QK;
    size_t supers = (nb + SUPER - 1) / SUPER;
    for (size_t k = 0; k < supers; k++) {
        uint32_t* words = packed + k * SUPER_WORDS;
        size_t b0 = k * SUPER, b1 = std::min((k + 1) * SUPER, nb);
        float fd[SUPER], fc[SUPER], fw[SUPER][QK];
        for (size_t b = b0; b < b1; b++) {
            const float* x = row + b * QK;
            float* w = fw[b - b0];
            for (int j = 0; j < QK; j++) {
                float imp = importance ? importance[b * QK + j] : 1.0f;
                w[j] = imp * std::sqrt(sigma2 + x[j] * x[j]);
            }
            float d, c;
            fit_q4_offset(x, w, &d, &c);
            fd[b - b0] = std::max(d, 0.0f);
            fc[b - b0] = c;
        }
        float dmax = 0.0f, cmax = 0.0f;
        for (size_t b = b0; b < b1; b++) {
            dmax = std::max(dmax, fd[b - b0]);
            cmax = std::max(cmax, std::fabs(fc[b - b0]));
        }
        uint16_t dh = f32_to_f16(dmax / 255.0f), mh = f32_to_f16(cmax / 127.0f);
        float step_d = f16_finite(dh), step_c = f16_finite(mh);
        for (int i = 0; i < SUPER_WORDS; i++) words[i] = 0;
        words[0] = uint32_t(dh) | (uint32_t(mh) << 16);
        for (size_t b = b0; b < b1; b++) {
            size_t j = b - b0;
            const float* x = row + b * QK;
            const float* w = fw[j];
            auto near2 = [](float v, float step, float lo, float hi, float out[2]) {
                float f = step > 0.0f ? std::floor(v / step) : 0.0f;
                out[0] = std::min(hi, std::max(lo, f));
                out[1] = std::min(hi, std::max(lo, f + 1.0f));
            };
            float ss2[2], oo2[2];
            near2(fd[j], step_d, 0.0f, 255.0f, ss2);
            near2(fc[j], step_c, -128.0f, 127.0f, oo2);
            float best_err = INFINITY;
            uint32_t best_s = 0, best_o = 0;
            uint8_t best_levels[QK];
            for (int i = 0; i < QK; i++) best_levels[i] = 8;
            for (int si = 0; si < 2; si++) {
                for (int oi = 0; oi < 2; oi++) {
                    float s = ss2[si], o = oo2[oi];
                    float dq = step_d * s, cq = step_c * o;
                    float id = dq > 0.0f ? 1.0f / dq : 0.0f;
                    uint8_t levels[QK];
                    float e = 0.0f;
                    for (int i = 0; i < QK; i++) {
                        float l = round_away((x[i] - cq) * id + 8.0f);
                        l = std::min(15.0f, std::max(0.0f, l));
                        levels[i] = uint8_t(l);
                        e += w[i] * powi2(x[i] - dq * (l - 8.0f) - cq);
                    }
                    if (e < best_err) {
                        best_err = e;
                        best_s = uint32_t(s);
                        best_o = uint32_t(uint8_t(int8_t(int(o))));
                        std::memcpy(best_levels, levels, QK);
                    }
                }
            }
            words[1 + j / 4] |= best_s << (8 * (j % 4));
            words[3 + j / 4] |= best_o << (8 * (j % 4));
            uint8_t* q = qs + b * (QK / 2);
            for (int i = 0; i < QK / 2; i++)
                q[i] = uint8_t(best_levels[i] | (best_levels[i + QK / 2] << 4));
        }
    }
}

// src/kernels.rs:256-267: packed scales -> per-block d and c (nb of each).
void unpack_q4(const uint32_t* packed, size_t nb, float* d, float* c) {
    for (size_t k = 0; k * SUPER < nb; k++) {
        const uint32_t* w = packed + k * SUPER_WORDS;
        float step_d = f16_finite(uint16_t(w[0])), step_c = f16_finite(uint16_t(w[0] >> 16));
        for (size_t j = 0; j < SUPER && k * SUPER + j < nb; j++) {
            uint32_t s = w[1 + j / 4] >> (8 * (j % 4)), o = w[3 + j / 4] >> (8 * (j % 4));
            d[k * SUPER + j] = step_d * float(uint8_t(s));
            c[k * SUPER + j] = step_c * float(int8_t(uint8_t(o)));
        }
    }
}

// src/kernels.rs:497-507
void dequantize_q8(const float* scales, const int8_t* qs, size_t n, float* out) {
    for (size_t i = 0; i < n; i++) out[i] = float(qs[i]) * scales[i / QK];
}

// src/kernels.rs:509-520
void dequantize_q4(const float* scales, const uint8_t* qs, size_t n, float* out) {
    for (size_t b = 0; b < n / QK; b++)
        for (int j = 0; j < QK / 2; j++) {
            uint8_t q = qs[b * (QK / 2) + j];
            out[b * QK + j] = float(int(q & 0xF) - 8) * scales[b];
            out[b * QK + j + QK / 2] = float(int(q >> 4) - 8) * scales[b];
        }
}

// ---------------------------------------------------------------- AVX2 dots

// src/kernels_x86.rs:33-38
inline float hsum(__m256 v) {
    __m128 s = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    s = _mm_add_ss(s, _mm_movehdup_ps(s));
    return _mm_cvtss_f32(s);
}

// src/kernels_x86.rs:43-46: eight lane sums of four int8 products each.
inline __m256 block_q8(__m256i w, __m256i x) {
    __m256i p = _mm256_maddubs_epi16(_mm256_sign_epi8(w, w), _mm256_sign_epi8(x, w));
    return _mm256_cvtepi32_ps(_mm256_madd_epi16(p, _mm256_set1_epi16(1)));
}

// src/kernels_x86.rs:52-58: 16 bytes -> 32 unsigned nibbles (low ones first).
inline __m256i nibbles(const uint8_t* p) {
    __m128i raw = _mm_loadu_si128(reinterpret_cast<const __m128i*>(p));
    __m128i mask = _mm_set1_epi8(0x0F);
    __m128i lo = _mm_and_si128(raw, mask);
    __m128i hi = _mm_and_si128(_mm_srli_epi16(raw, 4), mask);
    return _mm256_set_m128i(hi, lo);
}

// src/kernels_x86.rs:63-70: sum (q - 8) x per lane.
inline __m256 block_q4(__m256i w, __m256i x) {
    __m256i p = _mm256_maddubs_epi16(w, x);
    __m256i eights = _mm256_maddubs_epi16(_mm256_set1_epi8(8), x);
    return _mm256_cvtepi32_ps(_mm256_madd_epi16(_mm256_sub_epi16(p, eights), _mm256_set1_epi16(1)));
}

inline __m256i load256(const void* p) {
    return _mm256_loadu_si256(reinterpret_cast<const __m256i*>(p));
}

// Where a row's block scales come from (src/kernels.rs:278-356): expanded
// f32, f16 as stored, or packed 4-bit words. All give the same value.
struct ExpandedScales {
    const float* d;
    float get(size_t b) const { return d[b]; }
};
struct HalfScales {
    const uint16_t* h;
    float get(size_t b) const { return f16_finite(h[b]); }
};
struct PackedScales {
    const uint32_t* words;
    float get(size_t b) const {
        const uint32_t* w = words + b / SUPER * SUPER_WORDS;
        uint8_t s = reinterpret_cast<const uint8_t*>(w + 1)[b % SUPER];
        return f16_finite(uint16_t(w[0])) * float(s);
    }
};

// src/kernels_x86.rs:79-87
template <class S>
float dot_q8_avx(S ws, size_t nb, const int8_t* wq, const float* xs, const int8_t* xq) {
    __m256 acc = _mm256_setzero_ps();
    for (size_t b = 0; b < nb; b++) {
        __m256 s = block_q8(load256(wq + b * QK), load256(xq + b * QK));
        float d = ws.get(b) * xs[b];
        acc = _mm256_fmadd_ps(s, _mm256_set1_ps(d), acc);
    }
    return hsum(acc);
}

// src/kernels_x86.rs:90-101
void dot_q8_x4_avx(const float* ws, size_t nb, const int8_t* wq, const float* const xs[4],
                   const int8_t* const xq[4], float out[4]) {
    __m256 acc[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(),
                     _mm256_setzero_ps()};
    for (size_t b = 0; b < nb; b++) {
        __m256i w = load256(wq + b * QK);
        for (int j = 0; j < 4; j++) {
            __m256 s = block_q8(w, load256(xq[j] + b * QK));
            float d = ws[b] * xs[j][b];
            acc[j] = _mm256_fmadd_ps(s, _mm256_set1_ps(d), acc[j]);
        }
    }
    for (int j = 0; j < 4; j++) out[j] = hsum(acc[j]);
}

// src/kernels_x86.rs:104-115
template <class S>
float dot_q4_avx(S ws, size_t nb, const uint8_t* wq, const float* xs, const int8_t* xq) {
    __m256 acc = _mm256_setzero_ps();
    for (size_t b = 0; b < nb; b++) {
        __m256 s = block_q4(nibbles(wq + b * QK / 2), load256(xq + b * QK));
        float d = ws.get(b) * xs[b];
        acc = _mm256_fmadd_ps(s, _mm256_set1_ps(d), acc);
    }
    return hsum(acc);
}

// src/kernels_x86.rs:118-129
void dot_q4_x4_avx(const float* ws, size_t nb, const uint8_t* wq, const float* const xs[4],
                   const int8_t* const xq[4], float out[4]) {
    __m256 acc[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(),
                     _mm256_setzero_ps()};
    for (size_t b = 0; b < nb; b++) {
        __m256i w = nibbles(wq + b * QK / 2);
        for (int j = 0; j < 4; j++) {
            __m256 s = block_q4(w, load256(xq[j] + b * QK));
            float d = ws[b] * xs[j][b];
            acc[j] = _mm256_fmadd_ps(s, _mm256_set1_ps(d), acc[j]);
        }
    }
    for (int j = 0; j < 4; j++) out[j] = hsum(acc[j]);
}

// src/kernels_x86.rs:132-154
float dot_f32_avx(const float* a, const float* b, size_t n) {
    __m256 acc[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(),
                     _mm256_setzero_ps()};
    size_t i = 0;
    while (i + 32 <= n) {
        for (int k = 0; k < 4; k++) {
            size_t o = i + 8 * k;
            acc[k] = _mm256_fmadd_ps(_mm256_loadu_ps(a + o), _mm256_loadu_ps(b + o), acc[k]);
        }
        i += 32;
    }
    while (i + 8 <= n) {
        acc[0] = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc[0]);
        i += 8;
    }
    __m256 all = _mm256_add_ps(_mm256_add_ps(acc[0], acc[1]), _mm256_add_ps(acc[2], acc[3]));
    // The tail is a Rust iterator sum: it starts from zero and adds in order.
    float tail = 0.0f;
    for (size_t j = i; j < n; j++) tail += a[j] * b[j];
    return hsum(all) + tail;
}

// src/kernels_x86.rs:157-171
float dot_bf16_avx(const uint16_t* w, const float* x, size_t n) {
    __m256 acc[2] = {_mm256_setzero_ps(), _mm256_setzero_ps()};
    size_t i = 0;
    while (i + 16 <= n) {
        for (int k = 0; k < 2; k++) {
            __m128i h = _mm_loadu_si128(reinterpret_cast<const __m128i*>(w + i + 8 * k));
            __m256 f = _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(h), 16));
            acc[k] = _mm256_fmadd_ps(f, _mm256_loadu_ps(x + i + 8 * k), acc[k]);
        }
        i += 16;
    }
    float tail = 0.0f;
    for (size_t j = i; j < n; j++) tail += bf16_to_f32(w[j]) * x[j];
    return hsum(_mm256_add_ps(acc[0], acc[1])) + tail;
}

// ------------------------------------------------- scalar dots (kernels.rs:1404-1456)

float dot_q8_scalar(const float* ws, size_t nb, const int8_t* wq, const float* xs,
                    const int8_t* xq) {
    float total = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        int32_t s = 0;
        for (int j = 0; j < QK; j++) s += int32_t(wq[b * QK + j]) * int32_t(xq[b * QK + j]);
        total += float(s) * ws[b] * xs[b];
    }
    return total;
}

float dot_q4_scalar(const float* ws, size_t nb, const uint8_t* wq, const float* xs,
                    const int8_t* xq) {
    float total = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        int32_t s = 0;
        for (int j = 0; j < QK / 2; j++) {
            uint8_t byte = wq[b * QK / 2 + j];
            s += (int32_t(byte & 0xF) - 8) * int32_t(xq[b * QK + j]);
            s += (int32_t(byte >> 4) - 8) * int32_t(xq[b * QK + j + QK / 2]);
        }
        total += float(s) * ws[b] * xs[b];
    }
    return total;
}

// ------------------------------------------------- model of the GPU's fast arithmetic
//
// NOT a restatement of the reference: the CUDA backend's default ("fast")
// arithmetic folds a block's eight AVX lanes into one exact integer sum and
// keeps a single fma chain per output, blocks in order. These two functions
// state that order on the CPU so the fast kernels can be pinned bit for bit;
// how far it sits from the reference order above is what the tolerance tests
// measure.
float dot_q8_chain(const float* ws, size_t nb, const int8_t* wq, const float* xs, const int8_t* xq) {
    float acc = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        int32_t s = 0;
        for (int j = 0; j < QK; j++) s += int32_t(wq[b * QK + j]) * int32_t(xq[b * QK + j]);
        acc = std::fmaf(float(s), ws[b] * xs[b], acc);
    }
    return acc;
}

float dot_q4_chain(const float* ws, const float* cs, size_t nb, const uint8_t* wq, const float* xs,
                   const int8_t* xq, const float* sums) {
    float acc = 0.0f, off = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        int32_t s = 0;
        for (int j = 0; j < QK / 2; j++) {
            uint8_t byte = wq[b * QK / 2 + j];
            s += (int32_t(byte & 0xF) - 8) * int32_t(xq[b * QK + j]);
            s += (int32_t(byte >> 4) - 8) * int32_t(xq[b * QK + j + QK / 2]);
        }
        acc = std::fmaf(float(s), ws[b] * xs[b], acc);
        off = std::fmaf(cs[b], sums[b], off);
    }
    return acc + off;
}

int g_arith = 0;  // 0: the reference's lane order; 1: the chain model above

// ------------------------------------------------- offsets (kernels.rs:392-432)

// Eight lanes, one per block of a super-block, fma'd over super-blocks, then
// ((a0+a4)+(a1+a5))+((a2+a6)+(a3+a7)). `sums` is padded to whole super-blocks.
template <class Fill>
float offsets_lanes(const float* sums, size_t padded, Fill fill) {
    float acc[SUPER] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (size_t k = 0; k < padded / SUPER; k++) {
        float c[SUPER];
        fill(k, c);
        for (int j = 0; j < SUPER; j++) acc[j] = std::fmaf(c[j], sums[k * SUPER + j], acc[j]);
    }
    float a[4];
    for (int j = 0; j < 4; j++) a[j] = acc[j] + acc[j + 4];
    return (a[0] + a[1]) + (a[2] + a[3]);
}

float dot_offsets(const uint32_t* words, const float* sums, size_t padded) {
    return offsets_lanes(sums, padded, [&](size_t k, float* c) {
        const uint32_t* w = words + k * SUPER_WORDS;
        float step = f16_finite(uint16_t(w[0] >> 16));
        for (int j = 0; j < SUPER; j++)
            c[j] = step * float(int8_t(uint8_t(w[3 + j / 4] >> (8 * (j % 4)))));
    });
}

float dot_offsets_expanded(const float* c_exp, const float* sums, size_t padded) {
    return offsets_lanes(sums, padded, [&](size_t k, float* c) {
        for (int j = 0; j < SUPER; j++) c[j] = c_exp[k * SUPER + j];
    });
}

// ------------------------------------------------- elementwise (kernels.rs:522-610)

// src/kernels.rs:544-564: Cephes-style exp, the polynomial in Horner form
// with separate multiplies and adds.
float exp_scalar(float x) {
    static const float P[6] = {1.9875692e-4f, 1.3981999e-3f, 8.333452e-3f,
                               4.1665796e-2f, 0.16666665f,   0.5f};
    // f32::clamp: NaN stays NaN; otherwise max(lo) then min(hi).
    if (x < -87.33655f) x = -87.33655f;
    if (x > 88.7f) x = 88.7f;
    float n = round_away(x * 1.44269504088896340736f);
    float r = x - n * 0.6933594f - n * -2.1219444e-4f;
    float y = P[0];
    for (int i = 1; i < 6; i++) y = y * r + P[i];
    y = y * (r * r) + r + 1.0f;
    int32_t bits = int32_t(f32_bits(y)) + int32_t(uint32_t(int32_t(n)) << 23);
    return bits_f32(uint32_t(bits));
}

// src/kernels.rs:595-603
void silu_mul(const float* g, const float* u, size_t n, float* out) {
    for (size_t i = 0; i < n; i++) out[i] = exp_scalar(-g[i]);
    for (size_t i = 0; i < n; i++) out[i] = g[i] / (1.0f + out[i]) * u[i];
}

// src/kernels.rs:522-528
void rmsnorm(float* out, const float* x, const float* w, size_t n, float eps) {
    float ss = dot_f32_avx(x, x, n) / float(n);
    float inv = 1.0f / std::sqrt(ss + eps);
    for (size_t i = 0; i < n; i++) out[i] = x[i] * inv * w[i];
}

// src/kernels.rs:606-610: out += a * x, the product rounded before the add.
void axpy(float* out, float a, const float* x, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] += a * x[i];
}

// ------------------------------------------------- thread pool (pool.rs:126-145)

// parallel_for hands out chunks of `grain` items from a shared counter, as
// the reference's pool does. Which thread computes an output never changes
// its value, so this only matters for timing.
class Pool {
  public:
    explicit Pool(int threads) : n_(std::max(1, threads)) {
        for (int i = 1; i < n_; i++) workers_.emplace_back([this] { worker(); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> g(m_);
            stop_ = true;
            gen_++;
        }
        cv_.notify_all();
        for (auto& t : workers_) t.join();
    }
    int threads() const { return n_; }

    void parallel_for(size_t n, size_t grain, const std::function<void(size_t, size_t)>& f) {
        grain = std::max<size_t>(grain, 1);
        if (n <= grain || n_ == 1) {
            if (n > 0) f(0, n);
            return;
        }
        next_.store(0);
        n_items_ = n;
        grain_ = grain;
        job_ = &f;
        remaining_.store(n_ - 1);
        {
            std::lock_guard<std::mutex> g(m_);
            gen_++;
        }
        cv_.notify_all();
        run_chunks();
        while (remaining_.load(std::memory_order_acquire) != 0) _mm_pause();
        job_ = nullptr;
    }

  private:
    void run_chunks() {
        for (;;) {
            size_t start = next_.fetch_add(grain_);
            if (start >= n_items_) break;
            (*job_)(start, std::min(start + grain_, n_items_));
        }
    }
    void worker() {
        uint64_t seen = 0;
        for (;;) {
            // Spin a while before sleeping, as the reference's workers do.
            int spins = 0;
            while (gen_.load(std::memory_order_acquire) == seen && spins < (1 << 15)) {
                _mm_pause();
                spins++;
            }
            if (gen_.load(std::memory_order_acquire) == seen) {
                std::unique_lock<std::mutex> g(m_);
                cv_.wait(g, [&] { return gen_.load() != seen; });
            }
            seen = gen_.load(std::memory_order_acquire);
            if (stop_) return;
            run_chunks();
            remaining_.fetch_sub(1, std::memory_order_release);
        }
    }
    int n_;
    std::vector<std::thread> workers_;
    std::mutex m_;
    std::condition_variable cv_;
    std::atomic<uint64_t> gen_{0};
    bool stop_ = false;
    std::atomic<size_t> next_{0};
    std::atomic<int> remaining_{0};
    size_t n_items_ = 0, grain_ = 1;
    const std::function<void(size_t, size_t)>* job_ = nullptr;
};

Pool& pool_for(int threads) {
    static std::mutex m;
    static std::vector<Pool*> pools;
    std::lock_guard<std::mutex> g(m);
    for (Pool* p : pools)
        if (p->threads() == std::max(1, threads)) return *p;
    pools.push_back(new Pool(threads));
    return *pools.back();
}

// ------------------------------------------------- matrices (weights.rs:58-79)

enum Kind { KIND_BF16 = 0, KIND_Q8 = 1, KIND_Q4 = 2 };

struct MatrixView {
    int kind;
    size_t rows, cols;
    const void* scales;  // Q8: u16[rows*cols/32]; Q4: u32[rows*q4_words(cols)]; BF16: unused
    const void* data;    // BF16: u16[rows*cols]; Q8: i8[rows*cols]; Q4: u8[rows*cols/2]
};

// src/weights.rs:276-278
inline size_t q4_words(size_t cols) { return (cols / QK + SUPER - 1) / SUPER * SUPER_WORDS; }

// src/weights.rs:652-664
void quantize_input(Pool& pool, const float* x, size_t t, size_t cols, std::vector<float>& xs,
                    std::vector<int8_t>& xq) {
    size_t nb = cols / QK;
    xs.assign(t * nb, 0.0f);
    xq.assign(t * cols, 0);
    size_t grain = (t + pool.threads() - 1) / pool.threads();
    pool.parallel_for(t, grain, [&](size_t a, size_t b) {
        for (size_t i = a; i < b; i++)
            quantize_q8(x + i * cols, cols, xs.data() + i * nb, xq.data() + i * cols);
    });
}

// src/weights.rs:474-649, x86 arm: has_i8mm() is false (src/kernels.rs:709,
// 1458-1460), so rows never go through the paired-token kernels. What is left:
// t == 1 takes dot1 (scales converted as stored) and the packed offset dot;
// otherwise scales are expanded eight rows at a time, tokens go four per
// weight load through dot_x4, leftovers through dot, and offsets through the
// expanded offset dot.
void int_matmul(Pool& pool, const MatrixView& m, size_t row0, size_t rows, const float* x,
                size_t t, size_t grain, float* out) {
    const size_t cols = m.cols, nb = cols / QK;
    std::vector<float> xs;
    std::vector<int8_t> xq;
    quantize_input(pool, x, t, cols, xs, xq);
    const bool q4 = m.kind == KIND_Q4;
    const size_t padded = (nb + SUPER - 1) / SUPER * SUPER;
    std::vector<float> sums;
    if (q4) {
        sums.assign(t * padded, 0.0f);
        size_t g = (t + pool.threads() - 1) / pool.threads();
        pool.parallel_for(t, g, [&](size_t a, size_t b) {
            for (size_t i = a; i < b; i++)
                for (size_t blk = 0; blk < nb; blk++) {
                    size_t k = i * nb + blk;
                    int32_t q = 0;
                    for (int j = 0; j < QK; j++) q += int32_t(xq[k * QK + j]);
                    sums[i * padded + blk] = xs[k] * float(q);
                }
        });
    }
    const size_t stride = q4 ? padded : nb;
    const size_t words = q4_words(cols);
    const uint16_t* s8 = static_cast<const uint16_t*>(m.scales);
    const uint32_t* s4 = static_cast<const uint32_t*>(m.scales);
    const int8_t* q8 = static_cast<const int8_t*>(m.data);
    const uint8_t* q4d = static_cast<const uint8_t*>(m.data);

    if (g_arith == 1) {
        pool.parallel_for(rows, grain, [&](size_t ra, size_t rb) {
            std::vector<float> d(padded), c(padded);
            for (size_t r = ra; r < rb; r++) {
                size_t row = row0 + r;
                if (!q4)
                    for (size_t b = 0; b < nb; b++) d[b] = f16_finite(s8[row * nb + b]);
                else
                    unpack_q4(s4 + row * words, padded, d.data(), c.data());
                for (size_t i = 0; i < t; i++)
                    out[i * rows + r] =
                        q4 ? dot_q4_chain(d.data(), c.data(), nb, q4d + row * cols / 2,
                                          xs.data() + i * nb, xq.data() + i * cols,
                                          sums.data() + i * padded)
                           : dot_q8_chain(d.data(), nb, q8 + row * cols, xs.data() + i * nb,
                                          xq.data() + i * cols);
            }
        });
        return;
    }
    pool.parallel_for(rows, grain, [&](size_t ra, size_t rb) {
        if (t == 1) {
            for (size_t r = ra; r < rb; r++) {
                size_t row = row0 + r;
                float y;
                if (!q4) {
                    y = dot_q8_avx(HalfScales{s8 + row * nb}, nb, q8 + row * cols, xs.data(),
                                   xq.data());
                } else {
                    y = dot_q4_avx(PackedScales{s4 + row * words}, nb, q4d + row * cols / 2,
                                   xs.data(), xq.data());
                    y = y + dot_offsets(s4 + row * words, sums.data(), padded);
                }
                out[r] = y;
            }
            return;
        }
        constexpr size_t GROUP = 8;  // src/weights.rs:281
        std::vector<float> d(GROUP * stride, 0.0f), c(GROUP * stride, 0.0f);
        for (size_t g = ra; g < rb; g += GROUP) {
            size_t end = std::min(g + GROUP, rb);
            for (size_t r = g; r < end; r++) {
                size_t row = row0 + r;
                float* dr = d.data() + (r - g) * stride;
                float* cr = c.data() + (r - g) * stride;
                if (!q4) {
                    for (size_t b = 0; b < nb; b++) dr[b] = f16_finite(s8[row * nb + b]);
                } else {
                    // Whole super-blocks: packed bytes past the row's end are zero.
                    unpack_q4(s4 + row * words, padded, dr, cr);
                }
            }
            for (size_t r = g; r < end; r++) {
                size_t row = row0 + r;
                const float* dr = d.data() + (r - g) * stride;
                const float* cr = c.data() + (r - g) * stride;
                auto put = [&](size_t i, float y) {
                    if (q4) y = y + dot_offsets_expanded(cr, sums.data() + i * padded, padded);
                    out[i * rows + r] = y;
                };
                size_t i = 0;
                while (i + 4 <= t) {
                    const float* xsp[4];
                    const int8_t* xqp[4];
                    for (int j = 0; j < 4; j++) {
                        xsp[j] = xs.data() + (i + j) * nb;
                        xqp[j] = xq.data() + (i + j) * cols;
                    }
                    float ys[4];
                    if (!q4)
                        dot_q8_x4_avx(dr, nb, q8 + row * cols, xsp, xqp, ys);
                    else
                        dot_q4_x4_avx(dr, nb, q4d + row * cols / 2, xsp, xqp, ys);
                    for (int j = 0; j < 4; j++) put(i + j, ys[j]);
                    i += 4;
                }
                for (; i < t; i++) {
                    float y;
                    if (!q4)
                        y = dot_q8_avx(ExpandedScales{dr}, nb, q8 + row * cols, xs.data() + i * nb,
                                       xq.data() + i * cols);
                    else
                        y = dot_q4_avx(ExpandedScales{dr}, nb, q4d + row * cols / 2,
                                       xs.data() + i * nb, xq.data() + i * cols);
                    put(i, y);
                }
            }
        }
    });
}

// src/weights.rs:214-272: rows [row0, row0+rows) of m times t inputs.
void matmul_rows(Pool& pool, const MatrixView& m, const float* x, size_t t, float* out,
                 size_t row0, size_t rows) {
    // src/weights.rs:227: even, clamped grain.
    size_t grain = rows / (size_t(pool.threads()) * 8);
    grain = std::min<size_t>(256, std::max<size_t>(4, grain)) & ~size_t(1);
    if (m.kind == KIND_BF16) {
        const uint16_t* data = static_cast<const uint16_t*>(m.data);
        pool.parallel_for(rows, grain, [&](size_t a, size_t b) {
            for (size_t r = a; r < b; r++)
                for (size_t i = 0; i < t; i++)
                    out[i * rows + r] =
                        dot_bf16_avx(data + (row0 + r) * m.cols, x + i * m.cols, m.cols);
        });
        return;
    }
    int_matmul(pool, m, row0, rows, x, t, grain, out);
}

// src/model.rs:448-457. total_cmp on f32 orders by the sign-magnitude bits;
// ties go to the lower expert. Gates: softmax over the k kept, with libm expf.
inline int32_t total_key(float v) {
    int32_t b = int32_t(f32_bits(v));
    return b ^ int32_t(uint32_t(b >> 31) >> 1);
}

void route(const float* scores, size_t experts, size_t k, uint32_t* ids, float* gates) {
    std::vector<uint32_t> order(experts);
    for (size_t e = 0; e < experts; e++) order[e] = uint32_t(e);
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
        int32_t ka = total_key(scores[a]), kb = total_key(scores[b]);
        if (ka != kb) return ka > kb;
        return a < b;
    });
    k = std::min(k, experts);
    float mx = k ? scores[order[0]] : 0.0f;
    float sum = 0.0f;
    for (size_t j = 0; j < k; j++) sum += std::exp(scores[order[j]] - mx);
    for (size_t j = 0; j < k; j++) {
        ids[j] = order[j];
        gates[j] = std::exp(scores[order[j]] - mx) / sum;
    }
}

}  // namespace

// =================================================================== C ABI
// Plain pointers and sizes, for ctypes. Names carry the `to_` prefix
// ("tachyon oracle").

extern "C" {

uint16_t to_f32_to_bf16(float f) { return f32_to_bf16(f); }
uint16_t to_f32_to_f16(float f) { return f32_to_f16(f); }
float to_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
float to_f16_finite(uint16_t h) { return f16_finite(h); }
float to_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
float to_exp_scalar(float x) { return exp_scalar(x); }

void to_exp_many(const float* x, size_t n, float* out) {
    for (size_t i = 0; i < n; i++) out[i] = exp_scalar(x[i]);
}
void to_libm_exp_many(const float* x, size_t n, float* out) {
    for (size_t i = 0; i < n; i++) out[i] = std::exp(x[i]);
}

void to_quantize_q8(const float* x, size_t n, float* scales, int8_t* qs) {
    quantize_q8(x, n, scales, qs);
}
void to_quantize_q4(const float* x, size_t n, float* scales, uint8_t* qs) {
    quantize_q4(x, n, scales, qs);
}
void to_quantize_q8_weights(const float* x, size_t n, uint16_t* scales, int8_t* qs) {
    quantize_q8_weights(x, n, scales, qs);
}
size_t to_q4_words(size_t cols) { return q4_words(cols); }

// A whole matrix to packed 4-bit, rows spread over `threads`
// (src/weights.rs:108-126).
void to_quantize_q4_matrix(const float* data, size_t rows, size_t cols, const float* importance,
                           uint32_t* scales, uint8_t* qs, int threads) {
    size_t words = q4_words(cols);
    Pool& pool = pool_for(threads);
    pool.parallel_for(rows, 4, [&](size_t a, size_t b) {
        for (size_t r = a; r < b; r++)
            quantize_q4_packed(data + r * cols, cols, importance, scales + r * words,
                               qs + r * cols / 2);
    });
}
void to_unpack_q4(const uint32_t* packed, size_t nb, float* d, float* c) {
    unpack_q4(packed, nb, d, c);
}
void to_dequantize_q8(const float* scales, const int8_t* qs, size_t n, float* out) {
    dequantize_q8(scales, qs, n, out);
}
void to_dequantize_q4(const float* scales, const uint8_t* qs, size_t n, float* out) {
    dequantize_q4(scales, qs, n, out);
}

float to_dot_f32(const float* a, const float* b, size_t n) { return dot_f32_avx(a, b, n); }
float to_dot_bf16(const uint16_t* w, const float* x, size_t n) { return dot_bf16_avx(w, x, n); }
float to_dot_bf16_scalar(const uint16_t* w, const float* x, size_t n) {
    float s = 0.0f;
    for (size_t i = 0; i < n; i++) s += bf16_to_f32(w[i]) * x[i];
    return s;
}
float to_dot_q8(const float* ws, size_t nb, const int8_t* wq, const float* xs, const int8_t* xq) {
    return dot_q8_avx(ExpandedScales{ws}, nb, wq, xs, xq);
}
float to_dot_q8_half(const uint16_t* ws, size_t nb, const int8_t* wq, const float* xs,
                     const int8_t* xq) {
    return dot_q8_avx(HalfScales{ws}, nb, wq, xs, xq);
}
float to_dot_q4(const float* ws, size_t nb, const uint8_t* wq, const float* xs, const int8_t* xq) {
    return dot_q4_avx(ExpandedScales{ws}, nb, wq, xs, xq);
}
float to_dot_q4_packed(const uint32_t* words, size_t nb, const uint8_t* wq, const float* xs,
                       const int8_t* xq) {
    return dot_q4_avx(PackedScales{words}, nb, wq, xs, xq);
}
void to_dot_q8_x4(const float* ws, size_t nb, const int8_t* wq, const float* xs, const int8_t* xq,
                  size_t cols, float* out) {
    // xs: 4 rows of nb scales; xq: 4 rows of cols quants.
    const float* xsp[4];
    const int8_t* xqp[4];
    for (int j = 0; j < 4; j++) {
        xsp[j] = xs + j * nb;
        xqp[j] = xq + j * cols;
    }
    dot_q8_x4_avx(ws, nb, wq, xsp, xqp, out);
}
void to_dot_q4_x4(const float* ws, size_t nb, const uint8_t* wq, const float* xs, const int8_t* xq,
                  size_t cols, float* out) {
    const float* xsp[4];
    const int8_t* xqp[4];
    for (int j = 0; j < 4; j++) {
        xsp[j] = xs + j * nb;
        xqp[j] = xq + j * cols;
    }
    dot_q4_x4_avx(ws, nb, wq, xsp, xqp, out);
}
float to_dot_q8_scalar(const float* ws, size_t nb, const int8_t* wq, const float* xs,
                       const int8_t* xq) {
    return dot_q8_scalar(ws, nb, wq, xs, xq);
}
float to_dot_q4_scalar(const float* ws, size_t nb, const uint8_t* wq, const float* xs,
                       const int8_t* xq) {
    return dot_q4_scalar(ws, nb, wq, xs, xq);
}
float to_dot_offsets(const uint32_t* words, const float* sums, size_t padded) {
    return dot_offsets(words, sums, padded);
}
float to_dot_offsets_expanded(const float* c, const float* sums, size_t padded) {
    return dot_offsets_expanded(c, sums, padded);
}

void to_silu_mul(const float* g, const float* u, size_t n, float* out) { silu_mul(g, u, n, out); }
void to_rmsnorm(float* out, const float* x, const float* w, size_t n, float eps) {
    rmsnorm(out, x, w, n, eps);
}
void to_rmsnorm_rows(float* out, const float* x, const float* w, size_t t, size_t n, float eps) {
    for (size_t i = 0; i < t; i++) rmsnorm(out + i * n, x + i * n, w, n, eps);
}
void to_axpy(float* out, float a, const float* x, size_t n) { axpy(out, a, x, n); }

void to_route(const float* scores, size_t experts, size_t k, uint32_t* ids, float* gates) {
    route(scores, experts, k, ids, gates);
}

// Matrix::row_into (src/weights.rs:175-199): one row dequantized to f32.
void to_row_into(int kind, size_t rows, size_t cols, const void* scales, const void* data,
                 size_t r, float* out) {
    (void)rows;
    size_t nb = cols / QK;
    if (kind == KIND_BF16) {
        const uint16_t* d = static_cast<const uint16_t*>(data);
        for (size_t i = 0; i < cols; i++) out[i] = bf16_to_f32(d[r * cols + i]);
    } else if (kind == KIND_Q8) {
        const uint16_t* s = static_cast<const uint16_t*>(scales);
        std::vector<float> d(nb);
        for (size_t b = 0; b < nb; b++) d[b] = f16_finite(s[r * nb + b]);
        dequantize_q8(d.data(), static_cast<const int8_t*>(data) + r * cols, cols, out);
    } else {
        size_t w = q4_words(cols);
        std::vector<float> d(nb), c(nb);
        unpack_q4(static_cast<const uint32_t*>(scales) + r * w, nb, d.data(), c.data());
        dequantize_q4(d.data(), static_cast<const uint8_t*>(data) + r * cols / 2, cols, out);
        for (size_t b = 0; b < nb; b++)
            for (int j = 0; j < QK; j++) out[b * QK + j] += c[b];
    }
}

// Matrix::matmul_rows (src/weights.rs:214-272).
void to_matmul_rows(int kind, size_t rows_total, size_t cols, const void* scales, const void* data,
                    const float* x, size_t t, float* out, size_t row0, size_t rows, int threads) {
    MatrixView m{kind, rows_total, cols, scales, data};
    matmul_rows(pool_for(threads), m, x, t, out, row0, rows);
}

// quantize_input (src/weights.rs:652-664), exposed for the tests.
void to_quantize_input(const float* x, size_t t, size_t cols, float* xs, int8_t* xq) {
    for (size_t i = 0; i < t; i++)
        quantize_q8(x + i * cols, cols, xs + i * (cols / QK), xq + i * cols);
}

// The MoE block (src/model.rs:462-521) over normed inputs xb[t, hidden]:
// router matmul, route each token, then experts in ascending order, each over
// the tokens routed to it, outputs axpy'd into proj[t, hidden] (from zero).
// `router_bias` (may be null) is added to each token's logits before route():
// the reference router has none; the routing-skew workload adds one on both
// sides. Optional outputs (may be null): logits[t, experts], ids/gates
// [t, k] in descending score order, counts[experts].
void to_moe(size_t hidden, size_t experts, size_t k, size_t inter, const uint16_t* router_bf16,
            int gu_kind, const void* gu_scales, const void* gu_data, int dn_kind,
            const void* dn_scales, const void* dn_data, const float* xb, size_t t,
            const float* router_bias, float* proj, float* logits_out, uint32_t* ids_out,
            float* gates_out, uint32_t* counts_out, int threads) {
    Pool& pool = pool_for(threads);
    MatrixView router{KIND_BF16, experts, hidden, nullptr, router_bf16};
    MatrixView gu{gu_kind, experts * 2 * inter, hidden, gu_scales, gu_data};
    MatrixView dn{dn_kind, experts * hidden, inter, dn_scales, dn_data};

    std::vector<float> logits(t * experts, 0.0f);
    matmul_rows(pool, router, xb, t, logits.data(), 0, experts);
    if (router_bias)
        for (size_t i = 0; i < t; i++)
            for (size_t e = 0; e < experts; e++) logits[i * experts + e] += router_bias[e];
    if (logits_out) std::memcpy(logits_out, logits.data(), logits.size() * 4);

    struct Pick {
        size_t token;
        float gate;
    };
    std::vector<std::vector<Pick>> by_expert(experts);
    std::vector<uint32_t> ids(k);
    std::vector<float> gates(k);
    for (size_t i = 0; i < t; i++) {
        route(logits.data() + i * experts, experts, k, ids.data(), gates.data());
        for (size_t j = 0; j < k; j++) {
            by_expert[ids[j]].push_back({i, gates[j]});
            if (ids_out) ids_out[i * k + j] = ids[j];
            if (gates_out) gates_out[i * k + j] = gates[j];
        }
    }
    if (counts_out)
        for (size_t e = 0; e < experts; e++) counts_out[e] = uint32_t(by_expert[e].size());

    std::fill(proj, proj + t * hidden, 0.0f);
    std::vector<float> expert_in, gate_up, hid, expert_out;
    for (size_t e = 0; e < experts; e++) {
        const auto& tokens = by_expert[e];
        size_t m = tokens.size();
        if (m == 0) continue;
        expert_in.resize(m * hidden);
        for (size_t j = 0; j < m; j++)
            std::memcpy(expert_in.data() + j * hidden, xb + tokens[j].token * hidden, hidden * 4);
        gate_up.assign(m * 2 * inter, 0.0f);
        matmul_rows(pool, gu, expert_in.data(), m, gate_up.data(), e * 2 * inter, 2 * inter);
        hid.assign(m * inter, 0.0f);
        size_t grain = (m + 4 * pool.threads() - 1) / (4 * pool.threads());
        pool.parallel_for(m, grain, [&](size_t a, size_t b) {
            for (size_t j = a; j < b; j++)
                silu_mul(gate_up.data() + j * 2 * inter, gate_up.data() + j * 2 * inter + inter,
                         inter, hid.data() + j * inter);
        });
        expert_out.assign(m * hidden, 0.0f);
        matmul_rows(pool, dn, hid.data(), m, expert_out.data(), e * hidden, hidden);
        for (size_t j = 0; j < m; j++)
            axpy(proj + tokens[j].token * hidden, tokens[j].gate, expert_out.data() + j * hidden,
                 hidden);
    }
}

// The residual update the block's caller performs (src/model.rs:681).
void to_add_inplace(float* x, const float* p, size_t n) {
    for (size_t i = 0; i < n; i++) x[i] += p[i];
}

// 0 (default): the reference's arithmetic. 1: the model of the GPU's fast order.
void to_set_arith(int mode) { g_arith = mode; }

int to_default_threads() {
    // src/pool.rs:71-88 on Linux: all cores, less two when there are more than four.
    unsigned all = std::thread::hardware_concurrency();
    if (all == 0) all = 4;
    return all > 4 ? int(all) - 2 : int(all);
}

}  // extern "C"
