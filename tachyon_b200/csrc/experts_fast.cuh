// Building blocks of the bandwidth-oriented expert kernels, shared by the grouped
// kernels of experts_fast.cu and the one-kernel decode block (moe_decode.cu): the
// record layout of the re-tiled weights, the shared-memory operand loads, the
// warp-level int8 matrix instruction, and the per-record inner loop that keeps ONE
// fma chain per output over its row's blocks, in order:
//
//     acc = fma(float(sum_b), ws[row,b] * xs[token,b], acc)      b = 0, 1, ...
//
// (src/kernels_x86.rs:79-87 with the eight AVX lanes of a block folded into one
// exact integer; 4-bit rows add their offsets with a second chain,
// src/weights.rs:491-520.)
#pragma once

#include "experts_common.cuh"

namespace tc {

constexpr int F_KC = 256;         // columns per record
constexpr int F_NBC = F_KC / QK;  // blocks per record
constexpr int F_ROWS = 16;        // weight rows per unit (one m16 tile)

template <int KIND>
struct Rec {
    // 8-bit: 16 rows x (256 weights + 8 f16 scales).
    // 4-bit: 16 rows x (128 nibble bytes + words 0..3 of the super-block), then
    //        word 4 of each row.
    static constexpr int ROW_STRIDE = KIND == 1 ? F_KC + 16 : F_KC / 2 + 16;
    static constexpr int BYTES = KIND == 1 ? F_ROWS * ROW_STRIDE : F_ROWS * ROW_STRIDE + F_ROWS * 4;
};

// Shared-memory reads below are plain (non-volatile) asm so the compiler may
// interleave them across unrolled blocks; what keeps them behind the mbarrier
// wait that made their data visible is the `token` operand, a value that wait
// produced.
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t token, int& r0, int& r1, int& r2, int& r3) {
    asm("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4]; // %5"
        : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
        : "r"(addr), "r"(token));
}

__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t token, int& r0, int& r1) {
    asm("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2]; // %3" : "=r"(r0), "=r"(r1) : "r"(addr), "r"(token));
}

// D = A(16x32 s8, row) * B(32x8 s8, col) + c, s32 accumulate.
__device__ __forceinline__ void mma_s8(int (&d)[4], int a0, int a1, int a2, int a3, int b0, int b1,
                                       int c) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr, uint32_t token) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1]; // %2" : "=r"(v) : "r"(addr), "r"(token));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr, uint32_t token) {
    uint4 v;
    asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4]; // %5"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "r"(addr), "r"(token));
    return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t addr, uint32_t token) {
    float2 v;
    asm("ld.shared.v2.f32 {%0,%1}, [%2]; // %3" : "=f"(v.x), "=f"(v.y) : "r"(addr), "r"(token));
    return v;
}

// f16 bits of a weight scale to f32 (src/kernels.rs:127-130): one conversion
// instruction, exact for every half value.
__device__ __forceinline__ float f16_scale_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}

// One record (16 rows x up to 8 blocks) against G tiles of 8 staged tokens. The staged
// scales are transposed to [block][8 * GMAX tokens]; acc/off hold GMAX tiles.
template <int KIND, int G, int GMAX>
__device__ __forceinline__ void fast_chunk(uint32_t rec, uint32_t xq_s, uint32_t xsT_s, uint32_t xsumT_s,
                                           int x_stride, int nblk, int blk0, int lane, uint32_t wtok,
                                           uint32_t xtok, float (&acc)[GMAX][4],
                                           float (&off)[GMAX][4]) {
    using R = Rec<KIND>;
    const int g = lane >> 2, t = lane & 3;
    const int mat = lane >> 3, mr = lane & 7;
    // This thread's two rows' scales for the record's eight blocks.
    float wd[2][F_NBC], wc[2][F_NBC];
    if (KIND == 1) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint4 s = lds128(rec + (g + 8 * h) * R::ROW_STRIDE + F_KC, wtok);
            const uint32_t hw[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
            for (int b = 0; b < F_NBC; b += 2) {
                const uint32_t word = hw[b >> 1];
                wd[h][b] = f16_scale_to_f32(word & 0xFFFFu);
                wd[h][b + 1] = f16_scale_to_f32(word >> 16);
            }
        }
    } else {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint4 s = lds128(rec + (g + 8 * h) * R::ROW_STRIDE + F_KC / 2, wtok);
            const uint32_t o23 = lds32(rec + F_ROWS * R::ROW_STRIDE + (g + 8 * h) * 4, wtok);
            const float step_d = f16_bits_to_f32(uint16_t(s.x)), step_c = f16_bits_to_f32(uint16_t(s.x >> 16));
#pragma unroll
            for (int b = 0; b < F_NBC; b++) {
                wd[h][b] = step_d * float(((b < 4 ? s.y : s.z) >> (8 * (b & 3))) & 0xFFu);
                wc[h][b] = step_c * float(int(int8_t(uint8_t((b < 4 ? s.w : o23) >> (8 * (b & 3))))));
            }
        }
    }
    uint32_t a_addr;
    if (KIND == 1)
        a_addr = rec + (mr + (mat & 1) * 8) * R::ROW_STRIDE + (mat >> 1) * 16;
    else
        a_addr = rec + (mr + (mat & 1) * 8) * R::ROW_STRIDE;
    // B: token row (mr) of a tile, 16-byte half (mat & 1) of block b + (mat >> 1).
    const uint32_t b_addr = xq_s + mr * x_stride + blk0 * 32 + (mat & 1) * 16 + (mat >> 1) * 32;
    // Four blocks at a time, in three phases so that the loads, the matrix
    // instructions and the float chains of different blocks overlap: all
    // operand loads, then all matrix instructions, then the scaling.
#pragma unroll
    for (int h4 = 0; h4 < F_NBC; h4 += 4) {
        if (h4 < nblk) {
            int A[4][4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                if (KIND == 1) {
                    ldmatrix_x4(a_addr + (h4 + k) * 32, wtok, A[k][0], A[k][1], A[k][2], A[k][3]);
                } else {
                    // Word t of rows g and g+8: low nibbles are elements 4t..4t+3,
                    // high nibbles elements 16+4t..16+4t+3.
                    int w0, w1;
                    ldmatrix_x2(a_addr + (h4 + k) * 16, wtok, w0, w1);
                    A[k][0] = nibbles_minus8(uint32_t(w0) & 0x0F0F0F0Fu);
                    A[k][2] = nibbles_minus8((uint32_t(w0) >> 4) & 0x0F0F0F0Fu);
                    A[k][1] = nibbles_minus8(uint32_t(w1) & 0x0F0F0F0Fu);
                    A[k][3] = nibbles_minus8((uint32_t(w1) >> 4) & 0x0F0F0F0Fu);
                }
            }
#pragma unroll
            for (int n0 = 0; n0 < G; n0 += 2) {
                constexpr int PAIR = 2;
                int B[PAIR][4][2];
                float2 XS[PAIR][4], SU[PAIR][4];
#pragma unroll
                for (int p = 0; p < PAIR; p++) {
                    if (n0 + p < G) {
                        const uint32_t row = b_addr + (n0 + p) * 8 * x_stride + h4 * 32;
                        ldmatrix_x4(row, xtok, B[p][0][0], B[p][0][1], B[p][1][0], B[p][1][1]);
                        ldmatrix_x4(row + 64, xtok, B[p][2][0], B[p][2][1], B[p][3][0], B[p][3][1]);
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const uint32_t so = ((blk0 + h4 + k) * (8 * GMAX) + (n0 + p) * 8 + 2 * t) * 4;
                            XS[p][k] = lds_f2(xsT_s + so, xtok);
                            if (KIND == 2) SU[p][k] = lds_f2(xsumT_s + so, xtok);
                        }
                    }
                }
                int D[PAIR][4][4];
#pragma unroll
                for (int p = 0; p < PAIR; p++)
                    if (n0 + p < G) {
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            mma_s8(D[p][k], A[k][0], A[k][1], A[k][2], A[k][3], B[p][k][0], B[p][k][1], MAGIC_I);
                    }
#pragma unroll
                for (int p = 0; p < PAIR; p++)
                    if (n0 + p < G) {
                        const int nt = n0 + p;
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            if (h4 + k < nblk) {
                                const int b = h4 + k;
                                const float2 magic = make_float2(MAGIC_F, MAGIC_F);
#pragma unroll
                                for (int h = 0; h < 2; h++) {  // rows g and g+8; tokens 2t, 2t+1 side by side
                                    const float2 sum = sub2(make_float2(__int_as_float(D[p][k][2 * h]),
                                                                        __int_as_float(D[p][k][2 * h + 1])), magic);
                                    const float2 d = mul2(make_float2(wd[h][b], wd[h][b]), XS[p][k]);
                                    const float2 r = fma2(sum, d, make_float2(acc[nt][2 * h], acc[nt][2 * h + 1]));
                                    acc[nt][2 * h] = r.x;
                                    acc[nt][2 * h + 1] = r.y;
                                    if (KIND == 2) {
                                        const float2 o = fma2(make_float2(wc[h][b], wc[h][b]), SU[p][k],
                                                              make_float2(off[nt][2 * h], off[nt][2 * h + 1]));
                                        off[nt][2 * h] = o.x;
                                        off[nt][2 * h + 1] = o.y;
                                    }
                                }
                            }
                        }
                    }
            }
        }
    }
}

}  // namespace tc
