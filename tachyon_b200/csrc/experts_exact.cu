// Grouped expert products for decode-size groups: every selected expert's
// gate_up rows (with the SwiGLU epilogue) and down rows against the 8-bit
// activations of the tokens routed to it, over Tachyon's int8 and packed
// 4-bit weight layouts.
//
// Arithmetic: int_matmul's x86 arm (src/weights.rs:474-649) with the AVX2
// dots q8/q4 (src/kernels_x86.rs:79-129). For one (weight row, token) the CPU
// keeps eight float lanes; in each 32-block, lane j takes the exact integer
// sum of products of elements 4j..4j+3 (block_q8 / block_q4, lines 43-70),
// converts it to float and does acc_j = fma(sum_j, ws[b]*xs[b], acc_j); after
// the last block the lanes are added by the fixed hsum tree (33-38). Here one
// dp4a is exactly one lane's integer sum, so the same fma chain runs per lane
// and the result is bit-identical, whatever the batch size. 4-bit rows add the
// per-block offsets against the token's block sums (src/weights.rs:491-520,
// src/kernels.rs:392-432). SwiGLU is src/kernels.rs:595-603 with the
// polynomial exp of 544-564.
//
// Data movement: the kernel is persistent. Each warp owns 16 weight rows at a
// time and streams them through its own ring of shared-memory stages with
// bulk async copies (one copy per lane: 16 weight-row chunks, up to 8 token
// rows of int8 activations and their 8 scale rows), completion counted on an
// mbarrier per stage. Weight rows are padded in shared memory so that the
// 128-bit loads of a quarter-warp fall in distinct banks. Every wait on an
// mbarrier has a spin limit; a wait that runs out records
// ERR_COPY_WAIT_TIMEOUT in the status word and the warp stops.
#include "experts_common.cuh"

namespace tc {

namespace {

constexpr int EXP_WARPS = 8;
constexpr int EXP_THREADS = EXP_WARPS * 32;
constexpr int KC = 256;        // columns per staged chunk (one 4-bit super-block)
constexpr int NBC = KC / QK;   // blocks per chunk
constexpr int STAGES = 3;
constexpr int TOK = 8;         // tokens per group held in registers
constexpr int W_ROWS = 16;     // weight rows per warp

template <int KIND>
struct Stage {
    static constexpr int W_CHUNK = KIND == 1 ? KC : KC / 2;      // bytes per row chunk
    static constexpr int W_STRIDE = W_CHUNK + (KIND == 1 ? 32 : 16);
    static constexpr int W_BYTES = W_ROWS * W_STRIDE;
    static constexpr int X_BYTES = TOK * KC;
    static constexpr int XS_BYTES = TOK * NBC * 4;
    static constexpr int BYTES = W_BYTES + X_BYTES + XS_BYTES;
};

// Where a warp is in its sequence of (unit, token group, column chunk) steps.
struct Cursor {
    int unit, e, u, g0, c;
    uint32_t m, base;
    bool valid;
};

template <int KIND, bool GATE_UP>
struct Worker {
    const ExpertArgs& a;
    const int lane, nchunks, unit_stride, total_units;

    __device__ Worker(const ExpertArgs& args, int lane_, int stride)
        : a(args), lane(lane_), nchunks((args.cols + KC - 1) / KC), unit_stride(stride),
          total_units(args.experts * args.units_per_expert) {}

    __device__ void seek(Cursor& cur) const {
        // Moves to the first unit at or after cur.unit whose expert has tokens.
        while (cur.unit < total_units) {
            int e = cur.unit / a.units_per_expert;
            uint32_t m = a.counts[e];
            if (m > 0) {
                cur.e = e;
                cur.u = cur.unit - e * a.units_per_expert;
                cur.m = m;
                cur.base = a.offsets[e];
                cur.g0 = 0;
                cur.c = 0;
                cur.valid = true;
                return;
            }
            cur.unit += unit_stride;
        }
        cur.valid = false;
    }

    __device__ void advance(Cursor& cur) const {
        if (++cur.c < nchunks) return;
        cur.c = 0;
        cur.g0 += TOK;
        if (uint32_t(cur.g0) < cur.m) return;
        cur.unit += unit_stride;
        seek(cur);
    }

    // The matrix row weight-lane r (0..15) of a unit works on, or -1.
    __device__ int matrix_row(const Cursor& cur, int r) const {
        if (GATE_UP) {
            const int inter = a.rows_per_expert / 2;
            const int col = cur.u * 8 + (r & 7);
            if (col >= inter) return -1;
            return cur.e * a.rows_per_expert + (r < 8 ? 0 : inter) + col;
        }
        const int row = cur.u * W_ROWS + r;
        if (row >= a.rows_per_expert) return -1;
        return cur.e * a.rows_per_expert + row;
    }

    // The activation row of token j of the cursor's group.
    __device__ uint32_t act_row(const Cursor& cur, int j) const {
        const uint32_t p = cur.base + cur.g0 + j;
        return GATE_UP ? a.slot_token[p] : p;
    }

    __device__ void fill(uint8_t* stage, uint64_t* bar, const Cursor& cur) const {
        using S = Stage<KIND>;
        const int col0 = cur.c * KC;
        const int cols_c = min(KC, a.cols - col0);
        const int ntok = min(TOK, int(cur.m) - cur.g0);
        const uint32_t wbytes = KIND == 1 ? cols_c : cols_c / 2;
        const int nbp = (a.cols / QK + SUPER - 1) / SUPER * SUPER;
        int row = -1;
        if (lane < W_ROWS) row = matrix_row(cur, lane);
        const unsigned rows_mask = __ballot_sync(0xffffffffu, row >= 0);
        if (lane == 0) {
            uint32_t total = __popc(rows_mask) * wbytes + ntok * (cols_c + NBC * 4);
            mbar_expect_tx(bar, total);
        }
        __syncwarp();
        if (lane < W_ROWS) {
            if (row >= 0) {
                const uint8_t* src = a.wdata + (KIND == 1 ? size_t(row) * a.cols + col0
                                                          : (size_t(row) * a.cols + col0) / 2);
                bulk_copy(stage + lane * S::W_STRIDE, src, wbytes, bar);
            }
        } else if (lane < W_ROWS + TOK) {
            const int j = lane - W_ROWS;
            if (j < ntok) {
                const int8_t* src = a.xq + size_t(act_row(cur, j)) * a.cols + col0;
                bulk_copy(stage + S::W_BYTES + j * KC, src, cols_c, bar);
            }
        } else {
            const int j = lane - W_ROWS - TOK;
            if (j < ntok) {
                const float* src = a.xs + size_t(act_row(cur, j)) * nbp + cur.c * NBC;
                bulk_copy(stage + S::W_BYTES + S::X_BYTES + j * NBC * 4, src, NBC * 4, bar);
            }
        }
    }
};

// One staged chunk against T tokens: the per-lane fma chains.
template <int KIND, int T>
__device__ __forceinline__ void compute_chunk(const uint8_t* stage, int nblk, int r, int q,
                                              const float (&wsf)[NBC], float (&acc)[TOK][4]) {
    using S = Stage<KIND>;
    const uint8_t* wrow = stage + r * S::W_STRIDE;
    const uint8_t* xbase = stage + S::W_BYTES;
    const float* xsb = reinterpret_cast<const float*>(stage + S::W_BYTES + S::X_BYTES);
#pragma unroll
    for (int b = 0; b < NBC; b++) {
        if (b < nblk) {
            int w0, w1, w2, w3;
            if (KIND == 1) {
                const int4 w = *reinterpret_cast<const int4*>(wrow + b * 32 + q * 16);
                w0 = w.x, w1 = w.y, w2 = w.z, w3 = w.w;
            } else {
                // Bytes 8q..8q+7 of the block: low nibbles are elements
                // 8q..8q+7, high nibbles elements 16+8q..16+8q+7.
                const uint2 w = *reinterpret_cast<const uint2*>(wrow + b * 16 + q * 8);
                w0 = nibbles_minus8(w.x & 0x0F0F0F0Fu);
                w1 = nibbles_minus8(w.y & 0x0F0F0F0Fu);
                w2 = nibbles_minus8((w.x >> 4) & 0x0F0F0F0Fu);
                w3 = nibbles_minus8((w.y >> 4) & 0x0F0F0F0Fu);
            }
#pragma unroll
            for (int j = 0; j < T; j++) {
                int x0, x1, x2, x3;
                if (KIND == 1) {
                    const int4 x = *reinterpret_cast<const int4*>(xbase + j * KC + b * 32 + q * 16);
                    x0 = x.x, x1 = x.y, x2 = x.z, x3 = x.w;
                } else {
                    const int2 lo = *reinterpret_cast<const int2*>(xbase + j * KC + b * 32 + q * 8);
                    const int2 hi =
                        *reinterpret_cast<const int2*>(xbase + j * KC + b * 32 + 16 + q * 8);
                    x0 = lo.x, x1 = lo.y, x2 = hi.x, x3 = hi.y;
                }
                const float d = wsf[b] * xsb[j * NBC + b];
                acc[j][0] = fmaf(lane_sum(w0, x0), d, acc[j][0]);
                acc[j][1] = fmaf(lane_sum(w1, x1), d, acc[j][1]);
                acc[j][2] = fmaf(lane_sum(w2, x2), d, acc[j][2]);
                acc[j][3] = fmaf(lane_sum(w3, x3), d, acc[j][3]);
            }
        }
    }
}

// The hsum tree over the eight lanes two partner threads hold between them.
template <int KIND>
__device__ __forceinline__ float finish_row(const float (&a)[4]) {
    if (KIND == 1) {
        // This thread: lanes 4q..4q+3; the partner: the other four.
        float s0 = a[0] + __shfl_xor_sync(0xffffffffu, a[0], 1);
        float s1 = a[1] + __shfl_xor_sync(0xffffffffu, a[1], 1);
        float s2 = a[2] + __shfl_xor_sync(0xffffffffu, a[2], 1);
        float s3 = a[3] + __shfl_xor_sync(0xffffffffu, a[3], 1);
        return (s0 + s2) + (s1 + s3);
    }
    // q = 0 holds lanes 0,1,4,5; q = 1 holds 2,3,6,7.
    float p0 = a[0] + a[2];  // lane + (lane+4)
    float p1 = a[1] + a[3];
    float o0 = __shfl_xor_sync(0xffffffffu, p0, 1);
    float o1 = __shfl_xor_sync(0xffffffffu, p1, 1);
    return (p0 + o0) + (p1 + o1);
}

template <int KIND, bool GATE_UP>
__global__ void __launch_bounds__(EXP_THREADS, 1) expert_kernel(const ExpertArgs a) {
    using S = Stage<KIND>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* stages = smem + size_t(warp) * STAGES * S::BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + size_t(EXP_WARPS) * STAGES * S::BYTES) +
                     warp * STAGES;
    if (lane == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(bars + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    const int r = lane >> 1, q = lane & 1;
    Worker<KIND, GATE_UP> wk(a, lane, int(gridDim.x) * EXP_WARPS);
    Cursor prod;
    prod.unit = warp * int(gridDim.x) + int(blockIdx.x);
    wk.seek(prod);
    Cursor cons = prod;

    uint32_t fills = 0, takes = 0;
    for (int s = 0; s < STAGES - 1 && prod.valid; s++) {
        wk.fill(stages + (fills % STAGES) * S::BYTES, bars + fills % STAGES, prod);
        fills++;
        wk.advance(prod);
    }

    float acc[TOK][4];
    const int nb = a.cols / QK;
    const int words_per_row = (nb + SUPER - 1) / SUPER * SUPER_WORDS;
    bool ok = true;
    while (cons.valid) {
        if (prod.valid) {
            wk.fill(stages + (fills % STAGES) * S::BYTES, bars + fills % STAGES, prod);
            fills++;
            wk.advance(prod);
        }
        // This thread's weight row scales for the chunk, fetched before the wait.
        const int row = wk.matrix_row(cons, r);
        const int nblk = min(NBC, nb - cons.c * NBC);
        float wsf[NBC];
        if (row >= 0) {
            if (KIND == 1) {
                const uint16_t* sp =
                    reinterpret_cast<const uint16_t*>(a.wscales) + size_t(row) * nb + cons.c * NBC;
                if ((nb & 7) == 0) {
                    const uint4 h = *reinterpret_cast<const uint4*>(sp);
                    const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
                    for (int b = 0; b < NBC; b++)
                        wsf[b] = f16_bits_to_f32(uint16_t(hw[b >> 1] >> (16 * (b & 1))));
                } else {
#pragma unroll
                    for (int b = 0; b < NBC; b++) wsf[b] = b < nblk ? f16_bits_to_f32(sp[b]) : 0.0f;
                }
            } else {
                const uint32_t* wp = reinterpret_cast<const uint32_t*>(a.wscales) +
                                     size_t(row) * words_per_row + cons.c * SUPER_WORDS;
                const float step = f16_bits_to_f32(uint16_t(wp[0]));
                const uint32_t s01 = wp[1], s23 = wp[2];
#pragma unroll
                for (int b = 0; b < NBC; b++)
                    wsf[b] = step * float((b < 4 ? s01 : s23) >> (8 * (b & 3)) & 0xFFu);
            }
        } else {
#pragma unroll
            for (int b = 0; b < NBC; b++) wsf[b] = 0.0f;
        }
        if (cons.c == 0) {
#pragma unroll
            for (int j = 0; j < TOK; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
        }
        const uint32_t stage = takes % STAGES;
        const bool landed = mbar_wait_bounded(bars + stage, (takes / STAGES) & 1);
        if (!__all_sync(0xffffffffu, landed)) {
            ok = false;
            break;
        }
        const int ntok = min(TOK, int(cons.m) - cons.g0);
        const uint8_t* st = stages + stage * S::BYTES;
        if (ntok == 1)
            compute_chunk<KIND, 1>(st, nblk, r, q, wsf, acc);
        else if (ntok == 2)
            compute_chunk<KIND, 2>(st, nblk, r, q, wsf, acc);
        else if (ntok <= 4)
            compute_chunk<KIND, 4>(st, nblk, r, q, wsf, acc);
        else
            compute_chunk<KIND, 8>(st, nblk, r, q, wsf, acc);
        __syncwarp();

        if (cons.c == wk.nchunks - 1) {
            const int nbp = (nb + SUPER - 1) / SUPER * SUPER;
#pragma unroll
            for (int j = 0; j < TOK; j++) {
                if (j < ntok) {  // uniform across the warp
                    float y = finish_row<KIND>(acc[j]);
                    if (KIND == 2 && row >= 0) {
                        const uint32_t* words = reinterpret_cast<const uint32_t*>(a.wscales) +
                                                size_t(row) * words_per_row;
                        const float* sums = a.xsum + size_t(wk.act_row(cons, j)) * nbp;
                        y = y + offset_dot(words, sums, nbp / SUPER);
                    }
                    const uint32_t p = cons.base + cons.g0 + j;
                    if (GATE_UP) {
                        const float up = __shfl_down_sync(0xffffffffu, y, 16);
                        if (lane < 16 && q == 0 && row >= 0) {
                            const float e = exp_poly(-y);
                            const float h = __fdiv_rn(y, 1.0f + e) * up;
                            a.out[size_t(p) * a.out_cols + cons.u * 8 + r] = h;
                        }
                    } else if (q == 0 && row >= 0) {
                        a.out[size_t(p) * a.out_cols + cons.u * W_ROWS + r] = y;
                    }
                }
            }
        }
        takes++;
        wk.advance(cons);
    }
    if (!ok) {
        if (lane == 0) atomicExch(a.status, ERR_COPY_WAIT_TIMEOUT);
        // Give copies already in flight a bounded chance to land before the
        // shared memory they target is released.
        for (uint32_t k = takes; k < fills; k++) mbar_wait_bounded(bars + k % STAGES, (k / STAGES) & 1);
    }
}

template <int KIND>
constexpr size_t expert_smem_bytes() {
    return size_t(EXP_WARPS) * STAGES * Stage<KIND>::BYTES + EXP_WARPS * STAGES * sizeof(uint64_t);
}

template <int KIND, bool GATE_UP>
void launch_expert(const ExpertArgs& a, int sms, cudaStream_t stream) {
    using S = Stage<KIND>;
    const size_t smem = expert_smem_bytes<KIND>();
    const int total_units = a.experts * a.units_per_expert;
    int grid = min(sms, (total_units + EXP_WARPS - 1) / EXP_WARPS);
    if (grid < 1) grid = 1;
    expert_kernel<KIND, GATE_UP><<<grid, EXP_THREADS, smem, stream>>>(a);
}

// A warp per (sorted slot, 32-block) of the SwiGLU output: quantize_q8
// (src/kernels.rs:84-98), as the down projection's quantize_input does per
// gathered row (src/weights.rs:652-664).
__global__ void quant_hidden_kernel(const float* __restrict__ h, const uint32_t* __restrict__ offsets,
                                    int experts, int inter, int8_t* __restrict__ hq,
                                    float* __restrict__ hs, float* __restrict__ hsum) {
    const int nb = inter / QK;
    const int padded = (nb + SUPER - 1) / SUPER * SUPER;
    const uint32_t slots = offsets[experts];
    const int lane = threadIdx.x & 31;
    const size_t warp = size_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const size_t nwarps = size_t(gridDim.x) * (blockDim.x >> 5);
    for (size_t w = warp; w < size_t(slots) * padded; w += nwarps) {
        const size_t slot = w / padded;
        const int b = int(w - slot * padded);
        if (b >= nb) {
            if (lane == 0) {
                hs[slot * padded + b] = 0.0f;
                hsum[slot * padded + b] = 0.0f;
            }
            continue;
        }
        const float v = h[slot * inter + b * QK + lane];
        float amax = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        const float rr = roundf(v * id);
        const int qv = (rr != rr) ? 0 : int(fminf(127.0f, fmaxf(-128.0f, rr)));
        hq[slot * inter + b * QK + lane] = int8_t(qv);
        int qsum = qv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
        if (lane == 0) {
            hs[slot * padded + b] = d;
            hsum[slot * padded + b] = d * float(qsum);
        }
    }
}

}  // namespace

void init_kernels_exact() {
    cudaFuncSetAttribute(expert_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         int(expert_smem_bytes<1>()));
    cudaFuncSetAttribute(expert_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         int(expert_smem_bytes<1>()));
    cudaFuncSetAttribute(expert_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         int(expert_smem_bytes<2>()));
    cudaFuncSetAttribute(expert_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         int(expert_smem_bytes<2>()));
}

int launch_gate_up_exact(const MoeDims& d, const MatrixDev& m, int t, Workspace& ws, int sms,
                         cudaStream_t stream) {
    (void)t;
    const ExpertArgs a = gate_up_args(d, m, ws);
    if (m.kind == 1)
        launch_expert<1, true>(a, sms, stream);
    else
        launch_expert<2, true>(a, sms, stream);
    return 1;
}

int launch_quant_hidden(const MoeDims& d, int t, Workspace& ws, cudaStream_t stream) {
    const int nb = d.inter / QK;
    const int padded = (nb + SUPER - 1) / SUPER * SUPER;
    const size_t warps = size_t(t) * d.topk * padded;
    int blocks = int(warps + 7) / 8 < 148 * 16 ? int((warps + 7) / 8) : 148 * 16;
    if (blocks < 1) blocks = 1;
    quant_hidden_kernel<<<blocks, 256, 0, stream>>>(ws.hidden_f, ws.offsets, d.experts, d.inter,
                                                    ws.hq, ws.hs, ws.hsum);
    return 1;
}

int launch_down_exact(const MoeDims& d, const MatrixDev& m, int t, Workspace& ws, int sms,
                      cudaStream_t stream) {
    (void)t;
    const ExpertArgs a = down_args(d, m, ws);
    if (m.kind == 1)
        launch_expert<1, false>(a, sms, stream);
    else
        launch_expert<2, false>(a, sms, stream);
    return 1;
}

}  // namespace tc
