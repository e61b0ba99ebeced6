// Grouped expert products, fast path for decode-size groups: the integer sum of
// each 32-element block comes from one warp-level int8 matrix instruction
// (16 weight rows x 8 tokens x 32 deep = exactly one quantization block), and
// each output keeps ONE fma chain over its row's blocks, in order:
//
//     acc = fma(float(sum_b), ws[row,b] * xs[token,b], acc)      b = 0, 1, ...
//
// That is the sum Tachyon's CPU path computes (src/kernels_x86.rs:79-87) with
// the eight AVX lanes of a block folded into one exact integer before the
// float work, so it differs from the CPU result only in float rounding
// (~1e-7 relative); and because every fast path uses this same chain, a token's
// result does not depend on how many tokens share its expert. 4-bit rows add
// their per-block offsets with a second chain in the same loop:
// off = fma(c[row,b], xs[token,b]*sum(xq), off) (src/weights.rs:491-520).
//
// This kernel is bound by HBM, not by the tensor pipe: at decode sizes every
// selected expert's weights are read once and used for a handful of tokens.
// So the design is about bytes in flight. Persistent CTAs, one per SM; the
// units of work (16 weight rows of an expert with tokens) are cut into equal
// contiguous ranges per CTA; each warp streams its units' rows through a deep
// private ring of shared-memory stages with bulk async copies (one 256-byte
// row chunk per lane) counted on an mbarrier per stage. Rows are padded by 16
// bytes in shared memory so ldmatrix reads hit 32 distinct banks. Activations
// are tiny and shared by every warp working on the expert: they are read
// through L1. Every mbarrier wait has a spin limit.
#include "experts_common.cuh"

namespace tc {

namespace {

constexpr int F_WARPS = 8;
constexpr int F_THREADS = F_WARPS * 32;
constexpr int F_KC = 256;         // columns per staged chunk
constexpr int F_NBC = F_KC / QK;  // blocks per chunk
constexpr int F_ROWS = 16;        // weight rows per unit (one m16 tile)
constexpr int F_GMAX = 4;         // token tiles of 8 held in registers (32 tokens)

template <int KIND>
struct FStage {
    static constexpr int W_CHUNK = KIND == 1 ? F_KC : F_KC / 2;
    static constexpr int W_STRIDE = W_CHUNK + 16;
    static constexpr int BYTES = F_ROWS * W_STRIDE;
    static constexpr int STAGES = KIND == 1 ? 6 : 10;
};

template <int KIND>
constexpr size_t fast_smem_bytes() {
    return size_t(F_WARPS) * FStage<KIND>::STAGES * FStage<KIND>::BYTES +
           size_t(F_WARPS) * FStage<KIND>::STAGES * sizeof(uint64_t) + MAX_EXPERTS * sizeof(int) + 16;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, int& r0, int& r1, int& r2, int& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, int& r0, int& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
                 : "=r"(r0), "=r"(r1)
                 : "r"(addr));
}

// D = A(16x32 s8, row) * B(32x8 s8, col) + C, s32 accumulate.
__device__ __forceinline__ void mma_s8(int (&d)[4], int a0, int a1, int a2, int a3, int b0, int b1,
                                       int c) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}

struct FCursor {
    int a;        // index in the space of active units
    int e, u;     // expert, unit within the expert
    int sg0, c;   // first token of the 32-token super-group, column chunk
    uint32_t m, base;
    bool valid;
};

template <int KIND, bool GATE_UP>
struct FWorker {
    const ExpertArgs& a;
    const int* active;  // shared: experts with tokens, ascending
    const int lane, nchunks, hi;

    __device__ FWorker(const ExpertArgs& args, const int* act, int lane_, int hi_)
        : a(args), active(act), lane(lane_), nchunks((args.cols + F_KC - 1) / F_KC), hi(hi_) {}

    __device__ void seek(FCursor& cur) const {
        if (cur.a >= hi) {
            cur.valid = false;
            return;
        }
        const int ai = cur.a / a.units_per_expert;
        cur.e = active[ai];
        cur.u = cur.a - ai * a.units_per_expert;
        cur.m = a.counts[cur.e];
        cur.base = a.offsets[cur.e];
        cur.sg0 = 0;
        cur.c = 0;
        cur.valid = true;
    }

    __device__ void advance(FCursor& cur) const {
        if (++cur.c < nchunks) return;
        cur.c = 0;
        cur.sg0 += 8 * F_GMAX;
        if (uint32_t(cur.sg0) < cur.m) return;
        cur.a += F_WARPS;
        seek(cur);
    }

    // Matrix row of tile row r (0..15), or -1 past the expert's last row.
    __device__ int matrix_row(const FCursor& cur, int r) const {
        if (GATE_UP) {
            const int inter = a.rows_per_expert / 2;
            const int col = cur.u * 8 + (r & 7);
            if (col >= inter) return -1;
            return cur.e * a.rows_per_expert + (r < 8 ? 0 : inter) + col;
        }
        const int row = cur.u * F_ROWS + r;
        if (row >= a.rows_per_expert) return -1;
        return cur.e * a.rows_per_expert + row;
    }

    // Activation row of the expert's j-th token (clamped to its last one).
    __device__ uint32_t act_row(const FCursor& cur, int j) const {
        const uint32_t p = cur.base + min(uint32_t(j), cur.m - 1);
        return GATE_UP ? a.perm[p] / uint32_t(a.topk) : p;
    }

    __device__ void fill(uint8_t* stage, uint64_t* bar, const FCursor& cur) const {
        using S = FStage<KIND>;
        const int col0 = cur.c * F_KC;
        const int cols_c = min(F_KC, a.cols - col0);
        const uint32_t wbytes = KIND == 1 ? cols_c : cols_c / 2;
        int row = -1;
        if (lane < F_ROWS) row = matrix_row(cur, lane);
        const unsigned rows_mask = __ballot_sync(0xffffffffu, row >= 0);
        if (lane == 0) mbar_expect_tx(bar, __popc(rows_mask) * wbytes);
        __syncwarp();
        if (row >= 0) {
            const uint8_t* src = a.wdata + (KIND == 1 ? size_t(row) * a.cols + col0
                                                      : (size_t(row) * a.cols + col0) / 2);
            bulk_copy(stage + lane * S::W_STRIDE, src, wbytes, bar);
        }
    }
};

// Per-chunk weight-side scales of the two rows (g, g+8) a thread accumulates.
struct RowScales {
    float d[2][F_NBC];  // block scale
    float c[2][F_NBC];  // 4-bit block offset (unused for 8-bit)
};

template <int KIND>
__device__ __forceinline__ void load_row_scales(const ExpertArgs& a, int row, int nb, int chunk,
                                                int nblk, float (&d)[F_NBC], float (&c)[F_NBC]) {
    if (row < 0) {
#pragma unroll
        for (int b = 0; b < F_NBC; b++) d[b] = c[b] = 0.0f;
        return;
    }
    if (KIND == 1) {
        const uint16_t* sp = reinterpret_cast<const uint16_t*>(a.wscales) + size_t(row) * nb + chunk * F_NBC;
        if ((nb & 7) == 0) {
            const uint4 h = *reinterpret_cast<const uint4*>(sp);
            const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
            for (int b = 0; b < F_NBC; b++) d[b] = f16_bits_to_f32(uint16_t(hw[b >> 1] >> (16 * (b & 1))));
        } else {
#pragma unroll
            for (int b = 0; b < F_NBC; b++) d[b] = b < nblk ? f16_bits_to_f32(sp[b]) : 0.0f;
        }
    } else {
        const int words_per_row = (nb + SUPER - 1) / SUPER * SUPER_WORDS;
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(a.wscales) + size_t(row) * words_per_row +
                             chunk * SUPER_WORDS;
        const uint32_t w0 = wp[0], s01 = wp[1], s23 = wp[2], o01 = wp[3], o23 = wp[4];
        const float step_d = f16_bits_to_f32(uint16_t(w0)), step_c = f16_bits_to_f32(uint16_t(w0 >> 16));
#pragma unroll
        for (int b = 0; b < F_NBC; b++) {
            d[b] = step_d * float(((b < 4 ? s01 : s23) >> (8 * (b & 3))) & 0xFFu);
            c[b] = step_c * float(int(int8_t(uint8_t((b < 4 ? o01 : o23) >> (8 * (b & 3))))));
        }
    }
}

// One staged chunk of 16 weight rows against G tiles of 8 tokens.
template <int KIND, int G>
__device__ __forceinline__ void fast_chunk(const ExpertArgs& a, uint32_t stage_addr, int nblk, int lane,
                                           int col0, int nbp, int chunk, const RowScales& rs,
                                           const uint32_t (&rowB)[F_GMAX],
                                           const uint32_t (&rowC)[F_GMAX][2], float (&acc)[F_GMAX][4],
                                           float (&off)[F_GMAX][4]) {
    using S = FStage<KIND>;
    const int t = lane & 3;
    // ldmatrix row addresses: matrix = lane/8, row-in-matrix = lane%8.
    const int mat = lane >> 3, mr = lane & 7;
    uint32_t a_addr;
    if (KIND == 1)
        a_addr = stage_addr + (mr + (mat & 1) * 8) * S::W_STRIDE + (mat >> 1) * 16;
    else
        a_addr = stage_addr + (mr + (mat & 1) * 8) * S::W_STRIDE;
#pragma unroll
    for (int b = 0; b < F_NBC; b++) {
        if (b < nblk) {
            int a0, a1, a2, a3;
            if (KIND == 1) {
                ldmatrix_x4(a_addr + b * 32, a0, a1, a2, a3);
            } else {
                // Word t of rows g and g+8: low nibbles are elements 4t..4t+3,
                // high nibbles elements 16+4t..16+4t+3.
                int w0, w1;
                ldmatrix_x2(a_addr + b * 16, w0, w1);
                a0 = nibbles_minus8(uint32_t(w0) & 0x0F0F0F0Fu);
                a2 = nibbles_minus8((uint32_t(w0) >> 4) & 0x0F0F0F0Fu);
                a1 = nibbles_minus8(uint32_t(w1) & 0x0F0F0F0Fu);
                a3 = nibbles_minus8((uint32_t(w1) >> 4) & 0x0F0F0F0Fu);
            }
#pragma unroll
            for (int nt = 0; nt < G; nt++) {
                const int8_t* xrow = a.xq + size_t(rowB[nt]) * a.cols + col0 + b * 32 + 4 * t;
                const int b0 = *reinterpret_cast<const int*>(xrow);
                const int b1 = *reinterpret_cast<const int*>(xrow + 16);
                int d[4];
                mma_s8(d, a0, a1, a2, a3, b0, b1, MAGIC_I);
                const float xs0 = a.xs[size_t(rowC[nt][0]) * nbp + chunk * F_NBC + b];
                const float xs1 = a.xs[size_t(rowC[nt][1]) * nbp + chunk * F_NBC + b];
                acc[nt][0] = fmaf(__int_as_float(d[0]) - MAGIC_F, rs.d[0][b] * xs0, acc[nt][0]);
                acc[nt][1] = fmaf(__int_as_float(d[1]) - MAGIC_F, rs.d[0][b] * xs1, acc[nt][1]);
                acc[nt][2] = fmaf(__int_as_float(d[2]) - MAGIC_F, rs.d[1][b] * xs0, acc[nt][2]);
                acc[nt][3] = fmaf(__int_as_float(d[3]) - MAGIC_F, rs.d[1][b] * xs1, acc[nt][3]);
                if (KIND == 2) {
                    const float su0 = a.xsum[size_t(rowC[nt][0]) * nbp + chunk * F_NBC + b];
                    const float su1 = a.xsum[size_t(rowC[nt][1]) * nbp + chunk * F_NBC + b];
                    off[nt][0] = fmaf(rs.c[0][b], su0, off[nt][0]);
                    off[nt][1] = fmaf(rs.c[0][b], su1, off[nt][1]);
                    off[nt][2] = fmaf(rs.c[1][b], su0, off[nt][2]);
                    off[nt][3] = fmaf(rs.c[1][b], su1, off[nt][3]);
                }
            }
        }
    }
}

template <int KIND, bool GATE_UP>
__global__ void __launch_bounds__(F_THREADS, 1) expert_fast_kernel(const ExpertArgs a) {
    using S = FStage<KIND>;
    constexpr int STAGES = S::STAGES;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* stages = smem + size_t(warp) * STAGES * S::BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + size_t(F_WARPS) * STAGES * S::BYTES) + warp * STAGES;
    int* s_active = reinterpret_cast<int*>(smem + size_t(F_WARPS) * STAGES * (S::BYTES + sizeof(uint64_t)));
    int* s_nactive = s_active + MAX_EXPERTS;
    if (lane == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(bars + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // Experts with tokens, in ascending order (warp 0).
    if (warp == 0) {
        int n = 0;
        for (int e0 = 0; e0 < a.experts; e0 += 32) {
            const int e = e0 + lane;
            const bool on = e < a.experts && a.counts[e] > 0;
            const unsigned ballot = __ballot_sync(0xffffffffu, on);
            if (on) s_active[n + __popc(ballot & ((1u << lane) - 1u))] = e;
            n += __popc(ballot);
        }
        if (lane == 0) *s_nactive = n;
    }
    __syncthreads();
    const int total = *s_nactive * a.units_per_expert;
    const int lo = int((long long)blockIdx.x * total / gridDim.x);
    const int hi = int((long long)(blockIdx.x + 1) * total / gridDim.x);

    FWorker<KIND, GATE_UP> wk(a, s_active, lane, hi);
    FCursor prod;
    prod.a = lo + warp;
    wk.seek(prod);
    FCursor cons = prod;

    uint32_t fills = 0, takes = 0;
    for (int s = 0; s < STAGES - 1 && prod.valid; s++) {
        wk.fill(stages + (fills % STAGES) * S::BYTES, bars + fills % STAGES, prod);
        fills++;
        wk.advance(prod);
    }

    const int g = lane >> 2, t = lane & 3;
    const int nb = a.cols / QK;
    const int nbp = (nb + SUPER - 1) / SUPER * SUPER;
    float acc[F_GMAX][4], off[F_GMAX][4];
    uint32_t rowB[F_GMAX], rowC[F_GMAX][2];
    bool ok = true;
    while (cons.valid) {
        if (prod.valid) {
            wk.fill(stages + (fills % STAGES) * S::BYTES, bars + fills % STAGES, prod);
            fills++;
            wk.advance(prod);
        }
        const int row0 = wk.matrix_row(cons, g), row1 = wk.matrix_row(cons, g + 8);
        const int nblk = min(F_NBC, nb - cons.c * F_NBC);
        RowScales rs;
        load_row_scales<KIND>(a, row0, nb, cons.c, nblk, rs.d[0], rs.c[0]);
        load_row_scales<KIND>(a, row1, nb, cons.c, nblk, rs.d[1], rs.c[1]);
        const int ntok = min(8 * F_GMAX, int(cons.m) - cons.sg0);
        const int G = (ntok + 7) >> 3;
        if (cons.c == 0) {
#pragma unroll
            for (int nt = 0; nt < F_GMAX; nt++) {
                acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
                off[nt][0] = off[nt][1] = off[nt][2] = off[nt][3] = 0.0f;
                rowB[nt] = wk.act_row(cons, cons.sg0 + nt * 8 + g);
                rowC[nt][0] = wk.act_row(cons, cons.sg0 + nt * 8 + 2 * t);
                rowC[nt][1] = wk.act_row(cons, cons.sg0 + nt * 8 + 2 * t + 1);
            }
        }
        const uint32_t stage = takes % STAGES;
        const bool landed = mbar_wait_bounded(bars + stage, (takes / STAGES) & 1);
        if (!__all_sync(0xffffffffu, landed)) {
            ok = false;
            break;
        }
        const uint32_t st = smem_addr(stages + stage * S::BYTES);
        const int col0 = cons.c * F_KC;
        if (G == 1)
            fast_chunk<KIND, 1>(a, st, nblk, lane, col0, nbp, cons.c, rs, rowB, rowC, acc, off);
        else if (G == 2)
            fast_chunk<KIND, 2>(a, st, nblk, lane, col0, nbp, cons.c, rs, rowB, rowC, acc, off);
        else if (G == 3)
            fast_chunk<KIND, 3>(a, st, nblk, lane, col0, nbp, cons.c, rs, rowB, rowC, acc, off);
        else
            fast_chunk<KIND, 4>(a, st, nblk, lane, col0, nbp, cons.c, rs, rowB, rowC, acc, off);
        __syncwarp();

        if (cons.c == wk.nchunks - 1) {
#pragma unroll
            for (int nt = 0; nt < F_GMAX; nt++) {
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int j = cons.sg0 + nt * 8 + 2 * t + i;  // the expert's j-th token
                    if (nt < G && uint32_t(j) < cons.m) {
                        float y0 = acc[nt][i], y1 = acc[nt][2 + i];  // rows g and g+8
                        if (KIND == 2) {
                            y0 = y0 + off[nt][i];
                            y1 = y1 + off[nt][2 + i];
                        }
                        const size_t p = cons.base + j;
                        if (GATE_UP) {
                            if (row0 >= 0) {
                                const float e = exp_poly(-y0);
                                a.out[p * a.out_cols + cons.u * 8 + g] = __fdiv_rn(y0, 1.0f + e) * y1;
                            }
                        } else {
                            if (row0 >= 0) a.out[p * a.out_cols + cons.u * F_ROWS + g] = y0;
                            if (row1 >= 0) a.out[p * a.out_cols + cons.u * F_ROWS + g + 8] = y1;
                        }
                    }
                }
            }
        }
        takes++;
        wk.advance(cons);
    }
    if (!ok) {
        if (lane == 0) atomicExch(a.status, ERR_COPY_WAIT_TIMEOUT);
        for (uint32_t k = takes; k < fills; k++) mbar_wait_bounded(bars + k % STAGES, (k / STAGES) & 1);
    }
}

template <int KIND, bool GATE_UP>
void launch_fast(const ExpertArgs& a, int sms, cudaStream_t stream) {
    const int total_units = a.experts * a.units_per_expert;
    int grid = min(sms, (total_units + F_WARPS - 1) / F_WARPS);
    if (grid < 1) grid = 1;
    expert_fast_kernel<KIND, GATE_UP><<<grid, F_THREADS, fast_smem_bytes<KIND>(), stream>>>(a);
}

}  // namespace

void init_kernels_fast() {
    cudaFuncSetAttribute(expert_fast_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         int(fast_smem_bytes<1>()));
    cudaFuncSetAttribute(expert_fast_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         int(fast_smem_bytes<1>()));
    cudaFuncSetAttribute(expert_fast_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         int(fast_smem_bytes<2>()));
    cudaFuncSetAttribute(expert_fast_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         int(fast_smem_bytes<2>()));
}

int launch_gate_up_fast(const MoeDims& d, const MatrixDev& m, int t, Workspace& ws, int sms,
                        cudaStream_t stream) {
    (void)t;
    const ExpertArgs a = gate_up_args(d, m, ws);
    if (m.kind == 1)
        launch_fast<1, true>(a, sms, stream);
    else
        launch_fast<2, true>(a, sms, stream);
    return 1;
}

int launch_down_fast(const MoeDims& d, const MatrixDev& m, int t, Workspace& ws, int sms,
                     cudaStream_t stream) {
    (void)t;
    const ExpertArgs a = down_args(d, m, ws);
    if (m.kind == 1)
        launch_fast<1, false>(a, sms, stream);
    else
        launch_fast<2, false>(a, sms, stream);
    return 1;
}

}  // namespace tc
