// Grouped expert products for prefill-size groups on the 5th-generation tensor
// cores (tcgen05): int8 x int8 -> int32 MMAs issued by one thread per CTA,
// operands staged in shared memory by bulk async copies, accumulators in tensor
// memory (TMEM), read back with tcgen05.ld for the float work.
//
// Arithmetic: the same single fma chain per output as the decode-size kernel
// (experts_fast.cu), so a token's value does not depend on which kernel ran:
//     acc = fma(float(sum_b), ws[row,b] * xs[token,b], acc)      b = 0, 1, ...
// One MMA has K = 32 = one quantization block, and is issued WITHOUT
// accumulation into its own TMEM buffer: the per-block integer tile must leave
// the tensor core to be scaled by (weight scale x activation scale) before it
// can be added. That float work (about 2.5 instructions per output per block on
// the CUDA cores) bounds this kernel, not the tensor pipe.
//
// Work decomposition: a CTA computes one output tile: 128 weight rows (for
// gate_up: 64 gate rows interleaved with the 64 matching up rows, so SwiGLU
// pairs sit in adjacent lanes) x 64 tokens of one expert, over all of K.
// Roles: warp 16 streams operand chunks (8 blocks: 32 KB of weights + 16 KB of
// activations) through a 3-stage ring; one thread each of warps 17-20 issues the MMAs
// into a ring of 8 TMEM buffers (64 columns each, handed over four at a time);
// warps 0-15 drain the buffers
// (each TMEM lane quadrant is served by four warps, 16 columns each) and keep
// the float chains in registers. Every wait is bounded and watches a CTA-wide
// abort flag; TMEM is freed on every path.
#include <type_traits>

#include "experts_common.cuh"
#include "umma.cuh"

namespace tc {

namespace {

constexpr int P_ROWS = 128;           // MMA M
constexpr int P_TOK = 64;             // MMA N
constexpr int P_CHUNK = 8;            // blocks per smem stage
constexpr int P_STAGES = 3;
constexpr int P_TBUF = 8;             // TMEM buffers of P_TOK columns
constexpr int P_GROUP = 4;            // buffers per barrier: the ring is handed over in halves
constexpr int P_NGRP = P_TBUF / P_GROUP;
static_assert(P_GROUP == 4 && P_CHUNK % P_GROUP == 0, "block b of a group belongs to issuer b % P_MW");
constexpr int P_A_BLOCK = P_ROWS * 32;  // bytes of one block of weights
constexpr int P_B_BLOCK = P_TOK * 32;
constexpr int P_STAGE_BYTES = P_CHUNK * (P_A_BLOCK + P_B_BLOCK);
constexpr int P_EW = 16;               // epilogue warps: 4 TMEM lane quadrants x 4 column slices
constexpr int P_COLS = P_TOK * 4 / P_EW;  // columns (tokens) per epilogue warp
constexpr int P_MW = 4;                // MMA-issuing warps: block b belongs to warp b % P_MW
constexpr int P_THREADS = (P_EW + 1 + P_MW) * 32;  // + producer + MMA issuers
constexpr uint32_t P_SPIN = 1u << 16;
constexpr int P_SMEM_LIMIT = 226 * 1024;

struct PrefillArgs {
    const int8_t* wt;        // weight tiles [expert][row tile][block][128 x 32 canonical]
    const float* wd;         // weight block scales [expert][row tile][nb][128]
    const float* wc;         // 4-bit block offsets, same shape (null for 8-bit)
    const int8_t* xt;        // activation tiles [token tile][block][64 x 32 canonical]
    const float* xst;        // activation scales [token tile][nb][64]
    const float* xsumt;      // scale * sum of quants, same shape (4-bit only)
    const int* tile_expert;  // per token tile
    const uint32_t* tile_p0; // first sorted slot of the tile
    const int* tile_n;       // tokens in the tile (1..64)
    const int* tile_count;
    int nb, row_tiles, rows_per_expert, out_cols;
    float* out;
    const uint32_t* out_rows;
    int* status;
};

// Expert parallel (down only): row p of out_rows' numbering belongs to rank p / rows and goes
// straight into that rank's window, at row p % rows. (A kernel argument of its own: with these
// fields inside PrefillArgs the kernels that do not use them ran 9 % slower.)
struct PrefillPeer {
    float* out[MAX_PEERS];
    uint32_t rows;
    int ranks;
};
struct NoPeer {};

// Bounded wait that also gives up when another warp of the CTA has.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_test(bar, parity)) return true;  // the common case in steady state: no suspension machinery
    for (uint32_t i = 0; i < P_SPIN; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

template <bool Q4, bool GATE_UP, bool PEER = false>
__global__ void __launch_bounds__(P_THREADS, 1)
    expert_prefill_kernel(const PrefillArgs a, const std::conditional_t<PEER, PrefillPeer, NoPeer> peer) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stages = smem;                                                  // P_STAGES x P_STAGE_BYTES
    float* s_xs = reinterpret_cast<float*>(smem + P_STAGES * P_STAGE_BYTES);  // [nb][64]
    float* s_xsum = s_xs + a.nb * P_TOK;                                     // [nb][64] (4-bit)
    float* s_wd = s_xsum + (Q4 ? a.nb * P_TOK : 0);                          // [nb][128]
    float* s_wc = s_wd + a.nb * P_ROWS;                                      // [nb][128] (4-bit)
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_wc + (Q4 ? a.nb * P_ROWS : 0));
    uint64_t* full = bars;                    // [P_STAGES] operands landed
    uint64_t* empty = bars + P_STAGES;        // [P_STAGES] MMAs that read the stage are done
    uint64_t* tfull = bars + 2 * P_STAGES;    // [P_TBUF] a block's integer tile is in TMEM
    uint64_t* tempty = tfull + P_TBUF;        // [P_TBUF] drained by all epilogue warps
    uint64_t* xbar = tempty + P_TBUF;         // activation scales landed
    uint64_t* drain = xbar + 1;               // [P_MW] abort path only: an issuer's MMAs so far are done
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tt = blockIdx.y, rt = blockIdx.x;
    if (tt >= *a.tile_count) return;  // uniform: the whole CTA leaves before touching TMEM
    const int e = a.tile_expert[tt];
    const int tile_n = a.tile_n[tt];
    const uint32_t p0 = a.tile_p0[tt];
    const int nb = a.nb;
    const int nchunks = (nb + P_CHUNK - 1) / P_CHUNK;

    if (tid == 0) {
        for (int s = 0; s < P_STAGES; s++) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, P_MW);
        }
        for (int g = 0; g < P_NGRP; g++) {
            mbar_init(tfull + g, P_MW);
            mbar_init(tempty + g, P_EW);
        }
        mbar_init(xbar, 1);
        for (int i = 0; i < P_MW; i++) mbar_init(drain + i, 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    const size_t tile_index = size_t(e) * a.row_tiles + rt;
    const int8_t* wsrc = a.wt + tile_index * size_t(nb) * P_A_BLOCK;
    const int8_t* xsrc = a.xt + size_t(tt) * nb * P_B_BLOCK;
    auto issue_chunk = [&](int c) {
        const int s = c % P_STAGES;
        const int nblk = min(P_CHUNK, nb - c * P_CHUNK);
        uint8_t* st = stages + s * P_STAGE_BYTES;
        mbar_expect_tx(full + s, uint32_t(nblk) * (P_A_BLOCK + P_B_BLOCK));
        bulk_copy(st, wsrc + size_t(c) * P_CHUNK * P_A_BLOCK, uint32_t(nblk) * P_A_BLOCK, full + s);
        bulk_copy(st + P_CHUNK * P_A_BLOCK, xsrc + size_t(c) * P_CHUNK * P_B_BLOCK, uint32_t(nblk) * P_B_BLOCK,
                  full + s);
    };
    const int first_chunks = min(P_STAGES, nchunks);
    if (warp == P_EW + 1) {
        umma::tmem_alloc(&s_tmem, P_TBUF * P_TOK);
        umma::tmem_relinquish();
    } else if (warp == P_EW && lane == 0) {
        // The ring starts empty: the scales and the first stages' operands are requested
        // while TMEM is being allocated.
        const uint32_t xs_bytes = uint32_t(nb) * P_TOK * 4;
        const uint32_t ws_bytes = uint32_t(nb) * P_ROWS * 4;
        mbar_expect_tx(xbar, (Q4 ? 2 : 1) * (xs_bytes + ws_bytes));
        bulk_copy(s_xs, a.xst + size_t(tt) * nb * P_TOK, xs_bytes, xbar);
        bulk_copy(s_wd, a.wd + tile_index * nb * P_ROWS, ws_bytes, xbar);
        if (Q4) {
            bulk_copy(s_xsum, a.xsumt + size_t(tt) * nb * P_TOK, xs_bytes, xbar);
            bulk_copy(s_wc, a.wc + tile_index * nb * P_ROWS, ws_bytes, xbar);
        }
        for (int c = 0; c < first_chunks; c++) issue_chunk(c);
    }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = s_tmem;
    volatile int* abort_flag = &s_abort;

    if (warp == P_EW) {
        // ---- producer: the rest of the operand chunks, each once its stage is free again
        if (lane == 0) {
            int c = first_chunks;
            for (; c < nchunks; c++) {
                const int s = c % P_STAGES;
                if (!wait_or_abort(empty + s, ((c / P_STAGES) & 1) ^ 1, abort_flag)) break;
                issue_chunk(c);
            }
            if (*abort_flag) {
                // Giving up: let the copies already issued land before the CTA's shared memory is released.
                mbar_wait_bounded(xbar, 0);
                for (int i = max(0, c - P_STAGES); i < c; i++) mbar_wait_bounded(full + i % P_STAGES, (i / P_STAGES) & 1);
            }
        }
    } else if (warp > P_EW) {
        // ---- MMA issuers: one block = one MMA into its own TMEM buffer. A single thread
        // spends several hundred cycles per block on its waits, fence and commit, far more
        // than the MMA takes, so P_MW threads (one per warp) take the blocks in turn; the
        // blocks are independent (different TMEM buffers), so no order among them is needed.
        if (lane == 0) {
            const uint32_t idesc = umma::idesc_s8(P_ROWS, P_TOK);
            const int mw = warp - P_EW - 1;
            const int ngroups = (nb + P_GROUP - 1) / P_GROUP;
            for (int g = 0; g < ngroups; g++) {
                // Block mw of every group of P_GROUP (= P_MW) blocks; the group's TMEM half is
                // free once the epilogue warps have read group g - P_NGRP out of it.
                const int b = g * P_GROUP + mw, gi = g % P_NGRP;
                if (!wait_or_abort(tempty + gi, ((g / P_NGRP) & 1) ^ 1, abort_flag)) break;
                if (b >= nb) {  // ragged last group: keep the arrival count whole
                    mbar_arrive(tfull + gi);
                    continue;
                }
                const int c = b / P_CHUNK, k = b % P_CHUNK, s = c % P_STAGES, buf = b % P_TBUF;
                if (k < P_MW && !wait_or_abort(full + s, (c / P_STAGES) & 1, abort_flag)) break;
                umma::fence_after_sync();
                const uint32_t sa = smem_addr(stages + s * P_STAGE_BYTES + k * P_A_BLOCK);
                const uint32_t sb = smem_addr(stages + s * P_STAGE_BYTES + P_CHUNK * P_A_BLOCK + k * P_B_BLOCK);
                umma::mma_s8(tmem + buf * P_TOK, umma::smem_desc(sa, P_ROWS * 16, 128),
                             umma::smem_desc(sb, P_TOK * 16, 128), idesc, 0u);
                umma::commit(tfull + gi);
                // This thread's last block of the chunk. (A ragged last chunk may leave
                // `empty` short of arrivals: nothing waits for it.)
                if (k + P_MW >= P_CHUNK || b + P_MW >= nb) umma::commit(empty + s);
            }
            if (*abort_flag) {
                // Giving up: the MMAs in flight must finish before TMEM is freed.
                umma::commit(drain + mw);
                mbar_wait_bounded(drain + mw, 0);
            }
        }
    } else {
        // ---- epilogue: warp w drains lanes 32*(w%4).. and columns P_COLS*(w/4)..
        const int quad = warp & 3, slice = warp >> 2;
        const int row = quad * 32 + lane;  // row of the tile = TMEM lane
        float acc[P_COLS], off[Q4 ? P_COLS : 1];
#pragma unroll
        for (int j = 0; j < P_COLS; j++) acc[j] = 0.0f;
        if (Q4) {
#pragma unroll
            for (int j = 0; j < P_COLS; j++) off[j] = 0.0f;
        }
        bool ok = wait_or_abort(xbar, 0, abort_flag);
        const uint32_t tbase = tmem + (uint32_t(quad * 32) << 16) + slice * P_COLS;
        // One block's float work on the integer tile in v.
        auto consume = [&](int b, const int (&v)[P_COLS]) {
            const float wdb = s_wd[b * P_ROWS + row];
            const float wcb = Q4 ? s_wc[b * P_ROWS + row] : 0.0f;
            const float4* xs4 = reinterpret_cast<const float4*>(s_xs + b * P_TOK + slice * P_COLS);
            const float4* su4 = reinterpret_cast<const float4*>(s_xsum + b * P_TOK + slice * P_COLS);
#pragma unroll
            for (int j = 0; j < P_COLS / 4; j++) {
                const float4 x = xs4[j];
                const float2 xlo = make_float2(x.x, x.y), xhi = make_float2(x.z, x.w);
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int i = 4 * j + 2 * h;
                    // The conversion unit works beside the FP32 pipe, which the two packed
                    // operations below keep busy; the add-a-magic-number conversion used
                    // where issue slots are short would add a third FP32 operation here.
                    const float2 sum = make_float2(__int2float_rn(v[i]), __int2float_rn(v[i + 1]));
                    const float2 d = mul2(make_float2(wdb, wdb), h ? xhi : xlo);
                    const float2 r = fma2(sum, d, make_float2(acc[i], acc[i + 1]));
                    acc[i] = r.x;
                    acc[i + 1] = r.y;
                }
                if (Q4) {
                    const float4 u = su4[j];
                    const float2 o0 = fma2(make_float2(wcb, wcb), make_float2(u.x, u.y),
                                           make_float2(off[4 * j], off[4 * j + 1]));
                    const float2 o1 = fma2(make_float2(wcb, wcb), make_float2(u.z, u.w),
                                           make_float2(off[4 * j + 2], off[4 * j + 3]));
                    off[4 * j] = o0.x, off[4 * j + 1] = o0.y, off[4 * j + 2] = o1.x, off[4 * j + 3] = o1.y;
                }
            }
        };
        // Block b's tile is read from TMEM while block b-1's float work runs: the load is
        // asynchronous until wait_ld, and the two register tiles alternate.
        auto fetch = [&](int b, int (&v)[P_COLS]) -> bool {
            if (b % P_GROUP == 0) {  // first block of a group: its MMAs are all done
                if (!wait_or_abort(tfull + (b / P_GROUP) % P_NGRP, (b / P_TBUF) & 1, abort_flag)) return false;
                umma::fence_after_sync();
            }
            umma::ld_32x16(tbase + (b % P_TBUF) * P_TOK, v);
            return true;
        };
        auto release = [&](int b) {  // after wait_ld of a group's last block: its half may be overwritten
            if (b % P_GROUP == P_GROUP - 1 || b == nb - 1) {
                umma::fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty + (b / P_GROUP) % P_NGRP);
            }
        };
        int va[P_COLS], vb[P_COLS];
        if (ok) ok = fetch(0, va);
        for (int b = 0; ok && b < nb; b += 2) {
            umma::wait_ld(va);
            release(b);
            if (b + 1 < nb && !fetch(b + 1, vb)) {
                ok = false;
                break;
            }
            consume(b, va);
            if (b + 1 < nb) {
                umma::wait_ld(vb);
                release(b + 1);
                if (b + 2 < nb && !fetch(b + 2, va)) {
                    ok = false;
                    break;
                }
                consume(b + 1, vb);
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            if (GATE_UP) {
                // Lanes 2i / 2i+1 hold the gate / up row of hidden column 64*rt + i. The pair
                // trades halves so that each lane finishes one token of every two: the even
                // lane token j (its gate, the partner's up), the odd lane token j+1.
                const bool odd = lane & 1;
                const int col = rt * 64 + (row >> 1);
#pragma unroll
                for (int j = 0; j < P_COLS; j += 2) {
                    float y0 = acc[j], y1 = acc[j + 1];
                    if (Q4) y0 = y0 + off[j], y1 = y1 + off[j + 1];
                    const float got = __shfl_xor_sync(0xffffffffu, odd ? y0 : y1, 1);
                    const float g = odd ? got : y0, up = odd ? y1 : got;
                    const int n = slice * P_COLS + j + (odd ? 1 : 0);  // token of the tile
                    if (n < tile_n && col < a.out_cols) {
                        const float ex = exp_poly(-g);
                        a.out[size_t(p0 + n) * a.out_cols + col] = __fdiv_rn(g, 1.0f + ex) * up;
                    }
                }
            } else {
                const int r = rt * P_ROWS + row;
#pragma unroll
                for (int j = 0; j < P_COLS; j++) {
                    float y = acc[j];
                    if (Q4) y = y + off[j];
                    const int n = slice * P_COLS + j;
                    if (n < tile_n && r < a.out_cols) {
                        size_t p = p0 + n;
                        if (a.out_rows) p = a.out_rows[p];
                        float* dst = a.out;
                        if constexpr (PEER) {
                            const uint32_t home = uint32_t(p) / peer.rows;
                            p -= size_t(home) * peer.rows;
                            dst = peer.out[home];
                        }
                        dst[p * a.out_cols + r] = y;
                    }
                }
            }
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == P_EW + 1) umma::tmem_dealloc(tmem, P_TBUF * P_TOK);
    if (tid == 0 && s_abort) atomicExch(a.status, ERR_COPY_WAIT_TIMEOUT);
}

// ---------------------------------------------------------------- tiling kernels

// Weights of one (expert, row tile) into canonical 128 x 32 tiles per block,
// with their block scales (and 4-bit offsets) as f32 per (block, row). 4-bit
// values are expanded to int8 (q - 8). One CTA per (expert, row tile).
template <bool Q4, bool GATE_UP>
__global__ void tile_prefill_weights_kernel(const uint8_t* __restrict__ wdata, const void* __restrict__ wscales,
                                            int cols, int rows_per_expert, int row_tiles,
                                            int8_t* __restrict__ wt, float* __restrict__ wd,
                                            float* __restrict__ wc) {
    const int rt = blockIdx.x % row_tiles, e = blockIdx.x / row_tiles;
    const int nb = cols / QK;
    const size_t tile_index = size_t(e) * row_tiles + rt;
    int8_t* dst = wt + tile_index * size_t(nb) * P_A_BLOCK;
    for (int r = 0; r < P_ROWS; r++) {
        int row;
        if (GATE_UP) {
            const int inter = rows_per_expert / 2, col = rt * 64 + (r >> 1);
            row = col < inter ? e * rows_per_expert + (r & 1 ? inter : 0) + col : -1;
        } else {
            const int rr = rt * P_ROWS + r;
            row = rr < rows_per_expert ? e * rows_per_expert + rr : -1;
        }
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            const int b = i / QK, k = i % QK;
            int8_t v = 0;
            if (row >= 0) {
                if (!Q4) {
                    v = int8_t(wdata[size_t(row) * cols + i]);
                } else {
                    const uint8_t byte = wdata[(size_t(row) * cols) / 2 + b * 16 + (k & 15)];
                    v = int8_t(int(k < 16 ? (byte & 0xF) : (byte >> 4)) - 8);
                }
            }
            dst[size_t(b) * P_A_BLOCK + umma::tile_offset(P_ROWS, r, k)] = v;
        }
        for (int b = threadIdx.x; b < nb; b += blockDim.x) {
            float d = 0.0f, c = 0.0f;
            if (row >= 0) {
                if (!Q4) {
                    d = f16_bits_to_f32(reinterpret_cast<const uint16_t*>(wscales)[size_t(row) * nb + b]);
                } else {
                    const int words = (nb + SUPER - 1) / SUPER * SUPER_WORDS;
                    const uint32_t* w = reinterpret_cast<const uint32_t*>(wscales) + size_t(row) * words +
                                        (b / SUPER) * SUPER_WORDS;
                    const int j = b % SUPER;
                    d = f16_bits_to_f32(uint16_t(w[0])) * float((w[1 + j / 4] >> (8 * (j % 4))) & 0xFFu);
                    c = f16_bits_to_f32(uint16_t(w[0] >> 16)) *
                        float(int(int8_t(uint8_t(w[3 + j / 4] >> (8 * (j % 4))))));
                }
            }
            wd[(tile_index * nb + b) * P_ROWS + r] = d;
            if (Q4) wc[(tile_index * nb + b) * P_ROWS + r] = c;
        }
    }
}

// The token tiles of the experts: expert e with m tokens gets ceil(m / 64) tiles. One CTA.
__global__ void build_token_tiles_kernel(const uint32_t* __restrict__ counts, const uint32_t* __restrict__ offsets,
                                         int experts, int* __restrict__ tile_expert,
                                         uint32_t* __restrict__ tile_p0, int* __restrict__ tile_n,
                                         int* __restrict__ tile_count) {
    __shared__ int s_base[MAX_EXPERTS + 1];
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < experts; e++) {
            s_base[e] = run;
            run += (int(counts[e]) + P_TOK - 1) / P_TOK;
        }
        s_base[experts] = run;
        *tile_count = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const int m = int(counts[e]);
        for (int i = 0; i * P_TOK < m; i++) {
            const int tt = s_base[e] + i;
            tile_expert[tt] = e;
            tile_p0[tt] = offsets[e] + i * P_TOK;
            tile_n[tt] = min(P_TOK, m - i * P_TOK);
        }
    }
}

// Activations into canonical 64 x 32 tiles per (token tile, block), scales (and
// block sums) transposed to [block][token]. Source rows are already 8-bit
// (xq/xs/xsum through row_of_slot) or f32 rows to quantize here (xf), as
// quantize_q8 does (src/kernels.rs:84-98). A thread per (token, block).
template <bool Q4>
__global__ void tile_activations_kernel(const int8_t* __restrict__ xq, const float* __restrict__ xs,
                                        const float* __restrict__ xsum, const float* __restrict__ xf,
                                        const uint32_t* __restrict__ row_of_slot, int cols, int nbp,
                                        const uint32_t* __restrict__ tile_p0, const int* __restrict__ tile_n,
                                        const int* __restrict__ tile_count, int8_t* __restrict__ xt,
                                        float* __restrict__ xst, float* __restrict__ xsumt) {
    const int nb = cols / QK;
    const int tt = blockIdx.x;
    if (tt >= *tile_count) return;
    const int n_valid = tile_n[tt];
    const uint32_t p0 = tile_p0[tt];
    for (int task = threadIdx.x; task < P_TOK * nb; task += blockDim.x) {
        const int n = task % P_TOK, b = task / P_TOK;
        uint32_t q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        float d = 0.0f, su = 0.0f;
        if (n < n_valid) {
            const size_t p = p0 + n;
            const size_t row = row_of_slot ? row_of_slot[p] : p;
            if (xf) {
                const float4* src = reinterpret_cast<const float4*>(xf + row * cols + b * QK);
                float4 v[8];
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] = src[i];
                float amax = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++)
                    amax = fmaxf(fmaxf(fmaxf(fmaxf(amax, fabsf(v[i].x)), fabsf(v[i].y)), fabsf(v[i].z)),
                                 fabsf(v[i].w));
                d = __fdiv_rn(amax, 127.0f);
                const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
                auto q8 = [&](float x) {
                    const float rr = roundf(x * id);
                    return (rr != rr) ? 0 : int(fminf(127.0f, fmaxf(-128.0f, rr)));
                };
                int qsum = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int q0 = q8(v[i].x), q1 = q8(v[i].y), q2 = q8(v[i].z), q3 = q8(v[i].w);
                    qsum += q0 + q1 + q2 + q3;
                    q[i] = uint32_t(q0 & 0xFF) | (uint32_t(q1 & 0xFF) << 8) | (uint32_t(q2 & 0xFF) << 16) |
                           (uint32_t(q3 & 0xFF) << 24);
                }
                su = d * float(qsum);
            } else {
                const uint4* src = reinterpret_cast<const uint4*>(xq + row * cols + b * QK);
                const uint4 lo = src[0], hi = src[1];
                q[0] = lo.x, q[1] = lo.y, q[2] = lo.z, q[3] = lo.w;
                q[4] = hi.x, q[5] = hi.y, q[6] = hi.z, q[7] = hi.w;
                d = xs[row * nbp + b];
                if (Q4) su = xsum[row * nbp + b];
            }
        }
        // Bytes 0-15 and 16-31 of the token's block are the two K halves of its core-matrix row.
        int8_t* dst = xt + (size_t(tt) * nb + b) * P_B_BLOCK;
        *reinterpret_cast<uint4*>(dst + umma::tile_offset(P_TOK, n, 0)) = make_uint4(q[0], q[1], q[2], q[3]);
        *reinterpret_cast<uint4*>(dst + umma::tile_offset(P_TOK, n, 16)) = make_uint4(q[4], q[5], q[6], q[7]);
        xst[(size_t(tt) * nb + b) * P_TOK + n] = d;
        if (Q4) xsumt[(size_t(tt) * nb + b) * P_TOK + n] = su;
    }
}

size_t prefill_smem(int nb, bool q4) {
    return size_t(P_STAGES) * P_STAGE_BYTES + size_t(nb) * (P_TOK + P_ROWS) * 4 * (q4 ? 2 : 1) +
           (2 * P_STAGES + 2 * P_TBUF + 1 + P_MW) * 8 + 64;
}

}  // namespace

void init_kernels_prefill() {
    const int lim = P_SMEM_LIMIT;  // the kernel also has a few static words
    cudaFuncSetAttribute(expert_prefill_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(expert_prefill_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(expert_prefill_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(expert_prefill_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(expert_prefill_kernel<true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(expert_prefill_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
}

int prefill_row_tiles(const MoeDims& d, bool gate_up) {
    return gate_up ? (d.inter + 63) / 64 : (d.hidden + P_ROWS - 1) / P_ROWS;
}

bool prefill_fits(const MoeDims& d, bool q4_gate_up, bool q4_down) {
    return prefill_smem(d.hidden / QK, q4_gate_up) <= size_t(P_SMEM_LIMIT) &&
           prefill_smem(d.inter / QK, q4_down) <= size_t(P_SMEM_LIMIT);
}

size_t prefill_weight_bytes(const MoeDims& d, bool gate_up) {
    const int cols = gate_up ? d.hidden : d.inter;
    return size_t(d.experts) * prefill_row_tiles(d, gate_up) * (cols / QK) * P_A_BLOCK;
}

size_t prefill_scale_elems(const MoeDims& d, bool gate_up) {
    const int cols = gate_up ? d.hidden : d.inter;
    return size_t(d.experts) * prefill_row_tiles(d, gate_up) * P_ROWS * (cols / QK);
}

int prefill_max_token_tiles(int slots, int experts) { return (slots + P_TOK - 1) / P_TOK + experts; }
int prefill_token_tile() { return P_TOK; }

void tile_prefill_weights(const MoeDims& d, const MatrixDev& m, bool gate_up, int8_t* wt, float* wd, float* wc,
                          cudaStream_t stream) {
    const int cols = gate_up ? d.hidden : d.inter;
    const int rpe = gate_up ? 2 * d.inter : d.hidden;
    const int rts = prefill_row_tiles(d, gate_up);
    const unsigned grid = unsigned(d.experts * rts);
    const uint8_t* data = static_cast<const uint8_t*>(m.data);
    if (m.kind == 1) {
        if (gate_up) tile_prefill_weights_kernel<false, true><<<grid, 256, 0, stream>>>(data, m.scales, cols, rpe, rts, wt, wd, wc);
        else tile_prefill_weights_kernel<false, false><<<grid, 256, 0, stream>>>(data, m.scales, cols, rpe, rts, wt, wd, wc);
    } else {
        if (gate_up) tile_prefill_weights_kernel<true, true><<<grid, 256, 0, stream>>>(data, m.scales, cols, rpe, rts, wt, wd, wc);
        else tile_prefill_weights_kernel<true, false><<<grid, 256, 0, stream>>>(data, m.scales, cols, rpe, rts, wt, wd, wc);
    }
}

// One of the two grouped products on the tensor cores. `src` describes where the
// activations come from: 8-bit rows through row_of_slot (gate_up), or f32 rows
// in slot order to quantize (down).
int launch_prefill(const MoeDims& d, bool gate_up, bool q4, const PrefillWeights& w, const PrefillScratch& s,
                   const Workspace& ws, int slots, float* out, const uint32_t* out_rows, cudaStream_t stream,
                   float* const* peer_out, int peer_ranks, uint32_t peer_rows) {
    const int cols = gate_up ? d.hidden : d.inter;
    const int nb = cols / QK, nbp = (nb + 7) / 8 * 8;
    const int max_tiles = prefill_max_token_tiles(slots, d.experts);
    int launched = 0;
    if (gate_up) {
        build_token_tiles_kernel<<<1, 256, 0, stream>>>(ws.counts, ws.offsets, d.experts, s.tile_expert, s.tile_p0,
                                                        s.tile_n, s.tile_count);
        launched++;
    }
    if (q4)
        tile_activations_kernel<true><<<max_tiles, 256, 0, stream>>>(
            gate_up ? ws.xq : nullptr, gate_up ? ws.xs : nullptr, gate_up ? ws.xsum : nullptr,
            gate_up ? nullptr : ws.hidden_f, gate_up ? ws.slot_token : nullptr, cols, nbp, s.tile_p0, s.tile_n,
            s.tile_count, s.xt, s.xst, s.xsumt);
    else
        tile_activations_kernel<false><<<max_tiles, 256, 0, stream>>>(
            gate_up ? ws.xq : nullptr, gate_up ? ws.xs : nullptr, nullptr, gate_up ? nullptr : ws.hidden_f,
            gate_up ? ws.slot_token : nullptr, cols, nbp, s.tile_p0, s.tile_n, s.tile_count, s.xt, s.xst, s.xsumt);
    launched++;
    PrefillArgs a{};
    a.wt = gate_up ? w.gu_t : w.dn_t;
    a.wd = gate_up ? w.gu_d : w.dn_d;
    a.wc = gate_up ? w.gu_c : w.dn_c;
    a.xt = s.xt;
    a.xst = s.xst;
    a.xsumt = s.xsumt;
    a.tile_expert = s.tile_expert;
    a.tile_p0 = s.tile_p0;
    a.tile_n = s.tile_n;
    a.tile_count = s.tile_count;
    a.nb = nb;
    a.row_tiles = prefill_row_tiles(d, gate_up);
    a.rows_per_expert = gate_up ? 2 * d.inter : d.hidden;
    a.out_cols = gate_up ? d.inter : d.hidden;
    a.out = out;
    a.out_rows = out_rows;
    PrefillPeer pp{};
    const bool to_peers = peer_out && !gate_up;
    if (to_peers) {
        for (int r = 0; r < peer_ranks && r < MAX_PEERS; r++) pp.out[r] = peer_out[r];
        pp.ranks = peer_ranks;
        pp.rows = peer_rows;
    }
    a.status = ws.status;
    const dim3 grid(a.row_tiles, max_tiles);
    const size_t smem = prefill_smem(nb, q4);
    if (q4) {
        if (gate_up) expert_prefill_kernel<true, true><<<grid, P_THREADS, smem, stream>>>(a, NoPeer{});
        else if (to_peers) expert_prefill_kernel<true, false, true><<<grid, P_THREADS, smem, stream>>>(a, pp);
        else expert_prefill_kernel<true, false><<<grid, P_THREADS, smem, stream>>>(a, NoPeer{});
    } else {
        if (gate_up) expert_prefill_kernel<false, true><<<grid, P_THREADS, smem, stream>>>(a, NoPeer{});
        else if (to_peers) expert_prefill_kernel<false, false, true><<<grid, P_THREADS, smem, stream>>>(a, pp);
        else expert_prefill_kernel<false, false><<<grid, P_THREADS, smem, stream>>>(a, NoPeer{});
    }
    return launched + 1;
}

}  // namespace tc

