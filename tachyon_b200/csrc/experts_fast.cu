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
// The kernel is bound by HBM, not by the tensor pipe: at decode sizes every
// selected expert's weights are read once and used for a handful of tokens.
// So the design is about bytes in flight and about keeping the loop off global
// memory:
//  - Weights are re-tiled once, when a layer is created, into records of one
//    unit (16 rows) x one 256-column chunk: 16 rows of [weights | that row's
//    block scales], row stride 272 bytes (8-bit) or 144 bytes (4-bit). One
//    record is one bulk async copy and lands in shared memory already padded
//    so that ldmatrix reads hit 32 distinct banks.
//  - Persistent CTAs, one per SM; the units of experts that have tokens are
//    cut into equal contiguous ranges per CTA, and a CTA's units go to its
//    warps round-robin; each warp streams its units' records through a
//    private ring of shared-memory stages, completion counted on an mbarrier
//    per stage (every wait has a spin limit).
//  - The tokens of the experts a CTA's range touches (two segments of up to
//    16 tokens at a time, usually the whole range) are staged once per CTA:
//    int8 rows by bulk copies, their scales transposed by plain loads; for the
//    down projection the SwiGLU rows are quantized as they are staged.
#include "experts_fast.cuh"

namespace tc {

namespace {

constexpr int F_MAX_WARPS = 16;   // warps per CTA: 16, or fewer when that buys a deeper ring
constexpr int F_XBUF = 2;         // segments whose tokens are staged at the same time
constexpr int F_GMAX = 2;         // token tiles of 8 held in registers
constexpr int F_TOK = 8 * F_GMAX; // tokens staged per segment
constexpr int F_MAX_STAGES = 6;
constexpr size_t F_SMEM_LIMIT = 227 * 1024;

struct FastArgs {
    ExpertArgs e;
    const uint8_t* tiled;  // records [expert][unit][chunk]
    int stages;            // ring depth per warp
    int x_stride;          // bytes per staged activation row (cols + 16)
    int nbp;               // pad8(cols / 32)
    int dense;             // walk every expert (static partition) instead of the active list
};

// Shared memory carve-up (offsets in bytes).
template <int KIND>
struct Layout {
    int ring, bars, x0, xbytes, xs_off, xsum_off, total;
    __host__ __device__ Layout(int nwarps, int stages, int cols, int nbp) {
        int o = 0;
        ring = o;
        o += nwarps * stages * Rec<KIND>::BYTES;
        o = (o + 127) / 128 * 128;
        x0 = o;
        // One staged-token buffer: int8 rows, then scales [block][token], then (4-bit) block sums.
        xs_off = F_TOK * (cols + 16);
        xsum_off = xs_off + nbp * F_TOK * 4;
        xbytes = xsum_off + (KIND == 2 ? nbp * F_TOK * 4 : 0);
        xbytes = (xbytes + 127) / 128 * 128;
        o += F_XBUF * xbytes;
        bars = o;
        o += (F_MAX_WARPS * F_MAX_STAGES + 1) * 8;
        total = o;
    }
    __host__ __device__ int xq(int buf) const { return x0 + buf * xbytes; }
    __host__ __device__ int xsT(int buf) const { return x0 + buf * xbytes + xs_off; }
    __host__ __device__ int xsumT(int buf) const { return x0 + buf * xbytes + xsum_off; }
};

// A warp's place in its sequence of (expert, token segment, unit, chunk) steps.
// Units are numbered over the experts that have tokens; a CTA owns [lo, hi).
// Within a CTA the units of consecutive segments go to consecutive warps
// (rotation), so that a range spanning two experts still gives every warp one
// unit instead of giving the first few warps two.
struct FCursor {
    int ai;       // index into the active-expert list
    int sg0;      // first token of the segment
    int a;        // unit (in active-unit space)
    int c;        // chunk
    int seg_hi;   // end of this CTA's units of expert ai
    uint32_t m;   // tokens of the expert
    int e;        // expert id
    bool valid;
};

template <int KIND>
struct FWalker {
    const FastArgs& f;
    const int warp, nwarps, lo, hi, nchunks, upe;

    __device__ FWalker(const FastArgs& args, int warp_, int nwarps_, int lo_, int hi_)
        : f(args), warp(warp_), nwarps(nwarps_), lo(lo_), hi(hi_),
          nchunks((args.e.cols + F_KC - 1) / F_KC), upe(args.e.units_per_expert) {}

    // Positions at the warp's first unit of (ai, sg0) or of the next segment that has one.
    __device__ void settle(FCursor& cur) const {
        for (;;) {
            if (lo >= hi || cur.ai * upe >= hi) {
                cur.valid = false;
                return;
            }
            if (f.e.runs.expert) {  // ai counts runs of up to F_TOK slots
                cur.e = f.e.runs.expert[cur.ai];
                cur.m = f.e.runs.count[cur.ai];
            } else {
                cur.e = f.dense ? cur.ai : int(f.e.active[cur.ai]);
                cur.m = f.e.counts[cur.e];
            }
            if (f.dense && cur.m == 0) cur.m = 1;  // an expert nobody picked is walked once, with no tokens
            const int seg_lo = max(lo, cur.ai * upe);
            cur.seg_hi = min(hi, (cur.ai + 1) * upe);
            if (uint32_t(cur.sg0) < cur.m) {
                const int rot = (seg_lo - lo) % nwarps;
                cur.a = seg_lo + (warp - rot + nwarps) % nwarps;
                if (cur.a < cur.seg_hi) {
                    cur.c = 0;
                    cur.valid = true;
                    return;
                }
                cur.sg0 += F_TOK;  // no unit for this warp here: same answer for every segment
                continue;
            }
            cur.ai++;
            cur.sg0 = 0;
        }
    }

    __device__ void advance(FCursor& cur) const {
        if (++cur.c < nchunks) return;
        cur.c = 0;
        cur.a += nwarps;
        if (cur.a < cur.seg_hi) return;
        cur.sg0 += F_TOK;
        settle(cur);
    }

    __device__ const uint8_t* record(const FCursor& cur) const {
        const int u = cur.a - cur.ai * upe;
        return f.tiled + (size_t(cur.e * upe + u) * nchunks + cur.c) * Rec<KIND>::BYTES;
    }
};

// One segment of the CTA's walk: an expert and up to F_TOK of its tokens.
struct Segment {
    int ai, e, sg0, ntok, G;
    uint32_t m, mw, base;  // tokens of the expert; the same, at least 1 in a dense walk
    bool valid;
};

template <int KIND, bool GATE_UP>
__global__ void __launch_bounds__(F_MAX_WARPS * 32, 1) expert_fast_kernel(const FastArgs f) {
    using R = Rec<KIND>;
    const ExpertArgs& a = f.e;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5, nthreads = blockDim.x;
    const Layout<KIND> L(nwarps, f.stages, a.cols, f.nbp);
    const int STAGES = f.stages;
    grid_launch_dependents();
    uint8_t* ring = smem + L.ring + size_t(warp) * STAGES * R::BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bars) + warp * F_MAX_STAGES;
    if (lane == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(bars + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    const int upe = a.units_per_expert;
    const int nchunks = (a.cols + F_KC - 1) / F_KC;
    // Dense walk (batches that reach nearly every expert): the partition of units over
    // CTAs and warps does not depend on the routing, so each warp's first records are
    // requested before this grid waits for the one in front of it in the stream: the
    // weights stream in while the router (or the gate_up kernel's tail) still runs.
    int npre = 0;
    if (f.dense) {
        const int total_d = a.experts * upe;
        const int lo_d = int((long long)blockIdx.x * total_d / gridDim.x);
        const int hi_d = int((long long)(blockIdx.x + 1) * total_d / gridDim.x);
        const int a0 = lo_d + warp;  // the first expert of the range starts the rotation at warp 0
        if (a0 < min(hi_d, (lo_d / upe + 1) * upe)) {
            npre = min(STAGES, nchunks);  // the whole ring: the walk's first fill then waits for a free stage
            if (lane == 0) {
                for (int s = 0; s < npre; s++) {
                    mbar_expect_tx(bars + s, R::BYTES);
                    bulk_copy(ring + s * R::BYTES, f.tiled + (size_t(a0) * nchunks + s) * R::BYTES, R::BYTES,
                              bars + s);
                }
            }
        }
    }
    grid_dependency_wait();  // everything below reads what earlier kernels wrote
    const int total = (a.runs.expert ? *a.runs.n : f.dense ? a.experts : int(a.active[a.experts])) * upe;
    const int lo = int((long long)blockIdx.x * total / gridDim.x);
    const int hi = int((long long)(blockIdx.x + 1) * total / gridDim.x);

    FWalker<KIND> wk(f, warp, nwarps, lo, hi);
    FCursor prod;
    prod.ai = lo / upe;
    prod.sg0 = 0;
    wk.settle(prod);
    FCursor cons = prod;

    uint32_t fills = 0, takes = 0;
    auto fill_next = [&]() {
        if (!prod.valid) return;
        if (lane == 0) {
            uint64_t* bar = bars + fills % STAGES;
            mbar_expect_tx(bar, R::BYTES);
            bulk_copy(ring + (fills % STAGES) * R::BYTES, wk.record(prod), R::BYTES, bar);
        }
        fills++;
        wk.advance(prod);
    };
    for (int s = 0; s < npre; s++) {  // already on their way
        fills++;
        wk.advance(prod);
    }
    for (int s = npre; s < STAGES - 1; s++) fill_next();

    const int g = lane >> 2, t = lane & 3;
    const int nb = a.cols / QK;
    float acc[F_GMAX][4], off[F_GMAX][4];
    bool ok = true;
    uint32_t xphase = 0, xtok = 0;

    // The CTA's segments in order, the same walk in every thread.
    Segment next;
    next.ai = lo / upe;
    next.sg0 = -F_TOK;
    next.m = next.mw = 0;
    next.valid = lo < hi;
    bool walking = false;
    auto step_segment = [&](Segment& sgm) {
        if (!sgm.valid) return;
        sgm.sg0 += F_TOK;
        while (!walking || uint32_t(sgm.sg0) >= sgm.mw) {  // first call, or past this expert's tokens
            if (walking) sgm.ai++;
            walking = true;
            if (sgm.ai * upe >= hi) {
                sgm.valid = false;
                return;
            }
            if (a.runs.expert) {
                sgm.e = a.runs.expert[sgm.ai];
                sgm.m = a.runs.count[sgm.ai];
                sgm.base = a.runs.offset[sgm.ai];
            } else {
                sgm.e = f.dense ? sgm.ai : int(a.active[sgm.ai]);
                sgm.m = a.counts[sgm.e];
                sgm.base = a.offsets[sgm.e];
            }
            sgm.mw = f.dense && sgm.m == 0 ? 1u : sgm.m;
            sgm.sg0 = 0;
        }
        sgm.ntok = max(0, min(F_TOK, int(sgm.m) - sgm.sg0));
        sgm.G = (sgm.ntok + 7) >> 3;
    };
    step_segment(next);

    while (ok && next.valid) {
        // ---- a group: up to F_XBUF segments whose tokens are staged together, so that
        // warps working on different experts of this CTA's range run side by side.
        Segment seg[F_XBUF];
        int nseg = 0;
        for (; nseg < F_XBUF && next.valid; nseg++) {
            seg[nseg] = next;
            step_segment(next);
        }
        __syncthreads();  // everyone is done with the previous group's tokens
        if (!GATE_UP && a.xf) {
            // The down projection's inputs are the SwiGLU rows in f32: quantize the
            // segments' rows here exactly as quantize_q8 does (src/kernels.rs:84-98,
            // applied per gathered row by src/weights.rs:652-664), straight into the
            // staged layout. A thread per (token, 32-block): eight 16-byte loads in
            // flight, the block's maximum and its 32 roundings in registers.
#pragma unroll
            for (int sx = 0; sx < F_XBUF; sx++) {
                if (sx < nseg) {
                    const Segment& sg = seg[sx];
                    float* xsT = reinterpret_cast<float*>(smem + L.xsT(sx));
                    float* xsumT = reinterpret_cast<float*>(smem + L.xsumT(sx));
                    for (int task = threadIdx.x; task < sg.G * 8 * nb; task += nthreads) {
                        const int j = task / nb, b = task - j * nb;
                        const size_t row = sg.base + sg.sg0 + min(j, sg.ntok - 1);
                        const float4* src = reinterpret_cast<const float4*>(a.xf + row * a.cols + b * QK);
                        float4 v[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) v[i] = src[i];
                        float amax = 0.0f;
#pragma unroll
                        for (int i = 0; i < 8; i++)
                            amax = fmaxf(fmaxf(fmaxf(fmaxf(amax, fabsf(v[i].x)), fabsf(v[i].y)), fabsf(v[i].z)),
                                         fabsf(v[i].w));
                        const float d = __fdiv_rn(amax, 127.0f);
                        const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
                        auto q8 = [&](float x) {
                            const float rr = roundf(x * id);
                            return (rr != rr) ? 0 : int(fminf(127.0f, fmaxf(-128.0f, rr)));
                        };
                        uint32_t packed[8];
                        int qsum = 0;
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const int q0 = q8(v[i].x), q1 = q8(v[i].y), q2 = q8(v[i].z), q3 = q8(v[i].w);
                            qsum += q0 + q1 + q2 + q3;
                            packed[i] = uint32_t(q0 & 0xFF) | (uint32_t(q1 & 0xFF) << 8) |
                                        (uint32_t(q2 & 0xFF) << 16) | (uint32_t(q3 & 0xFF) << 24);
                        }
                        uint4* dst = reinterpret_cast<uint4*>(smem + L.xq(sx) + j * f.x_stride + b * QK);
                        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        xsT[b * F_TOK + j] = d;
                        if (KIND == 2) xsumT[b * F_TOK + j] = d * float(qsum);
                    }
                }
            }
            __syncthreads();
            // A value the compiler cannot know before the barrier: the staged reads depend on it.
            asm volatile("mov.u32 %0, %1;" : "=r"(xtok) : "r"(xphase) : "memory");
        } else {
            // Token rows by plain 16-byte loads, not bulk copies: the copy engine's queue
            // already holds this CTA's first weight records, and a bulk copy issued now
            // would wait behind all of them.
#pragma unroll
            for (int sx = 0; sx < F_XBUF; sx++) {
                if (sx < nseg) {
                    const Segment& sg = seg[sx];
                    const int vec_per_row = a.cols / 16;
                    const int n = sg.G * 8 * vec_per_row;
#pragma unroll 4
                    for (int i = threadIdx.x; i < n; i += nthreads) {
                        const int j = i / vec_per_row, v = i - j * vec_per_row;
                        const uint32_t p = sg.base + sg.sg0 + min(j, sg.ntok - 1);
                        const uint32_t row = GATE_UP ? a.slot_token[p] : p;
                        const uint4 val = *reinterpret_cast<const uint4*>(a.xq + size_t(row) * a.cols + v * 16);
                        *reinterpret_cast<uint4*>(smem + L.xq(sx) + j * f.x_stride + v * 16) = val;
                    }
                }
            }
#pragma unroll
            for (int sx = 0; sx < F_XBUF; sx++) {
                if (sx < nseg) {
                    // Scales transposed to [block][token]; token fastest, so stores do not
                    // conflict. Each thread looks its token's row up itself.
                    const Segment& sg = seg[sx];
                    const int n = nb * sg.G * 8;
                    float* xsT = reinterpret_cast<float*>(smem + L.xsT(sx));
                    float* xsumT = reinterpret_cast<float*>(smem + L.xsumT(sx));
#pragma unroll 2
                    for (int i = threadIdx.x; i < n; i += nthreads) {
                        const int b = i / (sg.G * 8), j = i - b * (sg.G * 8);
                        const uint32_t p = sg.base + sg.sg0 + min(j, sg.ntok - 1);
                        const uint32_t row = GATE_UP ? a.slot_token[p] : p;
                        const size_t src = size_t(row) * f.nbp + b;
                        xsT[b * F_TOK + j] = a.xs[src];
                        if (KIND == 2) xsumT[b * F_TOK + j] = a.xsum[src];
                    }
                }
            }
            __syncthreads();
            asm volatile("mov.u32 %0, %1;" : "=r"(xtok) : "r"(xphase) : "memory");
        }
        // ---- this warp's units of the group's segments
        for (int sx = 0; sx < nseg; sx++) {
            const Segment& sg = seg[sx];
            const uint32_t xq_s = smem_addr(smem + L.xq(sx)), xsT_s = smem_addr(smem + L.xsT(sx)),
                           xsumT_s = smem_addr(smem + L.xsumT(sx));
            while (ok && cons.valid && cons.ai == sg.ai && cons.sg0 == sg.sg0) {
                if (fills - takes < uint32_t(STAGES)) fill_next();
                if (cons.c == 0) {
#pragma unroll
                    for (int nt = 0; nt < F_GMAX; nt++) {
                        acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
                        off[nt][0] = off[nt][1] = off[nt][2] = off[nt][3] = 0.0f;
                    }
                }
                const uint32_t stage = takes % STAGES;
                const bool landed = mbar_wait_bounded(bars + stage, (takes / STAGES) & 1);
                if (!__all_sync(0xffffffffu, landed)) {
                    ok = false;
                    break;
                }
                const uint32_t wtok = uint32_t(landed);
                const uint32_t rec = smem_addr(ring + stage * R::BYTES);
                const int nblk = min(F_NBC, nb - cons.c * F_NBC);
                const int blk0 = cons.c * F_NBC;
                if (sg.G == 1)
                    fast_chunk<KIND, 1, F_GMAX>(rec, xq_s, xsT_s, xsumT_s, f.x_stride, nblk, blk0, lane, wtok, xtok, acc, off);
                else if (sg.G == 2)  // (0: an expert without tokens in a dense walk; its records are only drained)
                    fast_chunk<KIND, 2, F_GMAX>(rec, xq_s, xsT_s, xsumT_s, f.x_stride, nblk, blk0, lane, wtok, xtok, acc, off);
                __syncwarp();

                if (cons.c == wk.nchunks - 1) {
                    const int u = cons.a - sg.ai * upe;
#pragma unroll
                    for (int nt = 0; nt < F_GMAX; nt++) {
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            const int j = nt * 8 + 2 * t + i;
                            if (nt < sg.G && j < sg.ntok) {
                                float y0 = acc[nt][i], y1 = acc[nt][2 + i];  // rows g and g+8
                                if (KIND == 2) {
                                    y0 = y0 + off[nt][i];
                                    y1 = y1 + off[nt][2 + i];
                                }
                                size_t p = sg.base + sg.sg0 + j;
                                if (!GATE_UP && a.out_rows) p = a.out_rows[p];
                                if (GATE_UP) {
                                    const int col = u * 8 + g;
                                    if (col < a.out_cols) {
                                        const float ex = exp_poly(-y0);
                                        a.out[p * a.out_cols + col] = __fdiv_rn(y0, 1.0f + ex) * y1;
                                    }
                                } else {
                                    const int r0 = u * F_ROWS + g;
                                    float* dst = a.out;
                                    if (a.peer_out[0]) {  // the row's home rank's buffer, over NVLink
                                        const uint32_t home = uint32_t(p) / a.peer_rows;
                                        dst = a.peer_out[home];
                                        p -= size_t(home) * a.peer_rows;
                                    }
                                    if (r0 < a.out_cols) dst[p * a.out_cols + r0] = y0;
                                    if (r0 + 8 < a.out_cols) dst[p * a.out_cols + r0 + 8] = y1;
                                }
                            }
                        }
                    }
                }
                takes++;
                wk.advance(cons);
            }
        }
        // Keep the decision to stop uniform across the CTA's barriers.
        ok = __syncthreads_and(ok);
    }
    if (!GATE_UP && a.peer_ranks) {
        // Rows went into other ranks' windows. Order this CTA's stores before its ticket
        // (CTA barrier, then a cumulative system-scope fence); the last CTA to arrive then
        // release-stores the next value of this rank's counter into every rank's flag.
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            if (atomicAdd(a.peer_ticket, 1u) == gridDim.x - 1) {
                *a.peer_ticket = 0;  // ready for the next launch
                __threadfence_system();
                const uint32_t e = *a.peer_epoch + 1;
                *a.peer_epoch = e;
                for (int r = 0; r < a.peer_ranks; r++)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.peer_flag[r]), "r"(e) : "memory");
            }
        }
    }
    if (!ok) {
        if (threadIdx.x == 0) atomicExch(a.status, ERR_COPY_WAIT_TIMEOUT);
        // Give copies already in flight a bounded chance to land before the
        // shared memory they target is released.
        for (uint32_t k = takes; k < fills; k++) mbar_wait_bounded(bars + k % STAGES, (k / STAGES) & 1);
    }
}

// Builds the records from a matrix in Tachyon's row-major layout. One CTA per
// record; rows or blocks past the matrix's edge are zero.
template <int KIND, bool GATE_UP>
__global__ void tile_weights_kernel(const uint8_t* __restrict__ wdata, const void* __restrict__ wscales,
                                    int cols, int rows_per_expert, int upe, int nchunks,
                                    uint8_t* __restrict__ tiled) {
    using R = Rec<KIND>;
    const size_t rec_index = blockIdx.x;
    const int c = int(rec_index % nchunks);
    const int u = int((rec_index / nchunks) % upe);
    const int e = int(rec_index / nchunks / upe);
    uint8_t* rec = tiled + rec_index * R::BYTES;
    const int nb = cols / QK;
    for (int i = threadIdx.x; i < R::BYTES / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(rec)[i] = 0;
    __syncthreads();
    for (int r = 0; r < F_ROWS; r++) {
        int row;
        if (GATE_UP) {
            const int inter = rows_per_expert / 2, col = u * 8 + (r & 7);
            row = col < inter ? e * rows_per_expert + (r < 8 ? 0 : inter) + col : -1;
        } else {
            const int rr = u * F_ROWS + r;
            row = rr < rows_per_expert ? e * rows_per_expert + rr : -1;
        }
        if (row < 0) continue;
        const int col0 = c * F_KC, cols_c = min(F_KC, cols - col0);
        const int nblk = cols_c / QK;
        if (KIND == 1) {
            for (int i = threadIdx.x; i < cols_c; i += blockDim.x)
                rec[r * R::ROW_STRIDE + i] = wdata[size_t(row) * cols + col0 + i];
            const uint16_t* sp = reinterpret_cast<const uint16_t*>(wscales) + size_t(row) * nb + c * F_NBC;
            for (int b = threadIdx.x; b < nblk; b += blockDim.x)
                reinterpret_cast<uint16_t*>(rec + r * R::ROW_STRIDE + F_KC)[b] = sp[b];
        } else {
            for (int i = threadIdx.x; i < cols_c / 2; i += blockDim.x)
                rec[r * R::ROW_STRIDE + i] = wdata[(size_t(row) * cols + col0) / 2 + i];
            const int words_per_row = (nb + SUPER - 1) / SUPER * SUPER_WORDS;
            const uint32_t* wp = reinterpret_cast<const uint32_t*>(wscales) + size_t(row) * words_per_row +
                                 c * SUPER_WORDS;
            if (threadIdx.x < 4)
                reinterpret_cast<uint32_t*>(rec + r * R::ROW_STRIDE + F_KC / 2)[threadIdx.x] = wp[threadIdx.x];
            if (threadIdx.x == 4) reinterpret_cast<uint32_t*>(rec + F_ROWS * R::ROW_STRIDE)[r] = wp[4];
        }
    }
}

// Warps per CTA and ring depth: as many warps as possible while each still gets
// a ring of at least three stages (two copies in flight behind the one in use).
template <int KIND>
bool pick_config(int cols, int nbp, int& nwarps, int& stages) {
    int best_w = 0, best_s = 0;
    for (int w = F_MAX_WARPS; w >= 8; w -= 2) {
        int s = 0;
        for (int k = F_MAX_STAGES; k >= 2; k--)
            if (size_t(Layout<KIND>(w, k, cols, nbp).total) <= F_SMEM_LIMIT) {
                s = k;
                break;
            }
        if (s >= 3) {
            nwarps = w;
            stages = s;
            return true;
        }
        if (s > best_s) {
            best_s = s;
            best_w = w;
        }
    }
    nwarps = best_w;
    stages = best_s;
    return best_s >= 2;
}

template <int KIND, bool GATE_UP>
int launch_fast(const ExpertArgs& e, const uint8_t* tiled, int sms, bool dense, cudaStream_t stream) {
    FastArgs f;
    f.e = e;
    f.dense = dense ? 1 : 0;
    f.tiled = tiled;
    f.nbp = (e.cols / QK + SUPER - 1) / SUPER * SUPER;
    f.x_stride = e.cols + 16;
    int nwarps = 0;
    if (!pick_config<KIND>(e.cols, f.nbp, nwarps, f.stages)) return -1;
    const int total_units = e.experts * e.units_per_expert;
    int grid = e.runs.expert ? sms : min(sms, total_units);  // (runs: at least as many tasks as units)
    if (grid < 1) grid = 1;
    const Layout<KIND> L(nwarps, f.stages, e.cols, f.nbp);
    launch_overlapped(expert_fast_kernel<KIND, GATE_UP>, dim3(grid), dim3(nwarps * 32), size_t(L.total), stream, f);
    return 1;
}

template <int KIND, bool GATE_UP>
void run_tiling(const ExpertArgs& e, uint8_t* tiled, cudaStream_t stream) {
    const int nchunks = (e.cols + F_KC - 1) / F_KC;
    const size_t recs = size_t(e.experts) * e.units_per_expert * nchunks;
    tile_weights_kernel<KIND, GATE_UP><<<unsigned(recs), 128, 0, stream>>>(
        e.wdata, e.wscales, e.cols, e.rows_per_expert, e.units_per_expert, nchunks, tiled);
}

}  // namespace

void init_kernels_fast() {
    const int lim = int(F_SMEM_LIMIT);
    cudaFuncSetAttribute(expert_fast_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(expert_fast_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(expert_fast_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(expert_fast_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
}

size_t tiled_bytes(const MoeDims& d, const MatrixDev& m, bool gate_up) {
    const int cols = gate_up ? d.hidden : d.inter;
    const int upe = gate_up ? (d.inter + 7) / 8 : (d.hidden + 15) / 16;
    const int nchunks = (cols + F_KC - 1) / F_KC;
    const size_t rec = m.kind == 1 ? Rec<1>::BYTES : Rec<2>::BYTES;
    return size_t(d.experts) * upe * nchunks * rec;
}

bool fast_path_fits(const MoeDims& d, const MatrixDev& gate_up, const MatrixDev& down) {
    const int nbp_h = (d.hidden / QK + 7) / 8 * 8, nbp_i = (d.inter / QK + 7) / 8 * 8;
    int w = 0, st = 0;
    const bool g = gate_up.kind == 1 ? pick_config<1>(d.hidden, nbp_h, w, st) : pick_config<2>(d.hidden, nbp_h, w, st);
    const bool dn = down.kind == 1 ? pick_config<1>(d.inter, nbp_i, w, st) : pick_config<2>(d.inter, nbp_i, w, st);
    return g && dn;
}

void tile_weights(const MoeDims& d, const MatrixDev& m, bool gate_up, uint8_t* tiled, cudaStream_t stream) {
    Workspace none;
    const ExpertArgs e = gate_up ? gate_up_args(d, m, none) : down_args(d, m, none);
    if (gate_up) {
        if (m.kind == 1) run_tiling<1, true>(e, tiled, stream);
        else run_tiling<2, true>(e, tiled, stream);
    } else {
        if (m.kind == 1) run_tiling<1, false>(e, tiled, stream);
        else run_tiling<2, false>(e, tiled, stream);
    }
}

namespace {
// One CTA: expert e with m slots becomes ceil(m / F_TOK) runs.
__global__ void build_runs_kernel(const uint32_t* __restrict__ counts, const uint32_t* __restrict__ offsets,
                                  int experts, RunList runs) {
    __shared__ int s_first[MAX_EXPERTS + 1];
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < experts; e++) {
            s_first[e] = run;
            run += (int(counts[e]) + F_TOK - 1) / F_TOK;
        }
        s_first[experts] = run;
        *runs.n = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const uint32_t m = counts[e], base = offsets[e];
        for (uint32_t i = 0; i * F_TOK < m; i++) {
            const int r = s_first[e] + int(i);
            runs.expert[r] = e;
            runs.count[r] = min(uint32_t(F_TOK), m - i * F_TOK);
            runs.offset[r] = base + i * F_TOK;
        }
    }
}
}  // namespace

int launch_build_runs(const uint32_t* counts, const uint32_t* offsets, int experts, const RunList& runs,
                      cudaStream_t stream) {
    build_runs_kernel<<<1, 256, 0, stream>>>(counts, offsets, experts, runs);
    return 1;
}

int launch_gate_up_fast(const MoeDims& d, const MatrixDev& m, const uint8_t* tiled, int t, Workspace& ws,
                        int sms, cudaStream_t stream) {
    (void)t;
    const ExpertArgs a = gate_up_args(d, m, ws);
    const bool dense = !ws.runs.expert && (dense_walk(d, t) || !ws.active);
    return m.kind == 1 ? launch_fast<1, true>(a, tiled, sms, dense, stream)
                       : launch_fast<2, true>(a, tiled, sms, dense, stream);
}

int launch_down_fast(const MoeDims& d, const MatrixDev& m, const uint8_t* tiled, int t, Workspace& ws,
                     int sms, cudaStream_t stream) {
    ExpertArgs a = down_args(d, m, ws);
    a.xf = ws.hidden_f;  // quantized while staged: no separate pass over the SwiGLU rows
    const bool dense = dense_walk(d, t);
    return m.kind == 1 ? launch_fast<1, false>(a, tiled, sms, dense, stream)
                       : launch_fast<2, false>(a, tiled, sms, dense, stream);
}

// The down projection with each output row written to out_rows[slot] (expert
// parallelism: the row's place in the receive order).
int launch_down_fast_rows(const MoeDims& d, const MatrixDev& m, const uint8_t* tiled, Workspace& ws,
                          const uint32_t* out_rows, int sms, cudaStream_t stream, float* const* peer_out,
                          int ranks, uint32_t peer_rows, uint32_t* const* peer_flag, uint32_t* peer_epoch,
                          uint32_t* peer_ticket) {
    ExpertArgs a = down_args(d, m, ws);
    a.xf = ws.hidden_f;
    a.out_rows = out_rows;
    for (int r = 0; r < ranks && r < MAX_PEERS; r++) a.peer_out[r] = peer_out[r];
    a.peer_rows = peer_rows;
    if (peer_flag) {
        for (int r = 0; r < ranks && r < MAX_PEERS; r++) a.peer_flag[r] = peer_flag[r];
        a.peer_epoch = peer_epoch;
        a.peer_ticket = peer_ticket;
        a.peer_ranks = ranks;
    }
    const bool dense = !ws.runs.expert && !ws.active;  // a caller without a list of non-empty experts
    return m.kind == 1 ? launch_fast<1, false>(a, tiled, sms, dense, stream)
                       : launch_fast<2, false>(a, tiled, sms, dense, stream);
}

}  // namespace tc

