// The whole MoE block of a decode-size batch (up to 32 tokens; up to 128 in the run-walking
// form described further down) as ONE kernel:
// [RMSNorm +] router + top-k + gates + row quantization, gate_up + SwiGLU, down,
// weighted combine + residual add, by persistent CTAs (one per SM) that meet at
// three grid-wide arrival counters instead of at kernel boundaries.
//
// Why one kernel. At these sizes the block is a chain of short dependent steps around
// one large stream of bytes (the selected experts' weights, read once). As four
// launches, each step paid a launch boundary and its own ramp, and HBM idled through
// the router and the combine. Here the weight stream is decoupled from the steps:
//  - Every warp owns a private ring of shared-memory stages and a fixed sequence of
//    weight records: its 16-row units of gate_up, then its units of down. Lane 0
//    keeps the ring full with bulk async copies (cp.async.bulk + mbarrier); the copies
//    for the next step land while the current one computes.
//  - For batches that reach nearly every expert (dense_walk) the partition of units
//    over CTAs and warps does not depend on the routing, so the ring starts filling
//    before the kernel even waits for the previous kernel in the stream
//    (programmatic dependent launch), and keeps filling through the router phase.
//    Smaller batches walk only the experts that were picked: their sequence is known
//    after the router phase.
//  - The router phase runs on CTAs 0..t-1 (a token each); the others only stream.
//    The combine runs on the same CTAs; the rest have exited by then, which lets the
//    next block's kernel start streaming its weights under this block's combine.
//
// Partition. The 16-row units of the walked experts are cut over the CTAs so that a CTA stays
// inside one expert wherever that costs no extra wave of units per warp (an expert's units over
// nctas / experts CTAs, the CTAs left over idle): a CTA whose units span two experts lists and
// stages two experts' tokens, and every phase waits for its slowest CTA. A CTA's units go round
// its warps; 16 warps per CTA where each still gets a ring of two stages.
//
// Run-walking form (template parameter EP): experts sharded over the GPUs of one node, or one
// GPU with 33 to 128 tokens. An expert's slots are cut into runs of up to 32, 16 or 8 tokens
// (the length with the least work on the busiest warp), the (run, unit) pairs are what CTAs and
// warps share out, every CTA stays inside one run, and the run's slot list is built by all
// warps of the CTA. Rows, ids and expert outputs travel through per-rank windows (peer memory
// over NVLink, or local memory when there is one rank) and the rendezvous are system-scope
// counters in those windows that only grow. Which records a warp needs depends on the routing
// there, so nothing is copied into shared memory before the router phase; the rank's share of
// the layer is asked into L2 instead.
//
// No token -> expert permutation is built: with at most 32 tokens every CTA keeps
// the batch's expert ids in shared memory and lists, per expert of its range, the
// (token, pick) slots that named it (ascending tokens, the order of the per-expert
// lists of src/model.rs:474-482). SwiGLU rows and expert outputs are stored by slot
// (token * k + pick).
//
// Arithmetic: identical to the grouped kernels (experts_fast.cuh: one fma chain per
// output over the exact integer block sums), the router and quantization of
// route_common.cuh, and the combine order of combine.cu (ascending expert, product
// rounded then added: src/model.rs:513-519, src/kernels.rs:606-610), so a token's
// output has the same bits whichever path ran.
//
// Every wait is bounded: staged copies (mbar_wait_bounded) and the grid-wide counters
// (grid_wait). A wait that runs out sets the status word, and the CTA skips to the end,
// waits (bounded) for its copies in flight and returns; tc_sync reports it and clears
// the counters.
#include "experts_fast.cuh"
#include "route_common.cuh"

namespace tc {

namespace {

constexpr int D_MAX_WARPS = 16;
constexpr int D_MAX_STAGES = 8;
constexpr int D_GMAX = 4;          // token tiles of 8 held in registers
constexpr int D_TOK = 8 * D_GMAX;  // tokens per block this kernel takes; rows staged at a time
constexpr int D_NORM_HELD = 8;     // elements of the norm's weight a thread holds (rows of up to 8 x 256 floats)
constexpr int D_ROUTE_VEC = 10;    // 16-byte pieces of the router matrix a thread holds at a time
constexpr int D_NSEG = 4;          // experts of a CTA's range whose slot lists are held at a time
constexpr size_t D_SMEM_LIMIT = 227 * 1024 - 3072;  // dynamic part: the kernel also has up to 2.5 KB of static shared memory

constexpr int DECODE_EP_FLAG_ROUTE = 16, DECODE_EP_FLAG_DOWN = 17;  // words of the window's flag area

struct DecodeArgs {
    // router phase
    const uint16_t* router;
    const float* bias;
    const float* x;       // [t, hidden] normed input, or the residual stream when norm_w is set
    const float* norm_w;
    float eps;
    float* y;             // [t, hidden] residual stream: y += moe(x)
    int t, hidden, experts, topk, inter;
    float* logits;
    uint32_t* ids;
    float* gates;
    int8_t* xq;
    float* xs;
    float* xsum;
    // expert phases
    const uint8_t* gu_tiled;  // records [expert][unit][chunk]
    const uint8_t* dn_tiled;
    float* hidden_f;          // [t * k, inter] SwiGLU rows by slot
    float* out;               // [t * k, hidden] expert outputs by slot
    int stages, xcap;         // ring depth per warp; staged rows at a time (a multiple of 8, at most D_TOK)
    int route_rows;           // rows of the router matrix staged at a time in the router phase
    int l2_all;               // ask all of this GPU's expert records into L2 before the router phase
    int dense;
    uint32_t* sync;           // [GRID_SYNC_WORDS], zero between launches
    DecodeEp ep;              // ranks > 0: experts sharded over the GPUs of one node (see DecodeEp)
    int ids_slots;            // (token, pick) slots the block's ids take in shared memory
    uint32_t spin_limit;
    int* status;
    unsigned long long* stamps;  // when set: CTA 0 stores the wall clock (ns) at its phase boundaries [8]
};

// Shared memory carve-up (bytes). The token area is reused by the phases: the router's
// row and logits, then gate_up's staged rows, then down's.
template <int KIND>
struct DLayout {
    int ring, x0, xbytes, ids, lists, bars, total;
    __host__ __device__ static int token_bytes(int xcap, int hidden, int inter) {
        const int cols = hidden > inter ? hidden : inter;
        const int nbp = (cols / QK + 7) / 8 * 8;
        return xcap * (cols + 16) + nbp * D_TOK * 4 * (KIND == 2 ? 2 : 1);
    }
    __host__ __device__ static int route_base(int hidden, int experts) { return ((hidden + experts) * 4 + 127) / 128 * 128; }
    __host__ __device__ DLayout(int nwarps, int stages, int xcap, int route_rows, int hidden, int inter, int experts,
                                int topk, int ids_slots) {
        int o = nwarps * stages * Rec<KIND>::BYTES;
        ring = 0;
        o = (o + 127) / 128 * 128;
        x0 = o;
        xbytes = token_bytes(xcap, hidden, inter);
        // The router phase keeps the token's row, its logits and route_rows rows of the router matrix here.
        // (or, once the logits are done, the token's 8-bit row and scales on their way to the other ranks)
        const int row_bytes = hidden + 2 * 4 * ((hidden / QK + 7) / 8 * 8);
        const int staged = route_rows * (2 * hidden + 32);
        const int route_bytes = route_base(hidden, experts) + (staged > row_bytes ? staged : row_bytes) + 64;
        if (xbytes < route_bytes) xbytes = route_bytes;
        xbytes = (xbytes + 127) / 128 * 128;
        o += xbytes;
        ids = o;
        o += ids_slots * 4;
        lists = o;
        o += D_NSEG * D_TOK * 2 * 2;
        o = (o + 15) / 16 * 16;
        bars = o;
        o += D_MAX_WARPS * D_MAX_STAGES * 8;
        total = o;
    }
};

__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One thread: waits until *ctr >= target, at most `limit` polls.
__device__ __forceinline__ bool grid_wait(const uint32_t* ctr, uint32_t target, uint32_t limit) {
    for (uint32_t i = 0; i < limit; i++) {
        if (ld_acquire(ctr) >= target) return true;
        __nanosleep(32);
    }
    return false;
}

// Loads whose place in the program matters: requested early and used much later. (A plain
// read-only load may be re-issued by the compiler next to its use instead of being kept
// in registers, which would put the trip to memory back on the critical path.)
__device__ __forceinline__ uint4 load_now_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float load_now_f32(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ unsigned long long wall_clock_ns() {
    unsigned long long v;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
    return v;
}

// After a CTA barrier: a release at GPU scope orders this CTA's writes so far (cumulatively,
// through the barrier) before its arrival.
__device__ __forceinline__ void grid_arrive(uint32_t* ctr) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
}

// What one of the two expert phases needs to know about its matrix and this warp's share.
struct Phase {
    const uint8_t* tiled;
    int cols, upe, nchunks, nb, nbp, x_stride;
    int lo, hi;        // this CTA's units, in walk space (all experts, or the picked ones)
    int first, n;      // this warp's first unit and how many it owns (stride nwarps)
};

__device__ __forceinline__ void arrive_on_peer(uint32_t* flag) {
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(flag) : "memory");
}
// One thread: waits until the counter (written by other GPUs) has reached target, wrap-safe.
__device__ __forceinline__ bool peer_count_wait(const uint32_t* ctr, uint32_t target, uint32_t limit) {
    for (uint32_t i = 0; i < limit; i++) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(ctr) : "memory");
        if (int32_t(seen - target) >= 0) return true;
        __nanosleep(i < 64 ? 32 : 256);
    }
    return false;
}

template <int KIND, bool EP>
__global__ void __launch_bounds__(D_MAX_WARPS * 32, 1) moe_decode_kernel(const DecodeArgs a) {
    using R = Rec<KIND>;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float s_inv;
    __shared__ int s_abort;
    __shared__ int s_nactive;
    __shared__ int s_seg_count[D_NSEG];
    __shared__ uint8_t s_picked[MAX_EXPERTS];
    constexpr int MAX_RUNS = EP ? MAX_EXPERTS + 4096 / 8 / 8 : MAX_EXPERTS;  // (experts + slots / shortest run)
    __shared__ uint16_t s_active[MAX_RUNS];     // walk index -> expert (sparse walk); EP: -> the run's expert
    __shared__ uint16_t s_skip[EP ? MAX_RUNS : 1];      // EP: slots of that expert in earlier runs
    __shared__ int s_run_len;                           // EP: slots per run (32, 16 or 8)
    __shared__ uint32_t s_cnt[EP ? MAX_EXPERTS : 1];    // EP: slots per local expert
    __shared__ int s_part[EP ? D_NSEG * D_MAX_WARPS : 1];  // EP: a segment's hits per warp's slice of the ids
    __shared__ uint32_t s_rids[MAX_TOPK];               // the routed token's picks, on their way out
    __shared__ uint32_t s_cpos[MAX_TOPK];
    __shared__ float s_cgate[MAX_TOPK];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nwarps = blockDim.x >> 5, nthreads = blockDim.x;
    const int bid = blockIdx.x, nctas = gridDim.x;
    const int STAGES = a.stages;
    const int t = a.t, hidden = a.hidden, experts = a.experts, topk = a.topk, inter = a.inter;
    // Expert parallel: the expert phases see every rank's tokens (gathered in this rank's window).
    const int ranks = EP ? a.ep.ranks : 1, own = EP ? a.ep.me * t : 0;  // own: this rank's first token among all
    const int slots = ranks * t * topk;
    uint8_t* window = EP ? a.ep.base[a.ep.me] : nullptr;
    const int8_t* xq_all = EP ? reinterpret_cast<const int8_t*>(window + a.ep.off_xq) : a.xq;
    const float* xs_all = EP ? reinterpret_cast<const float*>(window + a.ep.off_xs) : a.xs;
    const float* xsum_all = EP ? reinterpret_cast<const float*>(window + a.ep.off_xsum) : a.xsum;
    const uint32_t* ids_all = EP ? reinterpret_cast<const uint32_t*>(window + a.ep.off_ids) : a.ids;
    const float* out_own = EP ? reinterpret_cast<const float*>(window + a.ep.off_out) : a.out;
    const uint32_t* flags = EP ? reinterpret_cast<const uint32_t*>(window + a.ep.off_flags) : nullptr;
    uint32_t epoch0 = 0;  // EP: blocks completed before this one
    uint32_t routed0 = 0; // EP: router-phase arrivals of those blocks (ranks x tokens each; the batch size may change)
    const DLayout<KIND> L(nwarps, STAGES, a.xcap, a.route_rows, hidden, inter, experts, topk, a.ids_slots);
    uint8_t* ring = smem + L.ring + size_t(warp) * STAGES * R::BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bars) + warp * D_MAX_STAGES;
    uint32_t* s_ids = reinterpret_cast<uint32_t*>(smem + L.ids);
    uint16_t* s_slot = reinterpret_cast<uint16_t*>(smem + L.lists);  // [D_NSEG][D_TOK] slots that named the segment's expert
    uint16_t* s_tok = s_slot + D_NSEG * D_TOK;                        // the same slots' tokens
    if (lane == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(bars + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (tid == 0) s_abort = 0;
    __syncthreads();
    grid_launch_dependents();
    const bool stamping = a.stamps && bid == 0 && tid == 0;
    if (stamping) a.stamps[0] = wall_clock_ns();

    // ---- the two expert phases and this warp's record sequence: gate_up records, then down's
    Phase P0, P1;
    P0.tiled = a.gu_tiled, P0.cols = hidden, P0.upe = (inter + 7) / 8;
    P1.tiled = a.dn_tiled, P1.cols = inter, P1.upe = (hidden + 15) / 16;
    auto derive = [&](Phase& P) {
        P.nchunks = (P.cols + F_KC - 1) / F_KC;
        P.nb = P.cols / QK;
        P.nbp = (P.nb + 7) / 8 * 8;
        P.x_stride = P.cols + 16;
    };
    derive(P0), derive(P1);
    auto share = [&](Phase& P, unsigned walk_experts) {  // (bid + 1) * total stays far below 2^32
        const unsigned total = walk_experts * unsigned(P.upe);
        // Every CTA inside one expert (or run) where that costs no extra wave of units per warp: a
        // CTA whose units span two experts lists and stages tokens twice, and the whole grid then
        // waits for it. The expert's units are cut into as many equal parts as there are whole
        // CTAs per expert; the CTAs left over stay idle. (granite-1b-a400m, batch 32: 4 CTAs of
        // 16 units per expert on 128 of the 148 SMs, 0.80 ms per step against 0.83 with 13.8
        // units on every SM.)
        bool inside = walk_experts > 0 && walk_experts <= unsigned(nctas);
        if (inside && !EP) {
            const unsigned per_run = unsigned(nctas) / walk_experts;
            const unsigned mine = (unsigned(P.upe) + per_run - 1) / per_run, even = (total + nctas - 1) / unsigned(nctas);
            inside = (mine + nwarps - 1) / nwarps <= (even + nwarps - 1) / nwarps;
        }
        if (inside) {
            const unsigned per_run = unsigned(nctas) / walk_experts, run = unsigned(bid) / per_run,
                           part = unsigned(bid) % per_run;
            if (run < walk_experts) {
                P.lo = int(run * unsigned(P.upe) + part * unsigned(P.upe) / per_run);
                P.hi = int(run * unsigned(P.upe) + (part + 1) * unsigned(P.upe) / per_run);
            } else {
                P.lo = P.hi = 0;
            }
        } else {
            P.lo = int(unsigned(bid) * total / unsigned(nctas));
            P.hi = int(unsigned(bid + 1) * total / unsigned(nctas));
        }
        P.first = P.lo + warp;
        P.n = P.first < P.hi ? (P.hi - P.first + nwarps - 1) / nwarps : 0;
    };
    // Where a unit's records start. Walk space counts the units of all experts (dense) or of
    // the picked ones (then the expert comes from the list made after the router phase).
    auto unit_ptr = [&](const Phase& P, int wu) {
        size_t flat = size_t(wu);
        if (!a.dense) flat = size_t(s_active[wu / P.upe] - (EP ? a.ep.first : 0)) * P.upe + wu % P.upe;
        return P.tiled + flat * P.nchunks * R::BYTES;
    };
    // Producer state: the next record's address, and what is left of its unit and phase.
    uint32_t fills = 0, takes = 0, nrec = 0;
    const uint64_t stream_policy = l2_evict_first_policy();
    const uint8_t* pptr = nullptr;
    int pphase = 0, pwu = 0, pchunks = 0, punits = 0, pslot = 0;
    auto start_phase = [&](int p) {
        pphase = p;
        const Phase& P = p ? P1 : P0;
        pwu = P.first, pchunks = P.nchunks, punits = P.n;
        if (P.n > 0) pptr = unit_ptr(P, pwu);
    };
    // Requests records until the ring is full or the sequence ends.
    auto top_up = [&]() {
#pragma unroll 1
        while (fills < nrec && fills - takes < uint32_t(STAGES)) {
            if (lane == 0) {
                mbar_expect_tx(bars + pslot, R::BYTES);
                bulk_copy_once(ring + pslot * R::BYTES, pptr, R::BYTES, bars + pslot, stream_policy);
            }
            fills++;
            pslot = pslot + 1 == STAGES ? 0 : pslot + 1;
            pptr += R::BYTES;
            if (--pchunks == 0) {
                const Phase& P = pphase ? P1 : P0;
                if (--punits > 0) {
                    pwu += nwarps;
                    pchunks = P.nchunks;
                    pptr = a.dense ? pptr + size_t(nwarps - 1) * P.nchunks * R::BYTES : unit_ptr(P, pwu);
                } else if (pphase == 0) {
                    start_phase(1);
                }
            }
        }
    };

    // ---- router phase, part one (constants only): CTA i < t takes token i. The router matrix
    // is staged in shared memory beside the token's row, route_rows rows at a time (rows
    // padded by 32 bytes, so the four-thread groups of a half-warp read distinct banks),
    // through registers: every thread requests its 16-byte pieces of the next part before
    // the current part is used, so a part costs one trip to memory, and the first trip is
    // made before this grid waits for the one in front of it. The norm's weight goes to
    // registers the same way.
    float* xrow = reinterpret_cast<float*>(smem + L.x0);
    float* slog = xrow + hidden;
    const int wstride = 2 * hidden + 32;
    uint8_t* wsm = smem + L.x0 + DLayout<KIND>::route_base(hidden, experts);
    const int pass_rows = a.route_rows > 0 ? a.route_rows : experts;  // (0: the logits read global memory)
    const int vec_per_wrow = hidden / 8;  // 16-byte pieces of a router row
    float nw[D_NORM_HELD];
    uint4 rv[D_ROUTE_VEC];
    auto request_router_rows = [&](int e_lo) {
        const int n = a.route_rows > 0 ? min(pass_rows, experts - e_lo) * vec_per_wrow : 0;
        const uint4* src = reinterpret_cast<const uint4*>(a.router + size_t(e_lo) * hidden);
#pragma unroll
        for (int k = 0; k < D_ROUTE_VEC; k++) {
            const int i = tid + k * nthreads;
            if (i < n) rv[k] = load_now_v4(src + i);
        }
    };
    auto store_router_rows = [&](int e_lo) {
        const int n = min(pass_rows, experts - e_lo) * vec_per_wrow;
        int r = tid / vec_per_wrow, v = tid - r * vec_per_wrow;  // piece tid + k * nthreads = (row r, piece v)
        const int dr = nthreads / vec_per_wrow, dv = nthreads - dr * vec_per_wrow;
#pragma unroll
        for (int k = 0; k < D_ROUTE_VEC; k++) {
            if (tid + k * nthreads < n) *reinterpret_cast<uint4*>(wsm + size_t(r) * wstride + v * 16) = rv[k];
            r += dr, v += dv;
            if (v >= vec_per_wrow) v -= vec_per_wrow, r++;
        }
    };
    const bool routing = bid < t;
    // Every CTA starts its stream here when the partition does not depend on the routing
    // (dense walk): the ring fills before this grid waits for the kernel in front of it, and
    // through the router phase. Otherwise after the router phase, once the picked experts are known.
    bool streaming = false;
#pragma unroll 1
    for (int pass = 0; pass < 2; pass++) {
        if (pass == 0 ? bool(a.dense) : !streaming) {
            if (pass == 1 && s_abort) break;
            const unsigned walk = a.dense ? unsigned(experts) : unsigned(s_nactive);
            share(P0, walk), share(P1, walk);
            nrec = uint32_t(P0.n * P0.nchunks + P1.n * P1.nchunks);
            start_phase(P0.n > 0 ? 0 : 1);
            top_up();
            streaming = true;
        }
        if (pass == 1) break;
        if (a.l2_all) {
            // Which records a warp needs is only known after the router phase (expert parallel, or a
            // batch small enough to walk only the picked experts), but most experts will be picked:
            // all of this GPU's share of the layer is asked into L2 now (every CTA a slice), and the
            // copies into shared memory that follow the router phase find it there.
            const Phase* Ps[2] = {&P0, &P1};
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const size_t bytes = size_t(EP ? a.ep.local : experts) * Ps[q]->upe * Ps[q]->nchunks * R::BYTES;
                const size_t piece = 4096, pieces = (bytes + piece - 1) / piece;
                for (size_t i = size_t(bid) * nthreads + tid; i < pieces; i += size_t(nctas) * nthreads) {
                    const size_t at = i * piece, n = min(piece, bytes - at) & ~size_t(15);
                    if (n)
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(Ps[q]->tiled + at), "r"(uint32_t(n))
                                     : "memory");
                }
            }
        }
        if (routing) {
            // Part 0 of the router matrix goes all the way into shared memory before the wait,
            // part 1 (if any) into registers.
            request_router_rows(0);
            if (a.route_rows > 0) store_router_rows(0);
            if (a.route_rows > 0 && pass_rows < experts) request_router_rows(pass_rows);
            if (a.norm_w) {
#pragma unroll
                for (int k = 0; k < D_NORM_HELD; k++) {
                    const int c = tid + k * nthreads;
                    nw[k] = c < hidden ? load_now_f32(a.norm_w + c) : 0.0f;
                }
            }
        }
        grid_dependency_wait();  // everything below reads or writes what other kernels touch
        if (stamping) a.stamps[1] = wall_clock_ns();

        // ---- router phase, part two
        if (routing) {
            const float* xin = a.x + size_t(bid) * hidden;
#pragma unroll 1
            for (int c = tid * 4; c < hidden; c += nthreads * 4)
                *reinterpret_cast<float4*>(xrow + c) = *reinterpret_cast<const float4*>(xin + c);
            __syncthreads();
            if (a.norm_w) {
                if (warp == 0) {
                    const float ss = __fdiv_rn(sum_squares_avx_order(xrow, hidden, lane), float(hidden));
                    if (lane == 0) s_inv = __fdiv_rn(1.0f, __fsqrt_rn(ss + a.eps));
                }
                __syncthreads();
                const float inv = s_inv;
#pragma unroll
                for (int k = 0; k < D_NORM_HELD; k++) {
                    const int c = tid + k * nthreads;
                    if (c < hidden) xrow[c] = xrow[c] * inv * nw[k];
                }
                __syncthreads();
            }
            float* logits_row = a.logits ? a.logits + size_t(bid) * experts : nullptr;
#pragma unroll 1
            for (int e_lo = 0; e_lo < experts; e_lo += pass_rows) {
                if (a.route_rows > 0) {
                    if (e_lo > 0) {  // (part 0 was stored before the wait above; the registers hold part 1)
                        store_router_rows(e_lo);
                        if (e_lo + pass_rows < experts) request_router_rows(e_lo + pass_rows);
                    }
                    __syncthreads();
                }
                route_logits(a.router, a.route_rows > 0 ? wsm : nullptr, wstride, xrow, a.bias, hidden, e_lo,
                             min(experts, e_lo + pass_rows), slog, logits_row, tid, nthreads);
                __syncthreads();  // the staged rows are no longer read; slog is complete up to here
            }
            if (warp == 0)
                route_topk_gates(slog, experts, topk, EP ? s_rids : a.ids + size_t(bid) * topk,
                                 a.gates + size_t(bid) * topk, lane);
            if (!EP) {
                route_quantize_row(xrow, hidden, a.xq + size_t(bid) * hidden, a.xs + size_t(bid) * P0.nbp,
                                   a.xsum + size_t(bid) * P0.nbp, warp, lane, 1, nwarps - 1);
                __syncthreads();
                if (tid == 0) grid_arrive(a.sync + 0);
            } else {
                // The row is quantized into shared memory (where the router matrix was), then stored
                // into every rank's window, this rank's included, and announced there.
                int8_t* sq = reinterpret_cast<int8_t*>(wsm);
                float* ss = reinterpret_cast<float*>(wsm + hidden);
                float* ssum = ss + P0.nbp;
                route_quantize_row(xrow, hidden, sq, ss, ssum, warp, lane, 1, nwarps - 1);
                __syncthreads();
                const size_t g = size_t(own + bid);  // this token among all ranks' tokens
                const int vq = hidden / 16, vs = P0.nbp / 4, per_rank = vq + 2 * vs + topk;
#pragma unroll 1
                for (int i = tid; i < ranks * per_rank; i += nthreads) {
                    const int r = i / per_rank, j = i - r * per_rank;
                    uint8_t* w = a.ep.base[r];
                    if (j < vq)
                        reinterpret_cast<uint4*>(w + a.ep.off_xq + g * hidden)[j] = reinterpret_cast<const uint4*>(sq)[j];
                    else if (j < vq + vs)
                        reinterpret_cast<uint4*>(w + a.ep.off_xs + g * P0.nbp * 4)[j - vq] = reinterpret_cast<const uint4*>(ss)[j - vq];
                    else if (j < vq + 2 * vs)
                        reinterpret_cast<uint4*>(w + a.ep.off_xsum + g * P0.nbp * 4)[j - vq - vs] =
                            reinterpret_cast<const uint4*>(ssum)[j - vq - vs];
                    else
                        reinterpret_cast<uint32_t*>(w + a.ep.off_ids)[g * topk + (j - vq - 2 * vs)] = s_rids[j - vq - 2 * vs];
                }
                if (tid < topk) a.ids[size_t(bid) * topk + tid] = s_rids[tid];  // (the routing taps read these)
                __syncthreads();
                if (tid < ranks && !a.ep.mute)
                    arrive_on_peer(reinterpret_cast<uint32_t*>(a.ep.base[tid] + a.ep.off_flags) + DECODE_EP_FLAG_ROUTE);
            }
        }
        if (EP) {
            epoch0 = a.ep.epoch[0];
            routed0 = a.ep.epoch[1];
            if (tid == 0 && !peer_count_wait(flags + DECODE_EP_FLAG_ROUTE, routed0 + uint32_t(ranks * t), a.spin_limit))
                s_abort = 4;
        } else if (tid == 0 && !grid_wait(a.sync + 0, uint32_t(t), a.spin_limit)) {
            s_abort = 1;
        }
        __syncthreads();
        if (stamping) a.stamps[2] = wall_clock_ns();

        // ---- the batch's expert ids; for small batches the experts that were picked
        if (!s_abort) {
#pragma unroll 1
            for (int i = tid; i < slots; i += nthreads) s_ids[i] = __ldcg(ids_all + i);
            if (EP) {
                // Runs: each local expert's slots in pieces of up to D_TOK; (run, unit) pairs are what the
                // CTAs and warps share out, so an expert with many tokens spreads over many warps.
#pragma unroll 1
                for (int e = tid; e < a.ep.local; e += nthreads) s_cnt[e] = 0;
                __syncthreads();
#pragma unroll 1
                for (int i = tid; i < slots; i += nthreads) {
                    const uint32_t e = s_ids[i] - uint32_t(a.ep.first);
                    if (e < uint32_t(a.ep.local)) atomicAdd(&s_cnt[e], 1u);
                }
                __syncthreads();
                if (warp == 0) {
                    // Run length 32, 16 or 8: the one with the least work on the busiest warp. A run's
                    // units go to nctas / runs CTAs (share()); a warp takes its CTA's units in waves
                    // of nwarps, and a unit costs about 3 + (tiles of 8 tokens) in units of a tile.
                    int runs[3] = {0, 0, 0}, most = 0;
#pragma unroll 1
                    for (int e = lane; e < a.ep.local; e += 32) {
                        const int c = int(s_cnt[e]);
                        most = max(most, c);
#pragma unroll
                        for (int k = 0; k < 3; k++) runs[k] += (c + (D_TOK >> k) - 1) / (D_TOK >> k);
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) most = max(most, __shfl_xor_sync(0xffffffffu, most, o));
                    int run_len = D_TOK, best = 0x7fffffff;
#pragma unroll
                    for (int k = 0; k < 3; k++) {
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) runs[k] += __shfl_xor_sync(0xffffffffu, runs[k], o);
                        const int len = D_TOK >> k, r = max(1, runs[k]);
                        const int per_cta = r <= nctas ? (P0.upe + nctas / r - 1) / (nctas / r) : (r * P0.upe + nctas - 1) / nctas;
                        const int cost = (per_cta + nwarps - 1) / nwarps * (3 + (min(len, most) + 7) / 8);
                        if (cost < best) best = cost, run_len = len;
                    }
                    // A lane per local expert, 32 at a time: the expert's runs after those before it.
                    int n = 0;
#pragma unroll 1
                    for (int e0 = 0; e0 < a.ep.local; e0 += 32) {
                        const int e = e0 + lane;
                        const int mine = e < a.ep.local ? (int(s_cnt[e]) + run_len - 1) / run_len : 0;
                        int before = mine;
#pragma unroll
                        for (int o = 1; o < 32; o <<= 1) {
                            const int up = __shfl_up_sync(0xffffffffu, before, o);
                            if (lane >= o) before += up;
                        }
                        const int total = __shfl_sync(0xffffffffu, before, 31);
                        before -= mine;
                        for (int j = 0; j < mine && n + before + j < MAX_RUNS; j++) {
                            s_active[n + before + j] = uint16_t(a.ep.first + e);
                            s_skip[n + before + j] = uint16_t(j * run_len);
                        }
                        n += total;
                    }
                    if (lane == 0) {
                        s_nactive = min(n, MAX_RUNS);
                        s_run_len = run_len;
                    }
                }
            } else if (!a.dense) {
#pragma unroll 1
                for (int e = tid; e < experts; e += nthreads) s_picked[e] = 0;
                __syncthreads();
#pragma unroll 1
                for (int i = tid; i < slots; i += nthreads) s_picked[s_ids[i]] = 1;
                __syncthreads();
                if (warp == 0) {
                    int n = 0;
#pragma unroll 1
                    for (int e0 = 0; e0 < experts; e0 += 32) {
                        const int e = e0 + lane;
                        const bool on = e < experts && s_picked[e];
                        const unsigned ballot = __ballot_sync(0xffffffffu, on);
                        if (on) s_active[n + __popc(ballot & ((1u << lane) - 1u))] = uint16_t(e);
                        n += __popc(ballot);
                    }
                    if (lane == 0) s_nactive = n;
                }
            }
            __syncthreads();
        }
    }
    bool ok = !s_abort;

    const int g = lane >> 2, tq = lane & 3;
    float acc[D_GMAX][4], off[D_GMAX][4];
    uint32_t xphase = 0, xtok = 0;
    int arrived = 0;  // expert phases this CTA has announced
    int cslot = 0;    // consumer's ring slot and the parity of its barrier
    uint32_t cpar = 0;

#pragma unroll 1
    for (int p = 0; p < 2 && ok; p++) {
        const Phase& P = p ? P1 : P0;
        const bool gate_up = p == 0;
        int cu = 0;  // consumer cursor: unit ordinal within the warp's share
        const int xs_off = a.xcap * P.x_stride;
        const int xsum_off = xs_off + P.nbp * D_TOK * 4;
        float* xsT = reinterpret_cast<float*>(smem + L.x0 + xs_off);
        float* xsumT = reinterpret_cast<float*>(smem + L.x0 + xsum_off);
        const int seg_first = P.lo < P.hi ? P.lo / P.upe : 0;
        const int seg_last = P.lo < P.hi ? (P.hi - 1) / P.upe : -1;
#pragma unroll 1
        for (int sb = seg_first; sb <= seg_last && ok; sb += D_NSEG) {
            const int nseg = min(D_NSEG, seg_last - sb + 1);
            if (sb != seg_first) __syncthreads();  // the previous lists and staged rows are no longer read
            // ---- the slots that named each expert of this batch of segments, ascending
            if (EP && slots > 8 * 32) {
                // Many slots (every rank's): all warps scan, each a slice of the ids. First the hits per
                // slice and segment, then, from the counts of the slices before it, where each hit goes.
                const int slice = ((slots + nwarps - 1) / nwarps + 31) & ~31;
                const int lo = min(slots, warp * slice), hi = min(slots, lo + slice);
                const int run_len = s_run_len;
#pragma unroll 1
                for (int k = 0; k < nseg; k++) {
                    const uint32_t e = uint32_t(s_active[sb + k]);
                    int count = 0;
#pragma unroll 1
                    for (int base = lo; base < hi; base += 32)
                        count += __popc(__ballot_sync(0xffffffffu, base + lane < hi && s_ids[base + lane] == e));
                    if (lane == 0) s_part[k * D_MAX_WARPS + warp] = count;
                }
                __syncthreads();
#pragma unroll 1
                for (int k = 0; k < nseg; k++) {
                    const uint32_t e = uint32_t(s_active[sb + k]);
                    const int skip = int(s_skip[sb + k]);
                    const int part = lane < nwarps ? s_part[k * D_MAX_WARPS + lane] : 0;
                    int before = lane < warp ? part : 0, total = part;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        before += __shfl_xor_sync(0xffffffffu, before, o);
                        total += __shfl_xor_sync(0xffffffffu, total, o);
                    }
                    int count = before, token = (lo + lane) / topk, pick = (lo + lane) - token * topk;
#pragma unroll 1
                    for (int base = lo; base < hi; base += 32) {
                        const bool hit = base + lane < hi && s_ids[base + lane] == e;
                        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
                        if (hit) {
                            const int ord = count + __popc(ballot & ((1u << lane) - 1u)) - skip;
                            if (ord >= 0 && ord < run_len) {
                                s_slot[k * D_TOK + ord] = uint16_t(base + lane);
                                s_tok[k * D_TOK + ord] = uint16_t(token);
                            }
                        }
                        count += __popc(ballot);
                        pick += 32;
                        while (pick >= topk) pick -= topk, token++;
                    }
                    if (tid == 0) s_seg_count[k] = min(run_len, max(0, total - skip));
                }
            } else if (warp < nseg) {
                const int walk = sb + warp;
                const uint32_t e = uint32_t(a.dense ? walk : int(s_active[walk]));
                const int skip = EP ? int(s_skip[walk]) : 0;  // the expert's slots that earlier runs took
                const int run_len = EP ? s_run_len : D_TOK;
                int count = 0, token = 0, pick = lane;  // slot base + lane = token * topk + pick
                while (pick >= topk) pick -= topk, token++;
#pragma unroll 1
                for (int base = 0; base < slots; base += 32) {
                    const bool hit = base + lane < slots && s_ids[base + lane] == e;
                    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
                    if (hit) {
                        const int ord = count + __popc(ballot & ((1u << lane) - 1u)) - skip;
                        if (ord >= 0 && ord < run_len) {
                            s_slot[warp * D_TOK + ord] = uint16_t(base + lane);
                            s_tok[warp * D_TOK + ord] = uint16_t(token);
                        }
                    }
                    count += __popc(ballot);
                    pick += 32;
                    while (pick >= topk) pick -= topk, token++;
                }
                if (lane == 0) s_seg_count[warp] = min(run_len, max(0, count - skip));
            }
            if (sb == seg_first && p == 1) {
                // The lists depend on the ids only: they were made while the other CTAs finished
                // gate_up. Their SwiGLU rows are read from here on.
                if (tid == 0 && !grid_wait(a.sync + 1, uint32_t(nctas), a.spin_limit)) s_abort = 2;
            }
            __syncthreads();
            if (sb == seg_first && p == 1) {
                if (stamping) a.stamps[3] = wall_clock_ns();
                if (s_abort) {
                    ok = false;
                    break;
                }
            }
            int si = 0;
#pragma unroll 1
            while (si < nseg && ok) {
                // ---- a group: consecutive segments whose rows (in tiles of 8) fit the staged area
                int row0[D_NSEG] = {0, 0, 0, 0}, sj = si, rows = 0;
#pragma unroll
                for (int k = 0; k < D_NSEG; k++) {  // (constant indices keep row0 in registers)
                    if (k == sj && k < nseg) {
                        const int need = (s_seg_count[k] + 7) & ~7;
                        if (k == si || rows + need <= a.xcap) {
                            row0[k] = rows;
                            rows += need;
                            sj = k + 1;
                        }
                    }
                }
                auto row_of = [&](int sx) { return sx == 0 ? row0[0] : sx == 1 ? row0[1] : sx == 2 ? row0[2] : row0[3]; };
                if (si > 0) __syncthreads();  // the previous group's rows are no longer read
                // Staged row r belongs to the last segment that starts at or before it; rows past a
                // segment's tokens (up to a whole tile of 8) repeat its last one.
                auto entry_of_row = [&](int r) {
                    int sx = si;
#pragma unroll
                    for (int k = 1; k < D_NSEG; k++)
                        if (k > si && k < sj && r >= row0[k]) sx = k;
                    return sx * D_TOK + min(r - row_of(sx), s_seg_count[sx] - 1);
                };
                if (gate_up) {
                    // Token rows by plain 16-byte loads (L2 hits: the router phase just wrote them), a
                    // warp per row; then the scales transposed to [block][token], a warp per block
                    // and a lane per row, so that the stores do not conflict.
                    const int vec_per_row = P.cols / 16;
#pragma unroll 1
                    for (int r = warp; r < rows; r += nwarps) {
                        const uint4* src = reinterpret_cast<const uint4*>(xq_all + size_t(s_tok[entry_of_row(r)]) * P.cols);
                        uint8_t* dst = smem + L.x0 + r * P.x_stride;
#pragma unroll 2
                        for (int v = lane; v < vec_per_row; v += 32) *reinterpret_cast<uint4*>(dst + v * 16) = __ldcg(src + v);
                    }
                    if (lane < rows) {
                        const size_t src = size_t(s_tok[entry_of_row(lane)]) * P.nbp;
#pragma unroll 2
                        for (int b = warp; b < P.nb; b += nwarps) {
                            xsT[b * D_TOK + lane] = __ldcg(xs_all + src + b);
                            if (KIND == 2) xsumT[b * D_TOK + lane] = __ldcg(xsum_all + src + b);
                        }
                    }
                } else {
                    // The down projection's inputs are the SwiGLU rows in f32: quantized here exactly as
                    // quantize_q8 does (src/kernels.rs:84-98, applied per gathered row by
                    // src/weights.rs:652-664), straight into the staged layout. A thread per
                    // (row, 32-block).
#pragma unroll 1
                    for (int task = tid; task < rows * P.nb; task += nthreads) {
                        const int r = task / P.nb, b = task - r * P.nb;
                        const size_t row = s_slot[entry_of_row(r)];
                        const float4* src = reinterpret_cast<const float4*>(a.hidden_f + row * P.cols + b * QK);
                        float4 v[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) v[i] = __ldcg(src + i);
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
                        uint4* dst = reinterpret_cast<uint4*>(smem + L.x0 + r * P.x_stride + b * QK);
                        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        xsT[b * D_TOK + r] = d;
                        if (KIND == 2) xsumT[b * D_TOK + r] = d * float(qsum);
                    }
                }
                __syncthreads();
                // A value the compiler cannot know before the barrier: the staged reads depend on it.
                asm volatile("mov.u32 %0, %1;" : "=r"(xtok) : "r"(xphase) : "memory");

                // ---- this warp's units of the group's segments, a unit (all its chunks) at a time
#pragma unroll 1
                while (ok && cu < P.n) {
                    const int wu = P.first + cu * nwarps;
                    const int seg = wu / P.upe;
                    const int sx = seg - sb;  // segment of the unit within this batch
                    if (sx >= sj) break;
                    const int u = wu - seg * P.upe;
                    const int cnt = s_seg_count[sx], G = (cnt + 7) >> 3, r0x = row_of(sx);
                    const uint32_t xq_s = smem_addr(smem + L.x0 + r0x * P.x_stride);
                    const uint32_t xsT_s = smem_addr(xsT + r0x), xsumT_s = smem_addr(xsumT + r0x);
#pragma unroll
                    for (int nt = 0; nt < D_GMAX; nt++) {
                        acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
                        off[nt][0] = off[nt][1] = off[nt][2] = off[nt][3] = 0.0f;
                    }
#pragma unroll 1
                    for (int cc = 0; cc < P.nchunks; cc++) {
                        // The unit's next record: the ring is topped up, then the record waited for.
                        top_up();
                        const bool landed = mbar_wait_poll(bars + cslot, cpar);
                        if (!__all_sync(0xffffffffu, landed)) {
                            ok = false;
                            break;
                        }
                        const uint32_t rec = smem_addr(ring + cslot * R::BYTES), wtok = uint32_t(landed);
                        const int nblk = min(F_NBC, P.nb - cc * F_NBC), blk0 = cc * F_NBC;
                        switch (G) {
                            case 0: break;  // an expert nobody picked (dense walk): its records are only drained
                            case 1: fast_chunk<KIND, 1, D_GMAX>(rec, xq_s, xsT_s, xsumT_s, P.x_stride, nblk, blk0, lane, wtok, xtok, acc, off); break;
                            case 2: fast_chunk<KIND, 2, D_GMAX>(rec, xq_s, xsT_s, xsumT_s, P.x_stride, nblk, blk0, lane, wtok, xtok, acc, off); break;
                            case 3: fast_chunk<KIND, 3, D_GMAX>(rec, xq_s, xsT_s, xsumT_s, P.x_stride, nblk, blk0, lane, wtok, xtok, acc, off); break;
                            default: fast_chunk<KIND, 4, D_GMAX>(rec, xq_s, xsT_s, xsumT_s, P.x_stride, nblk, blk0, lane, wtok, xtok, acc, off); break;
                        }
                        __syncwarp();
                        if (++cslot == STAGES) cslot = 0, cpar ^= 1;
                        takes++;
                    }
                    if (!ok) break;
#pragma unroll
                    for (int nt = 0; nt < D_GMAX; nt++) {
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            const int j = nt * 8 + 2 * tq + i;
                            if (j < cnt) {
                                float y0 = acc[nt][i], y1 = acc[nt][2 + i];  // rows g and g+8
                                if (KIND == 2) {
                                    y0 = y0 + off[nt][i];
                                    y1 = y1 + off[nt][2 + i];
                                }
                                const size_t slot = s_slot[sx * D_TOK + j];
                                if (gate_up) {
                                    const int col = u * 8 + g;
                                    if (col < inter) {
                                        const float ex = exp_poly(-y0);
                                        a.hidden_f[slot * inter + col] = __fdiv_rn(y0, 1.0f + ex) * y1;
                                    }
                                } else {
                                    const int r0 = u * F_ROWS + g;
                                    float* dst = a.out + slot * hidden;
                                    if (EP) {  // the row's place in its home rank's window, over NVLink
                                        const size_t per_rank = size_t(t) * topk, home = slot / per_rank;
                                        dst = reinterpret_cast<float*>(a.ep.base[home] + a.ep.off_out) + (slot - home * per_rank) * hidden;
                                    }
                                    if (r0 < hidden) dst[r0] = y0;
                                    if (r0 + 8 < hidden) dst[r0 + 8] = y1;
                                }
                            }
                        }
                    }
                    cu++;
                }
                ok = __syncthreads_and(ok);  // keep the decision to stop uniform across the CTA's barriers
                xphase++;
                si = sj;
            }
        }
        if (!ok) break;
        // The ring is topped up with the next phase's records before this CTA waits for the others.
        top_up();
        // ---- every CTA's part of this phase is in global memory before anyone reads it
        __syncthreads();
        arrived = p + 1;
        if (EP && p == 1) {
            if (tid < ranks)
                arrive_on_peer(reinterpret_cast<uint32_t*>(a.ep.base[tid] + a.ep.off_flags) + DECODE_EP_FLAG_DOWN);
        } else if (tid == 0) {
            grid_arrive(a.sync + 1 + p);
        }
    }
    if (!ok && tid == 0 && !s_abort) s_abort = 3;

    // ---- weighted combine + residual add: CTA i < t takes token i (src/model.rs:513-519, 681),
    // once every CTA's part of the down phase is in global memory.
    if (ok && bid < t) {
        if (tid == 0) {
            const bool came = EP ? peer_count_wait(flags + DECODE_EP_FLAG_DOWN, (epoch0 + 1u) * uint32_t(ranks * nctas),
                                                   a.spin_limit)
                                 : grid_wait(a.sync + 2, uint32_t(nctas), a.spin_limit);
            if (!came) s_abort = EP ? 4 : 2;
        }
        __syncthreads();
        ok = !s_abort;
        if (stamping) a.stamps[4] = wall_clock_ns();
    }
    if (ok && bid < t) {
        if (tid < topk) {
            const uint32_t* my_ids = s_ids + (own + bid) * topk;
            const uint32_t mine = my_ids[tid];
            int rank = 0;
            for (int j = 0; j < topk; j++) rank += my_ids[j] < mine ? 1 : 0;
            s_cpos[rank] = uint32_t(bid * topk + tid);
            s_cgate[rank] = __ldcg(a.gates + size_t(bid) * topk + tid);
        }
        __syncthreads();
        float* yr = a.y + size_t(bid) * hidden;
#pragma unroll 1
        for (int c = tid * 4; c < hidden; c += nthreads * 4) {
            float4 proj = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
            for (int j = 0; j < topk; j++) {
                const float gt = s_cgate[j];
                const float4 v = __ldcg(reinterpret_cast<const float4*>(out_own + size_t(s_cpos[j]) * hidden + c));
                proj.x = proj.x + gt * v.x;
                proj.y = proj.y + gt * v.y;
                proj.z = proj.z + gt * v.z;
                proj.w = proj.w + gt * v.w;
            }
            float4 r = *reinterpret_cast<float4*>(yr + c);
            r.x = r.x + proj.x;
            r.y = r.y + proj.y;
            r.z = r.z + proj.z;
            r.w = r.w + proj.w;
            *reinterpret_cast<float4*>(yr + c) = r;
        }
        // The last combining CTA leaves the counters at zero for the next launch. Every CTA
        // has passed its waits on them by now (all arrived at the last one).
        if (tid == 0 && atomicAdd(a.sync + 3, 1u) == uint32_t(t) - 1) {
            a.sync[0] = a.sync[1] = a.sync[2] = a.sync[3] = 0;
            if (EP) a.ep.epoch[0] = epoch0 + 1u, a.ep.epoch[1] = routed0 + uint32_t(ranks * t);
            __threadfence();
        }
    }
    if (stamping) a.stamps[5] = wall_clock_ns();
    if (!ok) {
        if (tid == 0) {
            atomicExch(a.status, s_abort == 3 ? ERR_COPY_WAIT_TIMEOUT : s_abort == 4 ? ERR_PEER_WAIT_TIMEOUT : ERR_GRID_WAIT_TIMEOUT);
            // Announce the phases this CTA will not run, so that nobody waits for it in vain.
            for (int p = arrived; p < 2; p++) atomicAdd(a.sync + 1 + p, 1u);
        }
        // Give copies already in flight a bounded chance to land before the shared memory
        // they target is released.
        for (uint32_t k = takes; k < fills; k++) {
            mbar_wait_poll(bars + cslot, cpar);
            if (++cslot == STAGES) cslot = 0, cpar ^= 1;
        }
    }
}

// Rows of the router matrix the router phase stages at a time: the whole matrix, or the
// fewest equal parts, within what the token area offers anyway (a dense walk, where the
// ring's depth matters) or within 72 KB (a sparse walk, where the ring is mostly idle).
template <int KIND>
int decode_route_rows(const MoeDims& d, int t, int xcap, int nthreads) {
    const int held = D_ROUTE_VEC * nthreads / (d.hidden / 8);  // rows the CTA's registers hold at a time
    const int tokens = DLayout<KIND>::token_bytes(xcap, d.hidden, d.inter);
    const int base = DLayout<KIND>::route_base(d.hidden, d.experts) + 64, wstride = 2 * d.hidden + 32;
    const int budget = dense_walk(d, t) ? tokens + 2048 : max(tokens, 72 * 1024);
    for (int parts = 1; parts <= 8; parts++) {
        const int rows = (d.experts + parts - 1) / parts;
        if (rows <= held && base + rows * wstride <= budget) return rows;
    }
    return max(0, min(held, (tokens - base) / wstride));
}

// Warps per CTA, ring depth and staged rows: as many warps as possible while each still
// gets a ring of at least two stages; then the deepest ring that fits.
template <int KIND>
bool decode_config(const MoeDims& d, int t, int ids_slots, int& nwarps, int& stages, int& xcap, int& route_rows) {
    // Rows staged at a time: an expert's tokens, up to D_TOK of them, out of all the tokens the expert
    // phases see (every rank's when expert-parallel: ids_slots / topk).
    xcap = min(D_TOK, (ids_slots / d.topk + 7) / 8 * 8);
    auto deepest = [&](int w, int rr) {
        for (int k = D_MAX_STAGES; k >= 2; k--)
            if (size_t(DLayout<KIND>(w, k, xcap, rr, d.hidden, d.inter, d.experts, d.topk, ids_slots).total) <= D_SMEM_LIMIT)
                return k;
        return 0;
    };
    int best_w = 0, best_s = 0, best_r = 0;
    for (int w = D_MAX_WARPS; w >= 8; w -= 2) {
        const int rr = decode_route_rows<KIND>(d, t, xcap, w * 32);
        const int s = deepest(w, rr);
        // (More warps matter more than a third stage: an expert's units are cut into parts of 16
        // where they can be, one per warp. Measured at granite-1b-a400m, batch 32: 0.83 ms per
        // step with 16 warps and two stages against 0.865 with 14 and three.)
        if (s >= 2) {
            nwarps = w, stages = s, route_rows = rr;
            return true;
        }
        if (s > best_s) best_s = s, best_w = w, best_r = rr;
    }
    nwarps = best_w, stages = best_s, route_rows = best_r;
    return best_s >= 2;
}

}  // namespace

void init_kernels_decode() {
    const int lim = int(D_SMEM_LIMIT);
    cudaFuncSetAttribute(moe_decode_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(moe_decode_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(moe_decode_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    cudaFuncSetAttribute(moe_decode_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
}

// `ranks` > 1 (or an expert-parallel layer of one rank): t is the tokens per rank. A token's router
// phase and combine take a CTA each; the expert-parallel form walks an expert's tokens in runs, so
// with one rank (nothing crosses a link) it takes up to 128 tokens.
bool decode_block_applies(const MoeDims& d, int kind_gate_up, int kind_down, int t, int ranks) {
    const int most = ranks == 1 ? 4 * D_TOK : D_TOK;
    if (t < 1 || t > most || kind_gate_up != kind_down || d.topk > MAX_TOPK || d.hidden > D_NORM_HELD * 256)
        return false;
    const int slots = (ranks > 0 ? ranks : 1) * t * d.topk;
    if (slots > 65535 / 16 || d.experts > MAX_EXPERTS) return false;  // (slot lists are 16-bit; ids live in shared memory)
    int w, s, x, r;
    return kind_gate_up == 1 ? decode_config<1>(d, t, slots, w, s, x, r) : decode_config<2>(d, t, slots, w, s, x, r);
}

int launch_decode_block(const MoeDims& d, int kind, const uint16_t* router, const float* bias, const float* x,
                        const float* norm_w, float eps, int t, float* y, const uint8_t* gate_up_tiled,
                        const uint8_t* down_tiled, Workspace& ws, int sms, uint32_t spin_limit,
                        unsigned long long* stamps, cudaStream_t stream, const DecodeEp* ep, float* hidden_f_all) {
    DecodeArgs a{};
    a.stamps = stamps;
    a.router = router, a.bias = bias, a.x = x, a.norm_w = norm_w, a.eps = eps, a.y = y;
    a.t = t, a.hidden = d.hidden, a.experts = d.experts, a.topk = d.topk, a.inter = d.inter;
    a.logits = ws.logits, a.ids = ws.ids, a.gates = ws.gates, a.xq = ws.xq, a.xs = ws.xs, a.xsum = ws.xsum;
    a.gu_tiled = gate_up_tiled, a.dn_tiled = down_tiled;
    a.hidden_f = ep ? hidden_f_all : ws.hidden_f, a.out = ws.out;
    a.dense = !ep && dense_walk(d, t) ? 1 : 0;
    // (For a sparse walk on one GPU, batches of 3 to 15 tokens, the same request made the step
    // slower, 1.06 ms against 0.86 at 8 tokens: 53 MB of requests are still in the way of the
    // picked experts' records when the router phase ends.)
    a.l2_all = ep && (long long)ep->ranks * t * d.topk >= 4LL * d.experts;
    if (ep) a.ep = *ep;
    a.ids_slots = (ep ? ep->ranks : 1) * t * d.topk;
    a.sync = ws.grid_sync;
    a.spin_limit = spin_limit;
    a.status = ws.status;
    int nwarps = 0;
    const bool fits = kind == 1 ? decode_config<1>(d, t, a.ids_slots, nwarps, a.stages, a.xcap, a.route_rows)
                                : decode_config<2>(d, t, a.ids_slots, nwarps, a.stages, a.xcap, a.route_rows);
    if (!fits) return -1;
    // One CTA per SM, all resident at once (they wait for one another): never more CTAs than SMs.
    const int grid = sms;
    const size_t smem = kind == 1 ? size_t(DLayout<1>(nwarps, a.stages, a.xcap, a.route_rows, d.hidden, d.inter, d.experts,
                                                      d.topk, a.ids_slots).total)
                                  : size_t(DLayout<2>(nwarps, a.stages, a.xcap, a.route_rows, d.hidden, d.inter, d.experts,
                                                      d.topk, a.ids_slots).total);
    auto kernel = kind == 1 ? (ep ? moe_decode_kernel<1, true> : moe_decode_kernel<1, false>)
                            : (ep ? moe_decode_kernel<2, true> : moe_decode_kernel<2, false>);
    launch_overlapped(kernel, dim3(grid), dim3(nwarps * 32), smem, stream, a);
    return 1;
}

}  // namespace tc
