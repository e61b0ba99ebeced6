// Internal declarations shared by the kernel files and the C ABI.
//
// Compile every file with -fmad=false: the CPU path this backend reproduces
// rounds a*b before adding c unless its source asks for a fused multiply-add
// (src/kernels_x86.rs uses _mm256_fmadd_ps, src/kernels.rs:427 mul_add), so
// the kernels spell fmaf() where the reference fuses and plain * and +
// everywhere else.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace tc {

constexpr int QK = 32;          // values per quantization block (src/kernels.rs:13)
constexpr int SUPER = 8;        // 4-bit blocks per packed super-block (src/kernels.rs:165)
constexpr int SUPER_WORDS = 5;  // words per super-block (src/kernels.rs:167)

constexpr int MAX_EXPERTS = 256;
constexpr int GRID_SYNC_WORDS = 8;
constexpr int MAX_TOPK = 32;

// Error codes a kernel may leave in the context's status word.
enum : int {
    ERR_NONE = 0,
    ERR_COPY_WAIT_TIMEOUT = 1,  // a staged weight copy did not arrive within the spin limit
    ERR_PEER_WAIT_TIMEOUT = 2,  // another rank's signal did not arrive within the spin limit
    ERR_BAD_EXPERT_ID = 3,      // the dispatch met an expert id out of range, or twice in one token
    ERR_GRID_WAIT_TIMEOUT = 4,  // a CTA gave up waiting for the other CTAs of its own grid
};

struct MatrixDev {
    int kind;
    size_t rows, cols;
    const void* scales;  // Q8: f16 [rows, cols/32]; Q4: u32 [rows, words]
    const void* data;    // BF16: u16; Q8: i8; Q4: u8 packed nibbles
};

// Per-context scratch, sized at layer creation for max_tokens.
// Waiting for other ranks' signals (expert parallelism over peer memory): flags[r] is
// written by rank r with its block counter; *epoch is this rank's own counter.
struct PeerWait {
    const uint32_t* flags = nullptr;  // [ranks], in this rank's memory
    const uint32_t* epoch = nullptr;
    int ranks = 0;
    int* status = nullptr;
    uint32_t limit = 1u << 23;        // polls before the wait gives up (about ten seconds by default)
};

// Sending this rank's rows to every rank's window, then announcing it (or, with t = 0,
// the announcement alone).
struct PeerPlan {
    uint8_t* base[8] = {};  // every rank's window as mapped here
    size_t off_xq = 0, off_xs = 0, off_ids = 0, off_flags = 0;
    const int8_t* xq = nullptr;
    const float* xs = nullptr;
    const uint32_t* ids = nullptr;
    int t = 0, hidden = 0, nbp = 0, topk = 0, me = 0, ranks = 0, flag_set = 0;
    uint32_t* epoch = nullptr;  // this rank's counters, one per flag set
    int mute = 0;               // testing: send the rows but not the announcement (a rank that never signals)
};

// The sorted slots cut into runs of at most 16 slots of one expert, for callers
// whose experts see several 16-token segments each (expert parallelism): the
// expert kernels then spread (run, unit) pairs evenly over CTAs and warps instead
// of giving all segments of an expert's unit to one warp.
struct RunList {
    int* expert = nullptr;        // [runs] expert of the run (index into the matrices held)
    uint32_t* count = nullptr;    // [runs] 1..16
    uint32_t* offset = nullptr;   // [runs] first sorted slot
    int* n = nullptr;             // number of runs
};

struct Workspace {
    int max_tokens = 0, hidden = 0, experts = 0, topk = 0, inter = 0;
    int sms = 0;                  // multiprocessors of the context's device
    float* logits = nullptr;      // [T, E]
    uint32_t* ids = nullptr;      // [T, k] descending score order
    float* gates = nullptr;       // [T, k]
    int8_t* xq = nullptr;         // [T, H] activations, 8-bit per 32-block
    float* xs = nullptr;          // [T, pad8(H/32)] their scales, zero padded
    float* xsum = nullptr;        // [T, pad8(H/32)] scale * sum of quants (4-bit offsets)
    uint32_t* counts = nullptr;   // [E] tokens per expert
    uint32_t* offsets = nullptr;  // [E+1] first sorted slot of each expert
    uint32_t* perm = nullptr;     // [T*k] sorted slot -> token*k + j
    uint32_t* pos = nullptr;      // [T*k] token*k + j -> sorted slot
    uint32_t* slot_token = nullptr;  // [T*k] sorted slot -> token
    int* active = nullptr;        // [E+1] experts with tokens, ascending; [E] = how many
    uint32_t* block_hist = nullptr;  // [blocks, E] dispatch: per-block histograms / bases
    float* hidden_f = nullptr;    // [T*k, I] silu(gate)*up, sorted order
    int8_t* hq = nullptr;         // [T*k, I]
    float* hs = nullptr;          // [T*k, pad8(I/32)]
    float* hsum = nullptr;        // [T*k, pad8(I/32)]
    float* out = nullptr;         // [T*k, H] expert outputs, sorted order
    int* status = nullptr;        // device status word
    int* ticket = nullptr;        // arrival counter of the router CTAs (zero between launches)
    uint32_t* grid_sync = nullptr;  // [GRID_SYNC_WORDS] arrival counters of the one-kernel decode block (zero between launches)
    RunList runs;                 // when set: the expert kernels walk these instead of counts/offsets/active
    PeerWait combine_wait;        // set for the peer-memory exchange only
    PeerWait dispatch_wait;       // the same, before the dispatch over every rank's tokens
    PeerPlan route_scatter;       // the same: rows sent by the router kernel's last CTA (ranks > 0)
};

struct MoeDims {
    int hidden, experts, topk, inter;
};

// Opt the kernels that need it into large dynamic shared memory (once per device).
void init_kernels_exact();
void init_kernels_fast();
void init_kernels_route();

// How the expert products add up a row's 32-element blocks.
enum : int {
    // One fma chain per output, blocks in order: acc = fma(float(block sum),
    // ws*xs, acc). The same on every fast path, so a token's result does not
    // depend on what it is batched with.
    ARITH_FAST = 0,
    // The CPU path's own order: eight float lanes per output, each block's sum
    // split across them four products at a time, then the AVX2 hsum tree.
    // Bit-identical to src/kernels_x86.rs; about five times the instructions.
    ARITH_CPU_LANES = 1,
};

// ---- launchers (each enqueues on `stream` and returns the number of kernels launched)

// Router logits (bf16 weights, f32 activations), top-k, gating softmax, and
// 8-bit quantization of each token's row.
// x is the block's normed input, or (norm_w set) the residual stream to be
// RMS-normed first. Batches of up to 256 tokens are dispatched by the same
// kernel; larger ones by launch_dispatch, which this then calls.
int launch_route(const MoeDims& d, const uint16_t* router, const float* bias, const float* x,
                 const float* norm_w, float eps, int t, Workspace& ws, cudaStream_t stream);

// Per-expert histogram, prefix scan and stable permutation of the t*k slots.
int launch_dispatch(const MoeDims& d, int t, Workspace& ws, cudaStream_t stream);

// The three-pass dispatch with its scratch in an array built into the library
// (no allocation). Returns null, or why the call was refused. *status_word receives the
// device address of the status word the kernels report bad expert ids in.
const char* dispatch_static(int device, const uint32_t* ids, int t, int experts, int topk,
                            uint32_t* counts, uint32_t* offsets, uint32_t* perm, uint32_t* pos,
                            uint32_t* slot_token, int* active, cudaStream_t stream, int** status_word);

// gate_up rows of each expert times its tokens, SwiGLU, into ws.hidden_f.
int launch_gate_up_exact(const MoeDims& d, const MatrixDev& gate_up, int t, Workspace& ws, int sms,
                         cudaStream_t stream);
int launch_gate_up_fast(const MoeDims& d, const MatrixDev& gate_up, const uint8_t* tiled, int t,
                        Workspace& ws, int sms, cudaStream_t stream);

// The fast kernels read weights re-tiled into per-(unit, 256-column chunk)
// records; these size, check and build that copy when a layer is created.
size_t tiled_bytes(const MoeDims& d, const MatrixDev& m, bool gate_up);
bool fast_path_fits(const MoeDims& d, const MatrixDev& gate_up, const MatrixDev& down);
void tile_weights(const MoeDims& d, const MatrixDev& m, bool gate_up, uint8_t* tiled, cudaStream_t stream);

// 8-bit quantization of ws.hidden_f rows into ws.hq / ws.hs / ws.hsum.
int launch_quant_hidden(const MoeDims& d, int t, Workspace& ws, cudaStream_t stream);

// down rows of each expert times its tokens' hidden rows, into ws.out.
int launch_down_exact(const MoeDims& d, const MatrixDev& down, int t, Workspace& ws, int sms,
                      cudaStream_t stream);
int launch_down_fast(const MoeDims& d, const MatrixDev& down, const uint8_t* tiled, int t,
                     Workspace& ws, int sms, cudaStream_t stream);

// y[i] += sum over the token's experts, ascending expert index, gate * out.
// (peer_out: when given, `ranks` buffers; output row p goes to rank p / peer_rows.)
int launch_down_fast_rows(const MoeDims& d, const MatrixDev& down, const uint8_t* tiled, Workspace& ws,
                          const uint32_t* out_rows, int sms, cudaStream_t stream,
                          float* const* peer_out = nullptr, int ranks = 0, uint32_t peer_rows = 0,
                          uint32_t* const* peer_flag = nullptr, uint32_t* peer_epoch = nullptr,
                          uint32_t* peer_ticket = nullptr);

// Fills `runs` from counts/offsets of `experts` experts (one CTA).
int launch_build_runs(const uint32_t* counts, const uint32_t* offsets, int experts, const RunList& runs,
                      cudaStream_t stream);

// ---- overlapping consecutive kernels of a block (programmatic dependent launch)
//
// The four kernels of a block are launched with the programmatic-stream-
// serialization attribute: each may start while the one in front of it still
// runs, does the part of its prologue that reads nothing an earlier kernel
// writes (barrier setup, weight prefetch), and then waits for the earlier grid
// to complete. Every such kernel executes grid_dependency_wait() on every path,
// before its first read or write of shared state, so completion stays
// transitive along the chain. Off: plain stream order.
extern bool g_launch_overlap;

#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_launch_overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

#ifdef __CUDACC__
// Bounded wait for rank r's signal: pw.limit polls (by default about ten seconds: ranks
// of one job can be seconds apart when they enqueue their first block), then an error
// status; the caller goes on, so the context stays usable.
__device__ __forceinline__ void peer_wait(const PeerWait& pw, int r) {
    const uint32_t want = *pw.epoch;
    for (uint32_t i = 0; i < pw.limit; i++) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(pw.flags + r) : "memory");
        if (int32_t(seen - want) >= 0) return;
        __nanosleep(i < 64 ? 32 : 512);
    }
    atomicExch(pw.status, ERR_PEER_WAIT_TIMEOUT);
}

// One CTA: copies this rank's rows into every window and release-stores the next value
// of this rank's counter into every rank's flag word. Writes of all the CTA's threads
// are ordered before the flags: CTA barrier, then a cumulative system-scope release.
__device__ __forceinline__ void peer_scatter_signal(const PeerPlan& a, uint32_t* s_epoch) {
    const int tid = threadIdx.x, n = blockDim.x;
    const size_t xq_vec = size_t(a.t) * a.hidden / 16, xs_vec = size_t(a.t) * a.nbp / 4;
    const size_t ids_n = size_t(a.t) * a.topk;
    for (int r = 0; r < a.ranks; r++) {
        uint8_t* w = a.base[r];
        uint4* dq = reinterpret_cast<uint4*>(w + a.off_xq + size_t(a.me) * a.t * a.hidden);
        const uint4* sq = reinterpret_cast<const uint4*>(a.xq);
        for (size_t i = tid; i < xq_vec; i += n) dq[i] = sq[i];
        uint4* ds = reinterpret_cast<uint4*>(w + a.off_xs + size_t(a.me) * a.t * a.nbp * 4);
        const uint4* ss = reinterpret_cast<const uint4*>(a.xs);
        for (size_t i = tid; i < xs_vec; i += n) ds[i] = ss[i];
        uint32_t* di = reinterpret_cast<uint32_t*>(w + a.off_ids) + size_t(a.me) * ids_n;
        for (size_t i = tid; i < ids_n; i += n) di[i] = a.ids[i];
    }
    __syncthreads();
    if (tid == 0) {
        *s_epoch = a.epoch[a.flag_set] + 1;
        a.epoch[a.flag_set] = *s_epoch;
    }
    __syncthreads();
    if (tid < a.ranks && !a.mute) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(a.base[tid] + a.off_flags) + a.flag_set * 8 + a.me;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(*s_epoch) : "memory");
    }
}
#endif

// Batches that reach (nearly) every expert walk all experts with a partition that
// does not depend on the routing; smaller ones walk the list of experts that have
// tokens. At 4 picks per expert on average an expert is left out with p < 2 %.
inline bool dense_walk(const MoeDims& d, int t) { return (long long)t * d.topk >= 4LL * d.experts; }

// ---- prefill-size groups on tcgen05 (experts_prefill.cu)
struct PrefillWeights {  // per layer: int8 tiles + f32 block scales (and 4-bit offsets)
    int8_t *gu_t = nullptr, *dn_t = nullptr;
    float *gu_d = nullptr, *gu_c = nullptr, *dn_d = nullptr, *dn_c = nullptr;
};
struct PrefillScratch {  // per context
    int *tile_expert = nullptr, *tile_n = nullptr, *tile_count = nullptr;
    uint32_t* tile_p0 = nullptr;
    int8_t* xt = nullptr;
    float *xst = nullptr, *xsumt = nullptr;
    size_t xt_bytes = 0, xst_elems = 0;
    size_t tile_bytes = 0;  // bytes of one token tile's 8-bit rows at the widest layer so far
    int max_tiles = 0;
};
void init_kernels_prefill();
bool prefill_fits(const MoeDims& d, bool q4_gate_up, bool q4_down);
size_t prefill_weight_bytes(const MoeDims& d, bool gate_up);
size_t prefill_scale_elems(const MoeDims& d, bool gate_up);
int prefill_max_token_tiles(int slots, int experts);
int prefill_token_tile();  // tokens per tile
void tile_prefill_weights(const MoeDims& d, const MatrixDev& m, bool gate_up, int8_t* wt, float* wd, float* wc,
                          cudaStream_t stream);
// peer_out (down only): null, or every rank's window for expert outputs; a row whose number in
// out_rows' numbering is p then goes to rank p / peer_rows, row p % peer_rows.
int launch_prefill(const MoeDims& d, bool gate_up, bool q4, const PrefillWeights& w, const PrefillScratch& s,
                   const Workspace& ws, int slots, float* out, const uint32_t* out_rows, cudaStream_t stream,
                   float* const* peer_out = nullptr, int peer_ranks = 0, uint32_t peer_rows = 0);

// One 128 x n x 32 int8 tcgen05 MMA (n = 64 or 128) through TMEM: a self-check of the encodings.
int launch_umma_selftest(const int8_t* a_tile, const int8_t* b_tile, int n, int* d_out, int* status,
                      cudaStream_t stream);

int launch_combine(const MoeDims& d, int t, Workspace& ws, float* y, cudaStream_t stream);

// The dense int8 tensor-core rate: `batches` batches of MMAs on each of `sms` SMs; returns the
// integer operations performed (int8_peak.cu).
double launch_int8_peak(int sms, int batches, int* status, cudaStream_t stream);

// Tachyon's weight quantizers on the device (quantize.cu): x[rows, cols] f32 into the buffers of a
// Matrix of `kind`; `scratch` holds rows * (1 + 2 * cols / 32) floats for the 4-bit fit.
int launch_quantize(int kind, const float* x, size_t rows, size_t cols, void* scales, void* data, float* scratch,
                    cudaStream_t stream);

// ---- the whole block of a decode-size batch as one kernel (moe_decode.cu)
// Expert parallelism inside the one-kernel block (ranks > 0). Every rank runs this kernel on
// its own GPU with its own t tokens and its own contiguous range of experts; the ranks'
// windows are mapped into one another (CUDA IPC). The router phase stores each token's 8-bit
// row, scales and expert ids into EVERY rank's window and announces it there with a
// system-scope reduction on a counter word; the expert phases then run over all ranks' tokens
// for this rank's experts; the down phase stores each output row into its home rank's window
// and announces itself the same way; the combine waits for every rank's CTAs. The counters
// only grow (a block is complete when they reach (blocks so far + 1) x arrivals per block), so
// nothing is reset across GPUs. Every wait is bounded.
struct DecodeEp {
    int ranks = 0, me = 0, first = 0, local = 0;  // this rank; its first expert and how many it holds
    uint8_t* base[8] = {};                // every rank's window as mapped here
    size_t off_xq = 0, off_xs = 0, off_xsum = 0, off_ids = 0, off_out = 0, off_flags = 0;
    uint32_t* epoch = nullptr;                    // two words: blocks this rank has completed on this path, and their router-phase arrivals
    int mute = 0;                                 // testing: rows are sent but not announced
};
void init_kernels_decode();
// True if a block of t tokens (per rank, when expert-parallel over `ranks` ranks) of this shape can
// take the one-kernel path.
bool decode_block_applies(const MoeDims& d, int kind_gate_up, int kind_down, int t, int ranks = 0);
// y[t, hidden] += moe(x) (or moe(rmsnorm(x)) when norm_w is set). Leaves the routing in
// ws.ids / ws.gates / ws.logits (and, on one GPU, the 8-bit rows in ws.xq / ws.xs); builds no dispatch.
// stamps: null, or 8 words that CTA 0 fills with the wall clock at its phase boundaries.
// ep: null, or the expert-parallel set-up (gate_up_tiled / down_tiled then hold this rank's experts
// and hidden_f_all is scratch for every rank's slots: ranks * t * topk rows of `inter` floats).
int launch_decode_block(const MoeDims& d, int kind, const uint16_t* router, const float* bias, const float* x,
                        const float* norm_w, float eps, int t, float* y, const uint8_t* gate_up_tiled,
                        const uint8_t* down_tiled, Workspace& ws, int sms, uint32_t spin_limit,
                        unsigned long long* stamps, cudaStream_t stream, const DecodeEp* ep = nullptr,
                        float* hidden_f_all = nullptr);

int launch_rmsnorm(const float* x, const float* w, float eps, int t, int n, float* out,
                   cudaStream_t stream);

}  // namespace tc
