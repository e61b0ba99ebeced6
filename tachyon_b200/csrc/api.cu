// The C ABI (include/tachyon_cuda.h): context, device buffers, weight upload,
// the MoE block and stream capture. Host-side only; kernels live in the other
// files of this directory.
#include "../../include/tachyon_cuda.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "ep.cuh"

struct tc_ctx {
    int device = 0;
    int sms = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev_start = nullptr, ev_stop = nullptr;
    std::string name;
    std::string error;
    tc::Workspace ws;
    std::vector<void*> ws_allocs;
    uint64_t launches = 0;
    bool capturing = false;
    uint64_t launches_before_capture = 0;
    bool profiling = false;
    int arith = tc::ARITH_FAST;
    std::vector<cudaEvent_t> ev_pool;                      // reused across reads
    size_t ev_used = 0;
    struct Span { int stage; size_t a, b; int launches; };
    std::vector<Span> spans;
    tc::EpState ep;           // expert parallelism (size 1 until tc_ep_init)
    tc::PrefillScratch pre;   // token tiles of the tcgen05 path
    std::vector<void*> pre_allocs;
    int prefill_min_avg = 32; // tokens per expert (on average) from which the tcgen05 kernels take over
    float* host_x = nullptr;  // device staging for the host-buffer entry point
    float* host_y = nullptr;
    size_t host_elems = 0;
    bool decode_block = true;      // decode-size blocks as one kernel (moe_decode.cu)
    int decode_block_tokens = 128; // ... up to this many tokens (above 32: through the window below)
    // Batches of 33 tokens and more take the one-kernel path in its expert-parallel form with
    // this GPU as the only rank: a window like a peer window, in local memory. The arrival
    // counters sit at its start, so they stay where they are whatever the shape of the launch.
    uint8_t* self_window = nullptr;
    uint32_t* self_epoch = nullptr;
    size_t self_bytes = 0;
    uint32_t grid_spin_limit = 1u << 22;
    unsigned long long* phase_stamps = nullptr;  // device [8], while phase profiling is on
    int* static_status = nullptr;  // status word of tc_dispatch_static on this device, once it has been used
};

struct tc_matrix {
    tc_ctx* ctx;
    tc::MatrixDev dev;
    void* scales_alloc;
    void* data_alloc;
};

struct tc_moe_layer {
    tc_ctx* ctx;
    tc::MoeDims dims;
    const tc_matrix *router, *gate_up, *down;  // (gate_up / down: null once the experts are detached)
    float* bias = nullptr;
    int max_tokens;
    int last_t = 0;
    bool dispatch_stale = false;       // the last forward built no dispatch (one-kernel block): built on demand
    uint8_t* gate_up_tiled = nullptr;  // the fast kernels' record layout of the two expert matrices
    uint8_t* down_tiled = nullptr;
    tc::PrefillWeights pw;             // the tcgen05 kernels' tiles of the two expert matrices
    std::vector<void*> pw_allocs;
    bool ep = false;                   // expert-parallel layer: gate_up/down hold this rank's experts only
    tc::EpLayerBuffers epb;
    tc::MatrixDev gu, dn;              // the expert matrices as uploaded (pointers null once detached)
};

struct tc_graph {
    tc_ctx* ctx;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    uint64_t launches;  // kernels recorded in the graph
};

namespace {

int fail(tc_ctx* ctx, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->error = buf;
    return -1;
}

bool cuda_ok(tc_ctx* ctx, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return true;
    fail(ctx, "%s: %s", what, cudaGetErrorString(e));
    return false;
}

void copy_message(const std::string& s, char* out, size_t len) {
    if (!out || len == 0) return;
    size_t n = s.size() < len - 1 ? s.size() : len - 1;
    memcpy(out, s.data(), n);
    out[n] = 0;
}

size_t pad8(size_t v) { return (v + 7) / 8 * 8; }

size_t next_event(tc_ctx* ctx) {
    if (ctx->ev_used == ctx->ev_pool.size()) {
        cudaEvent_t e;
        cudaEventCreate(&e);
        ctx->ev_pool.push_back(e);
    }
    return ctx->ev_used++;
}

// Runs one launcher, bracketed by events when profiling outside a capture.
template <class F>
int staged(tc_ctx* ctx, int stage, F launch) {
    const bool timed = ctx->profiling && !ctx->capturing;
    size_t a = 0;
    if (timed) {
        a = next_event(ctx);
        cudaEventRecord(ctx->ev_pool[a], ctx->stream);
    }
    int n = launch();
    if (timed) {
        size_t b = next_event(ctx);
        cudaEventRecord(ctx->ev_pool[b], ctx->stream);
        ctx->spans.push_back({stage, a, b, n});
    }
    return n;
}

template <class T>
bool ws_alloc(tc_ctx* ctx, T*& p, size_t elems) {
    void* raw = nullptr;
    if (!cuda_ok(ctx, cudaMalloc(&raw, elems * sizeof(T) + 256), "cudaMalloc(workspace)")) return false;
    ctx->ws_allocs.push_back(raw);
    p = static_cast<T*>(raw);
    return true;
}

void ws_release(tc_ctx* ctx) {
    for (void* p : ctx->ws_allocs) cudaFree(p);
    ctx->ws_allocs.clear();
    ctx->ws = tc::Workspace{};
}

// Scratch of the tcgen05 path: token tiles for up to max_tokens * topk slots. Shared by
// the context's layers, so it only ever grows: every dimension is the largest any
// layer has asked for. Growing it frees the old buffers, which invalidates graphs
// captured earlier; create every layer before capturing.
bool prefill_reserve(tc_ctx* ctx, const tc::MoeDims& d, int max_tokens) {
    const int tiles = tc::prefill_max_token_tiles(max_tokens * d.topk, d.experts);
    const int nb = std::max(d.hidden, d.inter) / 32;
    tc::PrefillScratch& p = ctx->pre;
    const size_t per_tile = size_t(nb) * tc::prefill_token_tile() * 32;
    if (p.max_tiles >= tiles && p.xt_bytes >= size_t(tiles) * per_tile && p.tile_bytes >= per_tile) return true;
    const int T = std::max(tiles, p.max_tiles);
    const size_t tile_bytes = std::max(per_tile, p.tile_bytes);
    const size_t xt_bytes = size_t(T) * tile_bytes, xst_elems = xt_bytes / 32;
    cudaStreamSynchronize(ctx->stream);
    for (void* q : ctx->pre_allocs) cudaFree(q);
    ctx->pre_allocs.clear();
    p = tc::PrefillScratch{};
    auto get = [&](auto*& dst, size_t bytes) {
        void* raw = nullptr;
        if (!cuda_ok(ctx, cudaMalloc(&raw, bytes + 256), "cudaMalloc(prefill scratch)")) return false;
        ctx->pre_allocs.push_back(raw);
        dst = static_cast<std::remove_reference_t<decltype(dst)>>(raw);
        return true;
    };
    if (!(get(p.tile_expert, size_t(T) * 4) && get(p.tile_n, size_t(T) * 4) && get(p.tile_count, 4) &&
          get(p.tile_p0, size_t(T) * 4) && get(p.xt, xt_bytes) && get(p.xst, xst_elems * 4) &&
          get(p.xsumt, xst_elems * 4))) {
        for (void* q : ctx->pre_allocs) cudaFree(q);
        ctx->pre_allocs.clear();
        p = tc::PrefillScratch{};
        return false;
    }
    p.max_tiles = T;
    p.tile_bytes = tile_bytes;
    p.xt_bytes = xt_bytes;
    p.xst_elems = xst_elems;
    return true;
}

constexpr size_t SELF_FLAG_BYTES = 256;
constexpr int SELF_WINDOW_TOKENS = 128;

// The one-rank window's layout for a block of t tokens; returns the bytes it needs.
size_t self_window_layout(const tc::MoeDims& d, int t, tc::DecodeEp* e) {
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    const size_t nbp = size_t(pad8(d.hidden / 32));
    size_t o = SELF_FLAG_BYTES;
    const size_t xq = o;
    o = up(o + size_t(t) * d.hidden);
    const size_t xs = o;
    o = up(o + size_t(t) * nbp * 4);
    const size_t xsum = o;
    o = up(o + size_t(t) * nbp * 4);
    const size_t ids = o;
    o = up(o + size_t(t) * d.topk * 4);
    const size_t out = o;
    o = up(o + size_t(t) * d.topk * d.hidden * 4);
    if (e) e->off_flags = 0, e->off_xq = xq, e->off_xs = xs, e->off_xsum = xsum, e->off_ids = ids, e->off_out = out;
    return o;
}

// Room in the one-rank window for blocks of this shape (it only grows; growing it frees the old
// one, which invalidates graphs captured earlier: create every layer before capturing).
bool self_window_reserve(tc_ctx* ctx, const tc::MoeDims& d, int max_tokens) {
    if (max_tokens <= 32) return true;  // those blocks need no window
    const size_t need = self_window_layout(d, std::min(max_tokens, SELF_WINDOW_TOKENS), nullptr);
    if (need <= ctx->self_bytes) return true;
    cudaStreamSynchronize(ctx->stream);
    if (ctx->self_window) cudaFree(ctx->self_window);
    ctx->self_window = nullptr, ctx->self_bytes = 0;
    if (!ctx->self_epoch) {
        if (!cuda_ok(ctx, cudaMalloc(reinterpret_cast<void**>(&ctx->self_epoch), 32), "cudaMalloc(window)")) return false;
    }
    if (!cuda_ok(ctx, cudaMalloc(reinterpret_cast<void**>(&ctx->self_window), need), "cudaMalloc(window)")) return false;
    cudaMemset(ctx->self_window, 0, SELF_FLAG_BYTES);
    cudaMemset(ctx->self_epoch, 0, 32);
    ctx->self_bytes = need;
    return true;
}

// Grows the context's scratch so a layer of these dimensions fits.
bool ws_reserve(tc_ctx* ctx, const tc::MoeDims& d, int max_tokens) {
    tc::Workspace& w = ctx->ws;
    if (w.max_tokens >= max_tokens && w.hidden >= d.hidden && w.experts >= d.experts &&
        w.topk >= d.topk && w.inter >= d.inter)
        return true;
    tc::MoeDims n{std::max(w.hidden, d.hidden), std::max(w.experts, d.experts),
                  std::max(w.topk, d.topk), std::max(w.inter, d.inter)};
    int T = std::max(w.max_tokens, max_tokens);
    cudaStreamSynchronize(ctx->stream);
    ws_release(ctx);
    size_t slots = size_t(T) * n.topk;
    size_t blocks = (size_t(T) + 255) / 256;
    bool ok = ws_alloc(ctx, w.logits, size_t(T) * n.experts) && ws_alloc(ctx, w.ids, slots) &&
              ws_alloc(ctx, w.gates, slots) && ws_alloc(ctx, w.xq, size_t(T) * n.hidden) &&
              ws_alloc(ctx, w.xs, size_t(T) * pad8(n.hidden / 32)) &&
              ws_alloc(ctx, w.xsum, size_t(T) * pad8(n.hidden / 32)) &&
              ws_alloc(ctx, w.counts, size_t(n.experts)) &&
              ws_alloc(ctx, w.offsets, size_t(n.experts) + 1) && ws_alloc(ctx, w.perm, slots) &&
              ws_alloc(ctx, w.pos, slots) && ws_alloc(ctx, w.slot_token, slots) &&
              ws_alloc(ctx, w.active, size_t(n.experts) + 1) && ws_alloc(ctx, w.block_hist, blocks * n.experts) &&
              ws_alloc(ctx, w.hidden_f, slots * n.inter) && ws_alloc(ctx, w.hq, slots * n.inter) &&
              ws_alloc(ctx, w.hs, slots * pad8(n.inter / 32)) &&
              ws_alloc(ctx, w.hsum, slots * pad8(n.inter / 32)) &&
              ws_alloc(ctx, w.out, slots * n.hidden) && ws_alloc(ctx, w.status, size_t(1)) &&
              ws_alloc(ctx, w.ticket, size_t(1)) && ws_alloc(ctx, w.grid_sync, size_t(tc::GRID_SYNC_WORDS));
    if (!ok) {
        ws_release(ctx);
        return false;
    }
    cudaMemset(w.status, 0, sizeof(int));
    cudaMemset(w.ticket, 0, sizeof(int));
    cudaMemset(w.grid_sync, 0, tc::GRID_SYNC_WORDS * sizeof(uint32_t));
    w.max_tokens = T;
    w.sms = ctx->sms;
    w.hidden = n.hidden;
    w.experts = n.experts;
    w.topk = n.topk;
    w.inter = n.inter;
    return true;
}

}  // namespace

namespace tc {
bool g_launch_overlap = true;
}

extern "C" {

tc_ctx* tc_create(int device_ordinal, char* err, size_t errlen) {
    auto bail = [&](const std::string& m) -> tc_ctx* {
        copy_message(m, err, errlen);
        return nullptr;
    };
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) return bail(std::string("no CUDA device: ") + cudaGetErrorString(e));
    if (device_ordinal < 0 || device_ordinal >= count) return bail("device ordinal out of range");
    if ((e = cudaSetDevice(device_ordinal)) != cudaSuccess)
        return bail(std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device_ordinal)) != cudaSuccess)
        return bail(std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
    if (prop.major != 10)
        return bail(std::string("this library is built for sm_100a only; found ") + prop.name);
    tc_ctx* ctx = new tc_ctx;
    ctx->device = device_ordinal;
    ctx->sms = prop.multiProcessorCount;
    ctx->name = prop.name;
    tc::init_kernels_exact();
    tc::init_kernels_fast();
    tc::init_kernels_route();
    tc::init_kernels_prefill();
    tc::init_kernels_decode();
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreate(&ctx->ev_start) != cudaSuccess ||
        cudaEventCreate(&ctx->ev_stop) != cudaSuccess) {
        delete ctx;
        return bail("could not create the stream or events");
    }
    return ctx;
}

void tc_destroy(tc_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    ws_release(ctx);
    for (void* q : ctx->pre_allocs) cudaFree(q);
    if (ctx->host_x) cudaFree(ctx->host_x);
    if (ctx->host_y) cudaFree(ctx->host_y);
    if (ctx->phase_stamps) cudaFree(ctx->phase_stamps);
    if (ctx->self_window) cudaFree(ctx->self_window);
    if (ctx->self_epoch) cudaFree(ctx->self_epoch);
    tc::ep_destroy(ctx->ep);
    for (cudaEvent_t e : ctx->ev_pool) cudaEventDestroy(e);
    cudaEventDestroy(ctx->ev_start);
    cudaEventDestroy(ctx->ev_stop);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

void tc_device_name(tc_ctx* ctx, char* out, size_t len) { copy_message(ctx->name, out, len); }

size_t tc_last_error(tc_ctx* ctx, char* out, size_t len) {
    copy_message(ctx->error, out, len);
    return ctx->error.size();
}

void* tc_stream(tc_ctx* ctx) { return ctx->stream; }

namespace {
const char* status_text(int status) {
    switch (status) {
        case tc::ERR_COPY_WAIT_TIMEOUT: return "a staged copy did not arrive within a kernel's wait limit";
        case tc::ERR_PEER_WAIT_TIMEOUT: return "another rank's signal did not arrive within a kernel's wait limit";
        case tc::ERR_BAD_EXPERT_ID: return "the dispatch met an expert id out of range or named twice by one token";
        case tc::ERR_GRID_WAIT_TIMEOUT: return "a kernel's CTAs gave up waiting for one another";
        default: return "unknown status";
    }
}
}  // namespace

int tc_sync(tc_ctx* ctx) {
    if (!cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize")) return -1;
    int* words[2] = {ctx->ws.status, ctx->static_status};
    int worst = 0;
    for (int* w : words) {
        if (!w) continue;
        int status = 0;
        if (!cuda_ok(ctx, cudaMemcpy(&status, w, sizeof status, cudaMemcpyDeviceToHost), "status readback"))
            return -1;
        if (status != 0) {
            cudaMemset(w, 0, sizeof(int));
            worst = status;
        }
    }
    if (worst) {
        // A kernel that gave up may have left its arrival counters part-way: start clean.
        if (ctx->ws.ticket) cudaMemset(ctx->ws.ticket, 0, sizeof(int));
        if (ctx->ws.grid_sync) cudaMemset(ctx->ws.grid_sync, 0, tc::GRID_SYNC_WORDS * sizeof(uint32_t));
        if (ctx->self_window) {
            cudaMemset(ctx->self_window, 0, SELF_FLAG_BYTES);
            cudaMemset(ctx->self_epoch, 0, 32);
        }
        return fail(ctx, "a kernel reported status %d: %s", worst, status_text(worst));
    }
    return 0;
}

void* tc_malloc(tc_ctx* ctx, size_t bytes) {
    void* p = nullptr;
    cudaSetDevice(ctx->device);
    if (!cuda_ok(ctx, cudaMalloc(&p, bytes ? bytes : 1), "cudaMalloc")) return nullptr;
    return p;
}

void tc_free(tc_ctx* ctx, void* dev) {
    if (!dev) return;
    cudaSetDevice(ctx->device);
    cudaFree(dev);
}

int tc_upload(tc_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!cuda_ok(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream), "upload"))
        return -1;
    return cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "upload sync") ? 0 : -1;
}

int tc_download(tc_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!cuda_ok(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream),
                 "download"))
        return -1;
    return cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "download sync") ? 0 : -1;
}

int tc_memset(tc_ctx* ctx, void* dst, int value, size_t bytes) {
    return cuda_ok(ctx, cudaMemsetAsync(dst, value, bytes, ctx->stream), "memset") ? 0 : -1;
}

int tc_copy(tc_ctx* ctx, void* dst, const void* src, size_t bytes) {
    return cuda_ok(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream), "copy") ? 0 : -1;
}

void* tc_host_alloc(tc_ctx* ctx, size_t bytes) {
    void* p = nullptr;
    if (!cuda_ok(ctx, cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault), "cudaHostAlloc")) return nullptr;
    return p;
}

void tc_host_free(tc_ctx* ctx, void* host) {
    (void)ctx;
    if (host) cudaFreeHost(host);
}

int tc_set_arithmetic(tc_ctx* ctx, int mode) {
    if (mode != TC_ARITH_FAST && mode != TC_ARITH_CPU_LANES) return fail(ctx, "unknown arithmetic mode %d", mode);
    ctx->arith = mode;
    return 0;
}

int tc_set_launch_overlap(tc_ctx* ctx, int on) {
    (void)ctx;
    tc::g_launch_overlap = on != 0;
    return 0;
}

int tc_set_decode_block(tc_ctx* ctx, int on) {
    ctx->decode_block = on != 0;
    ctx->decode_block_tokens = on > 1 ? std::min(on, SELF_WINDOW_TOKENS) : SELF_WINDOW_TOKENS;
    return 0;
}

int tc_profile_phases(tc_ctx* ctx, int on) {
    if (on && !ctx->phase_stamps) {
        cudaSetDevice(ctx->device);
        if (!cuda_ok(ctx, cudaMalloc(reinterpret_cast<void**>(&ctx->phase_stamps), 8 * sizeof(unsigned long long)),
                     "cudaMalloc(phase stamps)"))
            return -1;
        cudaMemset(ctx->phase_stamps, 0, 8 * sizeof(unsigned long long));
    } else if (!on && ctx->phase_stamps) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(ctx->phase_stamps);
        ctx->phase_stamps = nullptr;
    }
    return 0;
}

int tc_profile_read_phases(tc_ctx* ctx, uint64_t* ns6) {
    if (!ctx->phase_stamps) return fail(ctx, "phase profiling is off");
    if (!cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize")) return -1;
    return cuda_ok(ctx, cudaMemcpy(ns6, ctx->phase_stamps, 6 * sizeof(uint64_t), cudaMemcpyDeviceToHost),
                   "phase stamp readback") ? 0 : -1;
}

int tc_set_prefill_threshold(tc_ctx* ctx, int avg_tokens_per_expert) {
    if (avg_tokens_per_expert < 0) return fail(ctx, "the threshold cannot be negative");
    ctx->prefill_min_avg = avg_tokens_per_expert;
    return 0;
}

int tc_profile_enable(tc_ctx* ctx, int on) {
    ctx->profiling = on != 0;
    return 0;
}

int tc_profile_read(tc_ctx* ctx, float* ms, uint64_t* launches) {
    if (!cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize")) return -1;
    for (int i = 0; i < TC_PROFILE_STAGES; i++) {
        if (ms) ms[i] = 0.0f;
        if (launches) launches[i] = 0;
    }
    for (const auto& sp : ctx->spans) {
        float t = 0.0f;
        if (!cuda_ok(ctx, cudaEventElapsedTime(&t, ctx->ev_pool[sp.a], ctx->ev_pool[sp.b]), "cudaEventElapsedTime"))
            return -1;
        if (ms) ms[sp.stage] += t;
        if (launches) launches[sp.stage] += sp.launches;
    }
    ctx->spans.clear();
    ctx->ev_used = 0;
    return 0;
}

tc_matrix* tc_matrix_upload(tc_ctx* ctx, int kind, size_t rows, size_t cols, const void* scales,
                            size_t scales_bytes, const void* data, size_t data_bytes) {
    if (cols % 32 != 0) {
        fail(ctx, "GPU matrices need a multiple of 32 columns, not %zu", cols);
        return nullptr;
    }
    size_t want_scales = 0, want_data = 0;
    switch (kind) {
        case TC_BF16:
            want_data = rows * cols * 2;
            break;
        case TC_Q8:
            want_scales = rows * (cols / 32) * 2;
            want_data = rows * cols;
            break;
        case TC_Q4:
            want_scales = rows * ((cols / 32 + 7) / 8 * 5) * 4;
            want_data = rows * cols / 2;
            break;
        default:
            fail(ctx, "unknown matrix kind %d", kind);
            return nullptr;
    }
    if (scales_bytes != want_scales || data_bytes != want_data) {
        fail(ctx, "matrix buffers are %zu+%zu bytes, expected %zu+%zu for %zux%zu kind %d",
             scales_bytes, data_bytes, want_scales, want_data, rows, cols, kind);
        return nullptr;
    }
    cudaSetDevice(ctx->device);
    tc_matrix* m = new tc_matrix{ctx, {kind, rows, cols, nullptr, nullptr}, nullptr, nullptr};
    // Padded so that staged copies of a partial last chunk stay inside the allocation.
    if (want_scales) {
        if (!cuda_ok(ctx, cudaMalloc(&m->scales_alloc, want_scales + 256), "cudaMalloc(scales)") ||
            !cuda_ok(ctx, cudaMemcpy(m->scales_alloc, scales, want_scales, cudaMemcpyHostToDevice),
                     "scales upload")) {
            tc_matrix_free(m);
            return nullptr;
        }
    }
    if (!cuda_ok(ctx, cudaMalloc(&m->data_alloc, want_data + 256), "cudaMalloc(weights)") ||
        !cuda_ok(ctx, cudaMemcpy(m->data_alloc, data, want_data, cudaMemcpyHostToDevice),
                 "weights upload")) {
        tc_matrix_free(m);
        return nullptr;
    }
    m->dev.scales = m->scales_alloc;
    m->dev.data = m->data_alloc;
    return m;
}

namespace {
bool matrix_sizes(int kind, size_t rows, size_t cols, size_t* scales_bytes, size_t* data_bytes) {
    switch (kind) {
        case TC_BF16: *scales_bytes = 0, *data_bytes = rows * cols * 2; return true;
        case TC_Q8: *scales_bytes = rows * (cols / 32) * 2, *data_bytes = rows * cols; return true;
        case TC_Q4: *scales_bytes = rows * ((cols / 32 + 7) / 8 * 5) * 4, *data_bytes = rows * cols / 2; return true;
        default: return false;
    }
}
}  // namespace

tc_matrix* tc_matrix_quantize(tc_ctx* ctx, int kind, size_t rows, size_t cols, const float* data_host) {
    size_t want_scales = 0, want_data = 0;
    if (!matrix_sizes(kind, rows, cols, &want_scales, &want_data)) {
        fail(ctx, "unknown matrix kind %d", kind);
        return nullptr;
    }
    if (cols % 32 != 0 || rows == 0 || cols == 0) {
        fail(ctx, "GPU matrices need a positive multiple of 32 columns, not %zu x %zu", rows, cols);
        return nullptr;
    }
    cudaSetDevice(ctx->device);
    tc_matrix* m = new tc_matrix{ctx, {kind, rows, cols, nullptr, nullptr}, nullptr, nullptr};
    float *src = nullptr, *scratch = nullptr;
    const size_t n = rows * cols;
    bool ok = cuda_ok(ctx, cudaMalloc(reinterpret_cast<void**>(&src), n * 4), "cudaMalloc(f32 weights)") &&
              cuda_ok(ctx, cudaMemcpyAsync(src, data_host, n * 4, cudaMemcpyHostToDevice, ctx->stream), "f32 upload") &&
              cuda_ok(ctx, cudaMalloc(&m->data_alloc, want_data + 256), "cudaMalloc(weights)");
    if (ok && want_scales) ok = cuda_ok(ctx, cudaMalloc(&m->scales_alloc, want_scales + 256), "cudaMalloc(scales)");
    if (ok && kind == TC_Q4)
        ok = cuda_ok(ctx, cudaMalloc(reinterpret_cast<void**>(&scratch), (rows + 2 * (n / 32)) * 4), "cudaMalloc(fit)");
    if (ok) {
        ctx->launches += tc::launch_quantize(kind, src, rows, cols, m->scales_alloc, m->data_alloc, scratch, ctx->stream);
        ok = cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "quantization");
    }
    if (src) cudaFree(src);
    if (scratch) cudaFree(scratch);
    if (!ok) {
        tc_matrix_free(m);
        return nullptr;
    }
    m->dev.scales = m->scales_alloc;
    m->dev.data = m->data_alloc;
    return m;
}

int tc_matrix_download(const tc_matrix* m, void* scales_host, size_t scales_bytes, void* data_host, size_t data_bytes) {
    tc_ctx* ctx = m->ctx;
    size_t want_scales = 0, want_data = 0;
    matrix_sizes(m->dev.kind, m->dev.rows, m->dev.cols, &want_scales, &want_data);
    if (scales_bytes != want_scales || data_bytes != want_data)
        return fail(ctx, "tc_matrix_download: buffers of %zu+%zu bytes, the matrix holds %zu+%zu", scales_bytes,
                    data_bytes, want_scales, want_data);
    cudaSetDevice(ctx->device);
    if (want_scales && !cuda_ok(ctx, cudaMemcpy(scales_host, m->dev.scales, want_scales, cudaMemcpyDeviceToHost),
                                "scales download"))
        return -1;
    return cuda_ok(ctx, cudaMemcpy(data_host, m->dev.data, want_data, cudaMemcpyDeviceToHost), "weights download") ? 0 : -1;
}

void tc_matrix_free(tc_matrix* m) {
    if (!m) return;
    cudaSetDevice(m->ctx->device);
    if (m->scales_alloc) cudaFree(m->scales_alloc);
    if (m->data_alloc) cudaFree(m->data_alloc);
    delete m;
}

namespace {
tc_moe_layer* layer_create(tc_ctx* ctx, int hidden, int experts, int k, int inter, const tc_matrix* router,
                           const tc_matrix* gate_up, const tc_matrix* down, int max_tokens, bool ep);
}

tc_moe_layer* tc_moe_layer_create(tc_ctx* ctx, int hidden, int experts, int k, int inter,
                                  const tc_matrix* router, const tc_matrix* gate_up,
                                  const tc_matrix* down, int max_tokens) {
    return layer_create(ctx, hidden, experts, k, inter, router, gate_up, down, max_tokens, false);
}

tc_moe_layer* tc_moe_ep_layer_create(tc_ctx* ctx, int hidden, int experts, int k, int inter,
                                     const tc_matrix* router, const tc_matrix* gate_up_local,
                                     const tc_matrix* down_local, int max_tokens) {
    if (!ctx->ep.comm) {
        fail(ctx, "tc_moe_ep_layer_create: call tc_ep_init first");
        return nullptr;
    }
    return layer_create(ctx, hidden, experts, k, inter, router, gate_up_local, down_local, max_tokens, true);
}

int tc_ep_unique_id(char* out128) { return tc::ep_unique_id(out128) ? -1 : 0; }

int tc_ep_init(tc_ctx* ctx, const char* id128, int rank, int size) {
    cudaSetDevice(ctx->device);
    const char* why = tc::ep_init(ctx->ep, id128, rank, size);
    return why ? fail(ctx, "tc_ep_init: %s", why) : 0;
}

int tc_ep_enable_peer_exchange(tc_ctx* ctx, int hidden, int experts_per_token, int max_tokens) {
    cudaSetDevice(ctx->device);
    const char* why = tc::ep_peer_enable(ctx->ep, hidden, experts_per_token, max_tokens);
    return why ? fail(ctx, "tc_ep_enable_peer_exchange: %s", why) : 0;
}

int tc_ep_set_wait_limit(tc_ctx* ctx, uint32_t polls) {
    if (polls == 0) return fail(ctx, "the wait limit must be at least one poll");
    ctx->ep.peer.wait_limit = polls;
    return 0;
}

int tc_ep_test_mute_signals(tc_ctx* ctx, int blocks) {
    if (!ctx->ep.peer.on) return fail(ctx, "tc_ep_test_mute_signals: the peer-memory exchange is not enabled");
    ctx->ep.peer.mute_next = blocks < 0 ? 0 : blocks;
    return 0;
}

int tc_ep_barrier(tc_ctx* ctx) {
    cudaSetDevice(ctx->device);
    const char* why = tc::ep_barrier(ctx->ep, ctx->stream);
    return why ? fail(ctx, "tc_ep_barrier: %s", why) : 0;
}

int tc_ep_set_uniform_batch(tc_ctx* ctx, int on) {
    ctx->ep.uni.on = on != 0;
    return 0;
}

int tc_ep_expert_range(int experts, int rank, int size, int* first, int* count) {
    if (size < 1 || rank < 0 || rank >= size) return -1;
    tc::ep_expert_range(experts, rank, size, first, count);
    return 0;
}

}  // extern "C"

namespace {
tc_moe_layer* layer_create(tc_ctx* ctx, int hidden, int experts, int k, int inter, const tc_matrix* router,
                           const tc_matrix* gate_up, const tc_matrix* down, int max_tokens, bool ep) {
    auto bad = [&](const char* why) -> tc_moe_layer* {
        fail(ctx, "tc_moe_layer_create: %s", why);
        return nullptr;
    };
    int local = experts, first = 0;
    if (ep) tc::ep_expert_range(experts, ctx->ep.rank, ctx->ep.size, &first, &local);
    (void)first;
    if (!router || !gate_up || !down) return bad("a matrix is null");
    if (hidden <= 0 || hidden % 32 || inter <= 0 || inter % 32)
        return bad("hidden and intermediate sizes must be positive multiples of 32");
    if (experts <= 0 || experts > tc::MAX_EXPERTS) return bad("between 1 and 256 experts");
    if (k <= 0 || k > tc::MAX_TOPK || k > experts) return bad("between 1 and min(32, experts) experts per token");
    if (max_tokens <= 0) return bad("max_tokens must be positive");
    if (router->dev.kind != TC_BF16 || router->dev.rows != size_t(experts) ||
        router->dev.cols != size_t(hidden))
        return bad("the router must be bf16 [experts, hidden]");
    if (gate_up->dev.kind == TC_BF16 || down->dev.kind == TC_BF16)
        return bad("expert matrices must be 8-bit or 4-bit");
    if (gate_up->dev.rows != size_t(local) * 2 * inter || gate_up->dev.cols != size_t(hidden))
        return bad("gate_up must be [experts*2*inter, hidden] (this rank's experts when expert-parallel)");
    if (down->dev.rows != size_t(local) * hidden || down->dev.cols != size_t(inter))
        return bad("down must be [experts*hidden, inter] (this rank's experts when expert-parallel)");
    if (ep && local == 0) return bad("more ranks than experts");
    cudaSetDevice(ctx->device);
    tc::MoeDims d{hidden, experts, k, inter};
    if (!ws_reserve(ctx, d, max_tokens)) return nullptr;
    if (!ep && !self_window_reserve(ctx, d, max_tokens)) return nullptr;
    if (!tc::fast_path_fits(d, gate_up->dev, down->dev)) return bad("hidden or intermediate size too large for the staged-token buffers");
    tc_moe_layer* l = new tc_moe_layer{ctx, d, router, gate_up, down, nullptr, max_tokens, 0};
    l->ep = ep;
    l->gu = gate_up->dev, l->dn = down->dev;
    tc::MoeDims dl = d;  // the shape of the matrices held here
    dl.experts = local;
    if (ep && ctx->ep.uni.on && !tc::ep_uniform_reserve(ctx->ep, d, max_tokens)) {
        delete l;
        return bad("could not allocate the fixed-size exchange buffers");
    }
    if (ep && !tc::ep_layer_alloc(l->epb, ctx->ep, d, max_tokens)) {
        tc::ep_layer_free(l->epb);
        delete l;
        return bad("could not allocate the exchange buffers");
    }
    void *gu = nullptr, *dn = nullptr;
    if (!cuda_ok(ctx, cudaMalloc(&gu, tc::tiled_bytes(dl, gate_up->dev, true) + 256), "cudaMalloc(tiled gate_up)") ||
        !cuda_ok(ctx, cudaMalloc(&dn, tc::tiled_bytes(dl, down->dev, false) + 256), "cudaMalloc(tiled down)")) {
        if (gu) cudaFree(gu);
        delete l;
        return nullptr;
    }
    l->gate_up_tiled = static_cast<uint8_t*>(gu);
    l->down_tiled = static_cast<uint8_t*>(dn);
    tc::tile_weights(dl, gate_up->dev, true, l->gate_up_tiled, ctx->stream);
    tc::tile_weights(dl, down->dev, false, l->down_tiled, ctx->stream);
    // (Expert-parallel layers: tiles of this rank's experts; scratch for every rank's tokens.)
    const tc::MoeDims& dp = ep ? dl : d;
    if (tc::prefill_fits(dp, gate_up->dev.kind == TC_Q4, down->dev.kind == TC_Q4) &&
        prefill_reserve(ctx, d, ep ? max_tokens * ctx->ep.size : max_tokens)) {
        // Third copy of the experts, for prefill-size groups: int8 tiles in the tensor core's
        // canonical order and f32 block scales.
        auto get = [&](auto*& dst, size_t bytes) {
            void* raw = nullptr;
            if (!cuda_ok(ctx, cudaMalloc(&raw, bytes + 256), "cudaMalloc(prefill weights)")) return false;
            l->pw_allocs.push_back(raw);
            dst = static_cast<std::remove_reference_t<decltype(dst)>>(raw);
            return true;
        };
        const bool q4g = gate_up->dev.kind == TC_Q4, q4d = down->dev.kind == TC_Q4;
        bool okp = get(l->pw.gu_t, tc::prefill_weight_bytes(dp, true)) && get(l->pw.gu_d, tc::prefill_scale_elems(dp, true) * 4) &&
                   get(l->pw.dn_t, tc::prefill_weight_bytes(dp, false)) && get(l->pw.dn_d, tc::prefill_scale_elems(dp, false) * 4);
        if (okp && q4g) okp = get(l->pw.gu_c, tc::prefill_scale_elems(dp, true) * 4);
        if (okp && q4d) okp = get(l->pw.dn_c, tc::prefill_scale_elems(dp, false) * 4);
        if (!okp) {
            tc_moe_layer_free(l);
            return nullptr;
        }
        tc::tile_prefill_weights(dp, gate_up->dev, true, l->pw.gu_t, l->pw.gu_d, l->pw.gu_c, ctx->stream);
        tc::tile_prefill_weights(dp, down->dev, false, l->pw.dn_t, l->pw.dn_d, l->pw.dn_c, ctx->stream);
    }
    if (!cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "weight tiling")) {
        tc_moe_layer_free(l);
        return nullptr;
    }
    return l;
}
}  // namespace

extern "C" {

void tc_moe_layer_free(tc_moe_layer* layer) {
    if (!layer) return;
    if (layer->bias) cudaFree(layer->bias);
    for (void* q : layer->pw_allocs) cudaFree(q);
    if (layer->ep) tc::ep_layer_free(layer->epb);
    if (layer->gate_up_tiled) cudaFree(layer->gate_up_tiled);
    if (layer->down_tiled) cudaFree(layer->down_tiled);
    delete layer;
}

int tc_moe_layer_detach_experts(tc_moe_layer* layer) {
    tc_ctx* ctx = layer->ctx;
    // Anything still reading the uploaded copies (a layer being created, an exact-order block) is done first.
    if (!cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize")) return -1;
    layer->gu.data = layer->gu.scales = nullptr;
    layer->dn.data = layer->dn.scales = nullptr;
    layer->gate_up = layer->down = nullptr;
    return 0;
}

int tc_moe_set_router_bias(tc_moe_layer* layer, const float* bias_host) {
    tc_ctx* ctx = layer->ctx;
    if (!bias_host) {
        if (layer->bias) cudaFree(layer->bias);
        layer->bias = nullptr;
        return 0;
    }
    if (!layer->bias &&
        !cuda_ok(ctx, cudaMalloc(&layer->bias, layer->dims.experts * sizeof(float)), "cudaMalloc(bias)"))
        return -1;
    return tc_upload(ctx, layer->bias, bias_host, layer->dims.experts * sizeof(float));
}

}  // extern "C"

namespace {

// The block: route (+ optional norm), dispatch, experts, combine. x is the
// normed input, or the residual stream itself when norm_w is given.
int moe_enqueue(tc_moe_layer* layer, const float* x, const float* norm_w, float eps, int t, float* y) {
    tc_ctx* ctx = layer->ctx;
    if (t <= 0) return fail(ctx, "empty batch");
    if (t > layer->max_tokens) return fail(ctx, "%d tokens, layer was created for %d", t, layer->max_tokens);
    if (ctx->arith == tc::ARITH_CPU_LANES && !layer->gu.data)
        return fail(ctx, "TC_ARITH_CPU_LANES reads the expert matrices as uploaded, and this layer's were detached");
    const tc::MoeDims& d = layer->dims;
    tc::Workspace& ws = ctx->ws;
    cudaStream_t s = ctx->stream;
    int n = 0;
    if (layer->ep && tc::ep_peer_applies(ctx->ep, d, t)) {
        const char* why = tc::ep_forward_peer(ctx->ep, layer->epb, d,
                                              static_cast<const uint16_t*>(layer->router->dev.data), layer->bias,
                                              layer->gu, layer->gate_up_tiled, layer->dn,
                                              layer->down_tiled, x, norm_w, eps, t, y, ws, ctx->sms, s, &n,
                                              ctx->decode_block && ctx->arith == tc::ARITH_FAST, ctx->phase_stamps,
                                              ctx->arith == tc::ARITH_CPU_LANES ? nullptr : &layer->pw, &ctx->pre,
                                              ctx->prefill_min_avg);
        ctx->launches += n;
        layer->last_t = t;
        if (why) return fail(ctx, "expert-parallel block: %s", why);
        if (!ctx->capturing && !cuda_ok(ctx, cudaGetLastError(), "MoE launch")) return -1;
        return 0;
    }
    if (layer->ep && tc::ep_uniform_applies(ctx->ep, d, t) && ctx->ep.uni.big) {
        const char* why = tc::ep_forward_uniform(ctx->ep, layer->epb, d,
                                                 static_cast<const uint16_t*>(layer->router->dev.data), layer->bias,
                                                 layer->gu, layer->gate_up_tiled, layer->dn,
                                                 layer->down_tiled, x, norm_w, eps, t, y, ws, ctx->sms, s, &n);
        ctx->launches += n;
        layer->last_t = t;
        if (why) return fail(ctx, "expert-parallel block: %s", why);
        if (!ctx->capturing && !cuda_ok(ctx, cudaGetLastError(), "MoE launch")) return -1;
        return 0;
    }
    if (layer->ep) {
        if (ctx->capturing) return fail(ctx, "the expert-parallel block reads exchange sizes on the host: it cannot be captured");
        const char* why = tc::ep_forward(ctx->ep, layer->epb, d, static_cast<const uint16_t*>(layer->router->dev.data),
                                         layer->bias, layer->gu, layer->gate_up_tiled, layer->dn,
                                         layer->down_tiled, x, norm_w, eps, t, y, ws, ctx->sms, s, &n,
                                         ctx->arith == tc::ARITH_CPU_LANES ? nullptr : &layer->pw, &ctx->pre,
                                         ctx->prefill_min_avg);
        ctx->launches += n;
        layer->last_t = t;
        if (why) return fail(ctx, "expert-parallel block: %s", why);
        if (!cuda_ok(ctx, cudaGetLastError(), "MoE launch")) return -1;
        return 0;
    }
    const bool lanes = ctx->arith == tc::ARITH_CPU_LANES;
    layer->dispatch_stale = false;
    if (!lanes && ctx->decode_block &&
        tc::decode_block_applies(d, layer->gu.kind, layer->dn.kind, t)) {
        // Decode-size batch: the whole block is one kernel (no dispatch is built).
        n += staged(ctx, 7, [&] {
            return tc::launch_decode_block(d, layer->gu.kind,
                                           static_cast<const uint16_t*>(layer->router->dev.data), layer->bias, x,
                                           norm_w, eps, t, y, layer->gate_up_tiled, layer->down_tiled, ws, ctx->sms,
                                           ctx->grid_spin_limit, ctx->phase_stamps, s);
        });
        ctx->launches += n;
        layer->last_t = t;
        layer->dispatch_stale = true;
        if (!ctx->capturing && !cuda_ok(ctx, cudaGetLastError(), "MoE launch")) return -1;
        return 0;
    }
    const bool prefill = !lanes && layer->pw.gu_t &&
                         (long long)t * d.topk >= (long long)ctx->prefill_min_avg * d.experts;
    tc::DecodeEp self;
    if (!lanes && ctx->decode_block && t > 32 && t <= ctx->decode_block_tokens && t <= ctx->sms &&
        ctx->self_window &&
        self_window_layout(d, t, &self) <= ctx->self_bytes &&
        tc::decode_block_applies(d, layer->gu.kind, layer->dn.kind, t, 1)) {
        // Up to 128 tokens: still one kernel, in its expert-parallel form with this GPU as the only
        // rank (an expert's tokens in runs of up to 32; rows and outputs through the local window).
        // Measured at the 1b-a400m shape, 24 blocks: 1.14 ms against 1.82 at 64 tokens, 1.24 against
        // 2.17 at 96, 1.56 at 127 against 1.82 for the tcgen05 kernels at 128.
        self.ranks = 1, self.me = 0, self.first = 0, self.local = d.experts;
        self.base[0] = ctx->self_window;
        self.epoch = ctx->self_epoch + 4;
        n += staged(ctx, 7, [&] {
            return tc::launch_decode_block(d, layer->gu.kind,
                                           static_cast<const uint16_t*>(layer->router->dev.data), layer->bias, x,
                                           norm_w, eps, t, y, layer->gate_up_tiled, layer->down_tiled, ws, ctx->sms,
                                           ctx->grid_spin_limit, ctx->phase_stamps, s, &self, ws.hidden_f);
        });
        ctx->launches += n;
        layer->last_t = t;
        layer->dispatch_stale = true;
        if (!ctx->capturing && !cuda_ok(ctx, cudaGetLastError(), "MoE launch")) return -1;
        return 0;
    }
    n += staged(ctx, 0, [&] {
        return tc::launch_route(d, static_cast<const uint16_t*>(layer->router->dev.data), layer->bias,
                                x, norm_w, eps, t, ws, s);
    });
    if (prefill) {
        const int slots = t * d.topk;
        n += staged(ctx, 2, [&] {
            return tc::launch_prefill(d, true, layer->gu.kind == TC_Q4, layer->pw, ctx->pre, ws, slots,
                                      ws.hidden_f, nullptr, s);
        });
        n += staged(ctx, 4, [&] {
            return tc::launch_prefill(d, false, layer->dn.kind == TC_Q4, layer->pw, ctx->pre, ws, slots,
                                      ws.out, nullptr, s);
        });
        n += staged(ctx, 5, [&] { return tc::launch_combine(d, t, ws, y, s); });
        ctx->launches += n;
        layer->last_t = t;
        if (!ctx->capturing && !cuda_ok(ctx, cudaGetLastError(), "MoE launch")) return -1;
        return 0;
    }
    n += staged(ctx, 2, [&] {
        return lanes ? tc::launch_gate_up_exact(d, layer->gu, t, ws, ctx->sms, s)
                     : tc::launch_gate_up_fast(d, layer->gu, layer->gate_up_tiled, t, ws, ctx->sms, s);
    });
    if (lanes) n += staged(ctx, 3, [&] { return tc::launch_quant_hidden(d, t, ws, s); });
    n += staged(ctx, 4, [&] {
        return lanes ? tc::launch_down_exact(d, layer->dn, t, ws, ctx->sms, s)
                     : tc::launch_down_fast(d, layer->dn, layer->down_tiled, t, ws, ctx->sms, s);
    });
    n += staged(ctx, 5, [&] { return tc::launch_combine(d, t, ws, y, s); });
    ctx->launches += n;
    layer->last_t = t;
    if (!ctx->capturing && !cuda_ok(ctx, cudaGetLastError(), "MoE launch")) return -1;
    return 0;
}

}  // namespace

extern "C" {

int tc_moe_forward(tc_moe_layer* layer, const float* x, int t, float* y) {
    return moe_enqueue(layer, x, nullptr, 0.0f, t, y);
}

int tc_moe_block(tc_moe_layer* layer, const float* norm_weight, float eps, int t, float* y) {
    if (!norm_weight) return fail(layer->ctx, "tc_moe_block needs the norm's weight");
    return moe_enqueue(layer, y, norm_weight, eps, t, y);
}

int tc_moe_forward_host(tc_moe_layer* layer, const float* x_host, int t, float* y_host) {
    tc_ctx* ctx = layer->ctx;
    if (t <= 0) return fail(ctx, "empty batch");
    size_t elems = size_t(t) * layer->dims.hidden;
    if (elems > ctx->host_elems) {
        cudaStreamSynchronize(ctx->stream);
        if (ctx->host_x) cudaFree(ctx->host_x);
        if (ctx->host_y) cudaFree(ctx->host_y);
        ctx->host_x = ctx->host_y = nullptr;
        ctx->host_elems = 0;
        if (!cuda_ok(ctx, cudaMalloc(&ctx->host_x, elems * 4), "cudaMalloc(staging)") ||
            !cuda_ok(ctx, cudaMalloc(&ctx->host_y, elems * 4), "cudaMalloc(staging)"))
            return -1;
        ctx->host_elems = elems;
    }
    cudaStream_t s = ctx->stream;
    if (!cuda_ok(ctx, cudaMemcpyAsync(ctx->host_x, x_host, elems * 4, cudaMemcpyHostToDevice, s), "x upload") ||
        !cuda_ok(ctx, cudaMemcpyAsync(ctx->host_y, y_host, elems * 4, cudaMemcpyHostToDevice, s), "y upload"))
        return -1;
    if (tc_moe_forward(layer, ctx->host_x, t, ctx->host_y) != 0) return -1;
    if (!cuda_ok(ctx, cudaMemcpyAsync(y_host, ctx->host_y, elems * 4, cudaMemcpyDeviceToHost, s), "y download"))
        return -1;
    return tc_sync(ctx);
}

}  // extern "C"

namespace {
// The one-kernel block keeps no dispatch; the taps below build it from the ids it left.
int refresh_dispatch(tc_moe_layer* layer) {
    tc_ctx* ctx = layer->ctx;
    if (!layer->dispatch_stale) return 0;
    if (ctx->capturing) return fail(ctx, "the routing taps cannot run inside a capture");
    ctx->launches += tc::launch_dispatch(layer->dims, layer->last_t, ctx->ws, ctx->stream);
    layer->dispatch_stale = false;
    return cuda_ok(ctx, cudaGetLastError(), "dispatch launch") ? 0 : -1;
}
}  // namespace

extern "C" {

int tc_moe_last_routing(tc_moe_layer* layer, uint32_t* ids, float* gates, uint32_t* counts,
                        float* logits) {
    tc_ctx* ctx = layer->ctx;
    if (refresh_dispatch(layer) != 0) return -1;
    if (tc_sync(ctx) != 0) return -1;
    const tc::MoeDims& d = layer->dims;
    size_t slots = size_t(layer->last_t) * d.topk;
    auto get = [&](void* dst, const void* src, size_t bytes) {
        return !dst || cuda_ok(ctx, cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost), "routing readback");
    };
    if (!get(ids, ctx->ws.ids, slots * 4) || !get(gates, ctx->ws.gates, slots * 4) ||
        !get(counts, ctx->ws.counts, size_t(d.experts) * 4) ||
        !get(logits, ctx->ws.logits, size_t(layer->last_t) * d.experts * 4))
        return -1;
    return 0;
}

int tc_moe_last_dispatch(tc_moe_layer* layer, uint32_t* offsets, uint32_t* perm) {
    tc_ctx* ctx = layer->ctx;
    if (refresh_dispatch(layer) != 0) return -1;
    if (tc_sync(ctx) != 0) return -1;
    const tc::MoeDims& d = layer->dims;
    if (offsets && !cuda_ok(ctx, cudaMemcpy(offsets, ctx->ws.offsets, size_t(d.experts + 1) * 4,
                                            cudaMemcpyDeviceToHost), "dispatch readback"))
        return -1;
    if (perm && !cuda_ok(ctx, cudaMemcpy(perm, ctx->ws.perm, size_t(layer->last_t) * d.topk * 4,
                                         cudaMemcpyDeviceToHost), "dispatch readback"))
        return -1;
    return 0;
}

int tc_dispatch_static(tc_ctx* ctx, const uint32_t* ids, int t, int experts, int topk, uint32_t* counts,
                       uint32_t* offsets, uint32_t* perm, uint32_t* pos, uint32_t* slot_token, int* active) {
    const char* why = tc::dispatch_static(ctx->device, ids, t, experts, topk, counts, offsets, perm, pos,
                                          slot_token, active, ctx->stream, &ctx->static_status);
    if (why) return fail(ctx, "tc_dispatch_static: %s", why);
    ctx->launches += 3;
    return 0;
}

int tc_umma_selftest(tc_ctx* ctx, const int8_t* a_rows, const int8_t* b_rows, int n, int32_t* d_out) {
    // a_rows: 128 x 32 and b_rows: n x 32 int8, row-major on the host; d_out: 128 x n int32.
    if (n != 64 && n != 128) return fail(ctx, "tc_umma_selftest: n must be 64 or 128");
    std::vector<int8_t> ta(128 * 32), tb(size_t(n) * 32);
    auto off = [](uint32_t rows, uint32_t r, uint32_t k) {
        return (k / 16) * (rows / 8) * 128 + (r / 8) * 128 + (r % 8) * 16 + k % 16;
    };
    for (int r = 0; r < 128; r++)
        for (int k = 0; k < 32; k++) ta[off(128, r, k)] = a_rows[r * 32 + k];
    for (int r = 0; r < n; r++)
        for (int k = 0; k < 32; k++) tb[off(n, r, k)] = b_rows[r * 32 + k];
    void *da = nullptr, *db = nullptr, *dd = nullptr, *ds = nullptr;
    bool ok = cuda_ok(ctx, cudaMalloc(&da, ta.size()), "cudaMalloc") && cuda_ok(ctx, cudaMalloc(&db, tb.size()), "cudaMalloc") &&
              cuda_ok(ctx, cudaMalloc(&dd, size_t(128) * n * 4), "cudaMalloc") && cuda_ok(ctx, cudaMalloc(&ds, 4), "cudaMalloc");
    int status = 0;
    if (ok) {
        cudaMemcpy(da, ta.data(), ta.size(), cudaMemcpyHostToDevice);
        cudaMemcpy(db, tb.data(), tb.size(), cudaMemcpyHostToDevice);
        cudaMemset(dd, 0xFF, size_t(128) * n * 4);
        cudaMemset(ds, 0, 4);
        ctx->launches += tc::launch_umma_selftest(static_cast<int8_t*>(da), static_cast<int8_t*>(db), n,
                                              static_cast<int*>(dd), static_cast<int*>(ds), ctx->stream);
        ok = cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "tcgen05 self-test");
        if (ok) {
            cudaMemcpy(d_out, dd, size_t(128) * n * 4, cudaMemcpyDeviceToHost);
            cudaMemcpy(&status, ds, 4, cudaMemcpyDeviceToHost);
        }
    }
    cudaFree(da);
    cudaFree(db);
    cudaFree(dd);
    cudaFree(ds);
    if (!ok) return -1;
    if (status) return fail(ctx, "tc_umma_selftest: the MMA did not complete within the wait limit");
    return 0;
}

int tc_int8_peak(tc_ctx* ctx, int batches, double* ops_out, float* ms_out) {
    if (batches < 1) return fail(ctx, "tc_int8_peak: at least one batch");
    cudaSetDevice(ctx->device);
    int* status = nullptr;
    if (!cuda_ok(ctx, cudaMalloc(reinterpret_cast<void**>(&status), sizeof(int)), "cudaMalloc")) return -1;
    cudaMemsetAsync(status, 0, sizeof(int), ctx->stream);
    cudaEventRecord(ctx->ev_start, ctx->stream);
    const double ops = tc::launch_int8_peak(ctx->sms, batches, status, ctx->stream);
    ctx->launches += 1;
    cudaEventRecord(ctx->ev_stop, ctx->stream);
    int st = 0;
    float ms = 0.0f;
    const bool ok = cuda_ok(ctx, cudaEventSynchronize(ctx->ev_stop), "int8 peak kernel") &&
                    cuda_ok(ctx, cudaEventElapsedTime(&ms, ctx->ev_start, ctx->ev_stop), "cudaEventElapsedTime") &&
                    cuda_ok(ctx, cudaMemcpy(&st, status, sizeof st, cudaMemcpyDeviceToHost), "status readback");
    cudaFree(status);
    if (!ok) return -1;
    if (st) return fail(ctx, "tc_int8_peak: an MMA batch did not complete within the wait limit");
    if (ops_out) *ops_out = ops;
    if (ms_out) *ms_out = ms;
    return 0;
}

int tc_rmsnorm(tc_ctx* ctx, const float* x, const float* w, float eps, int t, int n, float* out) {
    if (t <= 0 || n <= 0) return fail(ctx, "rmsnorm over nothing");
    ctx->launches += staged(ctx, 6, [&] { return tc::launch_rmsnorm(x, w, eps, t, n, out, ctx->stream); });
    if (!ctx->capturing && !cuda_ok(ctx, cudaGetLastError(), "rmsnorm launch")) return -1;
    return 0;
}

int tc_capture_begin(tc_ctx* ctx) {
    if (ctx->capturing) return fail(ctx, "a capture is already open");
    if (!cuda_ok(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal),
                 "cudaStreamBeginCapture"))
        return -1;
    ctx->capturing = true;
    ctx->launches_before_capture = ctx->launches;
    return 0;
}

tc_graph* tc_capture_end(tc_ctx* ctx) {
    if (!ctx->capturing) {
        fail(ctx, "no capture is open");
        return nullptr;
    }
    ctx->capturing = false;
    ctx->launches = ctx->launches_before_capture;  // recorded, not run
    cudaGraph_t graph = nullptr;
    if (!cuda_ok(ctx, cudaStreamEndCapture(ctx->stream, &graph), "cudaStreamEndCapture")) return nullptr;
    cudaGraphExec_t exec = nullptr;
    if (!cuda_ok(ctx, cudaGraphInstantiate(&exec, graph, 0), "cudaGraphInstantiate")) {
        cudaGraphDestroy(graph);
        return nullptr;
    }
    size_t nodes = 0;
    cudaGraphGetNodes(graph, nullptr, &nodes);
    std::vector<cudaGraphNode_t> list(nodes);
    uint64_t kernels = 0;
    if (nodes && cudaGraphGetNodes(graph, list.data(), &nodes) == cudaSuccess) {
        for (size_t i = 0; i < nodes; i++) {
            cudaGraphNodeType ty;
            if (cudaGraphNodeGetType(list[i], &ty) == cudaSuccess && ty == cudaGraphNodeTypeKernel)
                kernels++;
        }
    }
    return new tc_graph{ctx, graph, exec, kernels};
}

int tc_graph_launch(tc_graph* g) {
    tc_ctx* ctx = g->ctx;
    if (!cuda_ok(ctx, cudaGraphLaunch(g->exec, ctx->stream), "cudaGraphLaunch")) return -1;
    ctx->launches += g->launches;
    return 0;
}

void tc_graph_free(tc_graph* g) {
    if (!g) return;
    cudaGraphExecDestroy(g->exec);
    cudaGraphDestroy(g->graph);
    delete g;
}

int tc_timer_start(tc_ctx* ctx) {
    return cuda_ok(ctx, cudaEventRecord(ctx->ev_start, ctx->stream), "cudaEventRecord") ? 0 : -1;
}

float tc_timer_stop_ms(tc_ctx* ctx) {
    if (!cuda_ok(ctx, cudaEventRecord(ctx->ev_stop, ctx->stream), "cudaEventRecord") ||
        !cuda_ok(ctx, cudaEventSynchronize(ctx->ev_stop), "cudaEventSynchronize"))
        return -1.0f;
    float ms = 0.0f;
    if (!cuda_ok(ctx, cudaEventElapsedTime(&ms, ctx->ev_start, ctx->ev_stop), "cudaEventElapsedTime"))
        return -1.0f;
    return ms;
}

uint64_t tc_launch_count(tc_ctx* ctx) { return ctx->launches; }

}  // extern "C"
