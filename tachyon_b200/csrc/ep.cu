// Expert parallelism over the GPUs of one node: experts are sharded by
// contiguous ranges (the remainder to the low ranks), the router is replicated,
// tokens stay data-parallel, and each MoE block exchanges rows twice with an
// all-to-all-v over NCCL (NVLink / NVSwitch): quantized token rows out to the
// ranks that own their experts, expert outputs back.
//
// Tachyon itself is single-device; this file has no counterpart there. What it
// preserves is the block's arithmetic: every (token, expert) slot is computed by
// the same kernels on the same quantized row as on one GPU, and the returning
// rows are combined by the same kernel in the same ascending-expert order, so
// the result is bit-identical to the single-GPU fast path.
//
// One block, on the context's stream:
//   1. route + dispatch over ALL experts (slots sorted by global expert, so the
//      slots bound for one rank are contiguous);
//   2. gather the slots' int8 rows and scales into send order;
//   3. all-gather the per-expert histograms, read them on the host (sizes of the
//      variable-length exchange have to be known there);
//   4. all-to-all-v of rows and scales;
//   5. merge the received runs into per-local-expert lists;
//   6. gate_up + SwiGLU, down (output rows written in receive order);
//   7. all-to-all-v back; 8. combine.
// No kernel here reads a peer's memory; NCCL moves the data.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "ep.cuh"
#include "experts_common.cuh"

namespace tc {

namespace {

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                                  cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi& nccl() {
    static NcclApi api;
    if (api.lib) return api;
    // The soname resolves to a copy already in the process (PyTorch bundles one) or the system's.
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return api;
    auto sym = [&](const char* name) { return dlsym(h, name); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(sym("ncclReduceScatter"));
    api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
    api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    if (api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.ReduceScatter && api.Send && api.Recv &&
        api.GroupStart && api.GroupEnd)
        api.lib = h;
    return api;
}

// send_xq[p] = xq[slot_token[p]], send_xs[p] = xs[slot_token[p]]: the slots' rows in
// expert-contiguous (= destination-contiguous) order.
__global__ void gather_rows_kernel(const int8_t* __restrict__ xq, const float* __restrict__ xs,
                                   const uint32_t* __restrict__ slot_token, int slots, int hidden, int nbp,
                                   int8_t* __restrict__ send_xq, float* __restrict__ send_xs) {
    const int vec = hidden / 16;
    for (int p = blockIdx.x; p < slots; p += gridDim.x) {
        const size_t row = slot_token[p];
        const uint4* src = reinterpret_cast<const uint4*>(xq + row * hidden);
        uint4* dst = reinterpret_cast<uint4*>(send_xq + size_t(p) * hidden);
        for (int i = threadIdx.x; i < vec; i += blockDim.x) dst[i] = src[i];
        for (int i = threadIdx.x; i < nbp; i += blockDim.x) send_xs[size_t(p) * nbp + i] = xs[row * nbp + i];
    }
}

// scale * sum of the 32 quants, per (row, block): what the 4-bit offsets multiply
// (src/weights.rs:491-507). Recomputed from the received rows rather than sent.
__global__ void block_sums_kernel(const int8_t* __restrict__ xq, const float* __restrict__ xs, size_t rows,
                                  int hidden, int nbp, float* __restrict__ xsum) {
    const int nb = hidden / QK, lane = threadIdx.x & 31;
    const size_t warp = size_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const size_t nwarps = size_t(gridDim.x) * (blockDim.x >> 5);
    for (size_t w = warp; w < rows * nbp; w += nwarps) {
        const size_t row = w / nbp;
        const int b = int(w - row * nbp);
        if (b >= nb) {
            if (lane == 0) xsum[w] = 0.0f;
            continue;
        }
        int q = xq[row * hidden + b * QK + lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
        if (lane == 0) xsum[w] = xs[row * nbp + b] * float(q);
    }
}

// From every rank's histogram over all experts: this rank's per-local-expert
// counts, offsets and active list, and for each expert-contiguous slot its row
// in the receive buffer (rows arrive grouped by source rank, and within a
// source by expert). One CTA.
__global__ void merge_received_kernel(const uint32_t* __restrict__ hist_all, int ranks, int experts,
                                      int first, int local, uint32_t* __restrict__ counts,
                                      uint32_t* __restrict__ offsets, int* __restrict__ active,
                                      uint32_t* __restrict__ slot_row) {
    __shared__ uint32_t s_off[MAX_EXPERTS + 1];
    __shared__ uint32_t s_recv_off[64 + 1];
    const int tid = threadIdx.x;
    if (tid == 0) {
        uint32_t run = 0;
        for (int s = 0; s < ranks; s++) {
            s_recv_off[s] = run;
            for (int e = 0; e < local; e++) run += hist_all[size_t(s) * experts + first + e];
        }
        s_recv_off[ranks] = run;
        uint32_t off = 0;
        int n = 0;
        for (int e = 0; e < local; e++) {
            uint32_t c = 0;
            for (int s = 0; s < ranks; s++) c += hist_all[size_t(s) * experts + first + e];
            counts[e] = c;
            s_off[e] = off;
            offsets[e] = off;
            off += c;
            if (c) active[n++] = e;
        }
        s_off[local] = off;
        offsets[local] = off;
        active[local] = n;
    }
    __syncthreads();
    // (expert, source) runs, one per thread at a time.
    for (int run = tid; run < local * ranks; run += blockDim.x) {
        const int e = run / ranks, s = run - e * ranks;
        uint32_t before_sources = 0;  // slots of expert e from sources < s
        for (int s2 = 0; s2 < s; s2++) before_sources += hist_all[size_t(s2) * experts + first + e];
        uint32_t before_experts = 0;  // rows of source s for local experts < e
        for (int e2 = 0; e2 < e; e2++) before_experts += hist_all[size_t(s) * experts + first + e2];
        const uint32_t n = hist_all[size_t(s) * experts + first + e];
        const uint32_t dst = s_off[e] + before_sources, src = s_recv_off[s] + before_experts;
        for (uint32_t i = 0; i < n; i++) slot_row[dst + i] = src + i;
    }
}

}  // namespace

void ep_expert_range(int experts, int rank, int size, int* first, int* count) {
    const int base = experts / size, rem = experts % size;
    *first = rank * base + (rank < rem ? rank : rem);
    *count = base + (rank < rem ? 1 : 0);
}

const char* ep_unique_id(char* out128) {
    NcclApi& n = nccl();
    if (!n.lib) return "libnccl.so.2 could not be loaded";
    ncclUniqueId id;
    if (n.GetUniqueId(&id) != ncclSuccess) return "ncclGetUniqueId failed";
    memcpy(out128, id.internal, NCCL_UNIQUE_ID_BYTES);
    return nullptr;
}

const char* ep_init(EpState& st, const char* id128, int rank, int size) {
    NcclApi& n = nccl();
    if (!n.lib) return "libnccl.so.2 could not be loaded";
    if (size < 1 || size > 64 || rank < 0 || rank >= size) return "bad rank or size";
    ncclUniqueId id;
    memcpy(id.internal, id128, NCCL_UNIQUE_ID_BYTES);
    if (n.CommInitRank(&st.comm, size, id, rank) != ncclSuccess) return "ncclCommInitRank failed";
    st.rank = rank;
    st.size = size;
    return nullptr;
}

void ep_destroy(EpState& st) {
    if (st.peer.on) {
        for (int r = 0; r < st.size; r++)
            if (r != st.rank && st.peer.base[r]) cudaIpcCloseMemHandle(st.peer.base[r]);
        cudaFree(st.peer.window);
        cudaFree(st.peer.epoch);
        st.peer = EpPeer{};
    }
    for (void* p : st.uni.allocs) cudaFree(p);
    st.uni.allocs.clear();
    if (st.comm) nccl().CommDestroy(st.comm);
    st.comm = nullptr;
    if (st.hist_host) cudaFreeHost(st.hist_host);
    st.hist_host = nullptr;
}

bool ep_layer_alloc(EpLayerBuffers& b, const EpState& st, const MoeDims& d, int max_tokens) {
    ep_expert_range(d.experts, st.rank, st.size, &b.first, &b.local);
    const size_t slots = size_t(max_tokens) * d.topk;
    b.capacity = slots * st.size;  // every rank could send everything here
    const size_t nbp_h = (d.hidden / QK + 7) / 8 * 8;
    auto get = [&](auto*& p, size_t elems) {
        void* raw = nullptr;
        if (cudaMalloc(&raw, elems * sizeof(*p) + 256) != cudaSuccess) return false;
        b.allocs.push_back(raw);
        p = static_cast<std::remove_reference_t<decltype(p)>>(raw);
        return true;
    };
    return get(b.send_xq, slots * d.hidden) && get(b.send_xs, slots * nbp_h) &&
           get(b.recv_xq, b.capacity * d.hidden) && get(b.recv_xs, b.capacity * nbp_h) &&
           get(b.recv_xsum, b.capacity * nbp_h) &&
           get(b.hist_all, size_t(st.size) * d.experts) && get(b.counts, size_t(b.local) + 1) &&
           get(b.offsets, size_t(b.local) + 2) && get(b.active, size_t(b.local) + 2) &&
           get(b.slot_row, b.capacity) && get(b.hidden_f, b.capacity * d.inter) &&
           get(b.out_recv, b.capacity * d.hidden);
}

void ep_layer_free(EpLayerBuffers& b) {
    for (void* p : b.allocs) cudaFree(p);
    b.allocs.clear();
}

// ---------------------------------------------------------------------------
// The fixed-size exchange, for decode-size blocks where every rank brings the
// same number of tokens t. Nothing is read on the host, so the block can be
// captured in a CUDA graph:
//   1. route (own tokens);
//   2. one grouped all-gather of every rank's 8-bit rows, scales and expert ids;
//   3. dispatch over all size * t tokens and all experts (the same kernels as on one
//      GPU); this rank's experts are a contiguous run of the sorted slots;
//   4. gate_up + SwiGLU and down on the local experts, each output row written at
//      its (home rank, token, pick) place in a zeroed [size * t * k, H] buffer;
//   5. reduce-scatter (sum): every row has one producer, so a home rank receives
//      x + 0 + ... + 0 = x exactly, in (token, pick) order;
//   6. the usual combine, reading the rows in place.
// The return moves size * t * k * H * 4 bytes per rank whatever the routing, which
// is why this path is limited to blocks where that is a few megabytes.
constexpr size_t UNIFORM_MAX_BYTES = size_t(64) << 20;

__global__ void iota_kernel(uint32_t* out, size_t n) {
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
        out[i] = uint32_t(i);
}

bool ep_uniform_reserve(EpState& st, const MoeDims& d, int max_tokens) {
    EpUniform& u = st.uni;
    const int G = max_tokens * st.size;
    if (G > 16384) return true;  // not for this size
    if (u.tokens >= G && u.hidden >= d.hidden && u.experts >= d.experts && u.topk >= d.topk && u.inter >= d.inter)
        return true;
    cudaDeviceSynchronize();
    for (void* p : u.allocs) cudaFree(p);
    u.allocs.clear();
    const int T = G > u.tokens ? G : u.tokens, H = d.hidden > u.hidden ? d.hidden : u.hidden,
              E = d.experts > u.experts ? d.experts : u.experts, K = d.topk > u.topk ? d.topk : u.topk,
              I = d.inter > u.inter ? d.inter : u.inter;
    const size_t nbp = (H / QK + 7) / 8 * 8, slots = size_t(T) * K;
    auto get = [&](auto*& p, size_t elems) {
        void* raw = nullptr;
        if (cudaMalloc(&raw, elems * sizeof(*p) + 256) != cudaSuccess) return false;
        u.allocs.push_back(raw);
        p = static_cast<std::remove_reference_t<decltype(p)>>(raw);
        return true;
    };
    const bool ok = get(u.xq, size_t(T) * H) && get(u.xs, size_t(T) * nbp) && get(u.xsum, size_t(T) * nbp) &&
                    get(u.ids, slots) && get(u.counts, size_t(E) + 1) && get(u.offsets, size_t(E) + 2) &&
                    get(u.perm, slots) && get(u.pos, slots) && get(u.slot_token, slots) &&
                    get(u.active, size_t(E) + 2) && get(u.block_hist, size_t((T + 255) / 256) * E) &&
                    get(u.hidden_f, slots * I) && get(u.identity, slots) &&
                    // (the reduce-scatter buffer of the exchange over NCCL; the peer windows do without it)
                    (slots * H * 4 > UNIFORM_MAX_BYTES ? (u.big = nullptr, true) : get(u.big, slots * H)) &&
                    get(u.runs.expert, size_t(E) + slots / 16 + 2) && get(u.runs.count, size_t(E) + slots / 16 + 2) &&
                    get(u.runs.offset, size_t(E) + slots / 16 + 2) && get(u.runs.n, size_t(2));
    if (!ok) {
        for (void* p : u.allocs) cudaFree(p);
        u.allocs.clear();
        u.tokens = 0;
        return false;
    }
    iota_kernel<<<64, 256>>>(u.identity, slots);
    cudaDeviceSynchronize();
    u.tokens = T, u.hidden = H, u.experts = E, u.topk = K, u.inter = I;
    return true;
}

bool ep_uniform_applies(const EpState& st, const MoeDims& d, int t) {
    const EpUniform& u = st.uni;
    return u.on && size_t(t) * st.size <= size_t(u.tokens) && d.hidden <= u.hidden && d.experts <= u.experts &&
           d.topk <= u.topk && d.inter <= u.inter;
}

const char* ep_forward_uniform(EpState& st, EpLayerBuffers& b, const MoeDims& d, const uint16_t* router,
                               const float* bias, const MatrixDev& gate_up, const uint8_t* gate_up_tiled,
                               const MatrixDev& down, const uint8_t* down_tiled, const float* x,
                               const float* norm_w, float eps, int t, float* y, Workspace& ws, int sms,
                               cudaStream_t stream, int* launches) {
    NcclApi& n = nccl();
    EpUniform& u = st.uni;
    const int R = st.size, G = R * t;
    const int nbp = (d.hidden / QK + 7) / 8 * 8;
    *launches += launch_route(d, router, bias, x, norm_w, eps, t, ws, stream);
    n.GroupStart();
    n.AllGather(ws.xq, u.xq, size_t(t) * d.hidden, ncclInt8, st.comm, stream);
    n.AllGather(ws.xs, u.xs, size_t(t) * nbp, ncclFloat32, st.comm, stream);
    n.AllGather(ws.ids, u.ids, size_t(t) * d.topk, ncclUint32, st.comm, stream);
    if (n.GroupEnd() != ncclSuccess) return "all-gather of the token rows failed";

    Workspace gw = ws;  // the view over every rank's tokens
    gw.ids = u.ids;
    gw.xq = u.xq;
    gw.xs = u.xs;
    gw.xsum = u.xsum;
    gw.counts = u.counts;
    gw.offsets = u.offsets;
    gw.perm = u.perm;
    gw.pos = u.pos;
    gw.slot_token = u.slot_token;
    gw.active = u.active;
    gw.block_hist = u.block_hist;
    *launches += launch_dispatch(d, G, gw, stream);
    if (gate_up.kind == 2) {
        const size_t want_blocks = (size_t(G) * nbp + 7) / 8;
        block_sums_kernel<<<unsigned(want_blocks < 148 * 16 ? want_blocks : 148 * 16), 256, 0, stream>>>(
            u.xq, u.xs, size_t(G), d.hidden, nbp, u.xsum);
        *launches += 1;
    }
    cudaMemsetAsync(u.big, 0, size_t(G) * d.topk * d.hidden * sizeof(float), stream);

    MoeDims ld = d;
    ld.experts = b.local;
    Workspace lw = gw;  // this rank's experts: a contiguous run of the sorted slots
    lw.counts = u.counts + b.first;
    lw.offsets = u.offsets + b.first;
    lw.active = nullptr;
    lw.runs = u.runs;  // experts here see several 16-token segments each: spread them over the CTAs
    *launches += launch_build_runs(lw.counts, lw.offsets, b.local, u.runs, stream);
    lw.hidden_f = u.hidden_f;
    lw.out = u.big;
    *launches += launch_gate_up_fast(ld, gate_up, gate_up_tiled, G, lw, sms, stream);
    *launches += launch_down_fast_rows(ld, down, down_tiled, lw, u.perm, sms, stream);

    if (n.ReduceScatter(u.big, ws.out, size_t(t) * d.topk * d.hidden, ncclFloat32, ncclSum, st.comm, stream) !=
        ncclSuccess)
        return "reduce-scatter of the expert outputs failed";
    Workspace cw = ws;
    cw.pos = u.identity;  // rows arrive in (token, pick) order
    *launches += launch_combine(d, t, cw, y, stream);
    return nullptr;
}

// ---------------------------------------------------------------------------
// The exchange over peer memory. Same plan as the fixed-size exchange, with the
// two collectives replaced by stores into the destination rank's window:
//   1. route (own tokens);
//   2. this rank's 8-bit rows, scales and expert ids into every rank's window (NVLink
//      stores), then a release-store of this rank's block counter into every rank's flag
//      word: by the router kernel's last CTA up to 256 tokens, else by
//      peer_scatter_rows_kernel + peer_rows_sent_kernel;
//   3. the dispatch kernel waits (bounded) until all ranks' rows have arrived here;
//   4. dispatch over all ranks' tokens, gate_up + SwiGLU, down on this rank's experts;
//      the down kernel stores each output row into its home rank's window at
//      (token, pick) and announces it (its last CTA, or peer_announce_kernel after the
//      tcgen05 kernels);
//   5. the combine kernel waits for every rank's announcement and reads the rows in place.
// Every wait is bounded (peer_wait) and leaves an error status instead of hanging.
// Ordering across blocks needs no second buffer: a rank can only reach step 2 of block
// n+1 after its combine of block n, which waited for every rank's step 5 of block n,
// i.e. for every reader of the rows of block n.
// Step 2 for batches of more than 256 tokens: every CTA copies a share of this rank's rows, scales
// and ids into every window; peer_rows_sent_kernel, next in the stream, announces them.
__global__ void __launch_bounds__(256) peer_scatter_rows_kernel(const PeerPlan a) {
    const size_t xq_vec = size_t(a.t) * a.hidden / 16, xs_vec = size_t(a.t) * a.nbp / 4;
    const size_t ids_n = size_t(a.t) * a.topk;
    const size_t tid = size_t(blockIdx.x) * blockDim.x + threadIdx.x, n = size_t(gridDim.x) * blockDim.x;
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
}

__global__ void peer_rows_sent_kernel(const PeerPlan a) {
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t e = a.epoch[a.flag_set] + 1;
        a.epoch[a.flag_set] = e;
        for (int r = 0; r < a.ranks && !a.mute; r++) {
            uint32_t* flag = reinterpret_cast<uint32_t*>(a.base[r] + a.off_flags) + a.flag_set * 8 + a.me;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(e) : "memory");
        }
    }
}

// The signal alone (t = 0 rows): after the down kernel, whose stores into the other
// ranks' windows are complete when this kernel starts.
__global__ void peer_wait_kernel(const PeerWait pw) {
    if (int(threadIdx.x) < pw.ranks) peer_wait(pw, threadIdx.x);
    __syncwarp();
}

struct PeerFlags {
    uint32_t* p[8];
};

// After a kernel that stored expert outputs into the other ranks' windows (complete when this
// one starts): this rank's next counter value, release-stored into every rank's flag.
__global__ void peer_announce_kernel(uint32_t* epoch, PeerFlags flags, int ranks) {
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t e = *epoch + 1;
        *epoch = e;
        for (int r = 0; r < ranks; r++)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[r]), "r"(e) : "memory");
    }
}

const char* ep_barrier(EpState& st, cudaStream_t stream) {
    NcclApi& n = nccl();
    if (!st.comm) return "no communicator";
    uint32_t* buf = nullptr;
    if (cudaMalloc(reinterpret_cast<void**>(&buf), size_t(st.size + 1) * 4) != cudaSuccess) return "cudaMalloc failed";
    const bool ok = n.AllGather(buf + st.size, buf, 1, ncclUint32, st.comm, stream) == ncclSuccess &&
                    cudaStreamSynchronize(stream) == cudaSuccess;
    cudaFree(buf);
    return ok ? nullptr : "barrier all-gather failed";
}

const char* ep_peer_enable(EpState& st, int hidden, int topk, int max_tokens) {
    NcclApi& n = nccl();
    EpPeer& p = st.peer;
    if (!st.comm) return "call tc_ep_init first";
    if (st.size > 8) return "the peer-memory exchange is for up to 8 ranks";
    if (p.on) return "already enabled";
    const size_t G = size_t(max_tokens) * st.size, nbp = (hidden / QK + 7) / 8 * 8;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    size_t o = 0;
    p.off_xq = o, o = up(o + G * hidden);
    p.off_xs = o, o = up(o + G * nbp * 4);
    p.off_xsum = o, o = up(o + G * nbp * 4);
    p.off_ids = o, o = up(o + G * topk * 4);
    p.off_out = o, o = up(o + size_t(max_tokens) * topk * hidden * 4);
    p.off_flags = o, o = up(o + 3 * 8 * 4);  // two sets of per-rank flags, then the one-kernel path's counters
    p.bytes = o;
    if (cudaMalloc(reinterpret_cast<void**>(&p.window), p.bytes) != cudaSuccess) return "cudaMalloc(window) failed";
    cudaMemset(p.window, 0, p.bytes);
    if (cudaMalloc(reinterpret_cast<void**>(&p.epoch), 32) != cudaSuccess) return "cudaMalloc failed";
    cudaMemset(p.epoch, 0, 32);
    cudaIpcMemHandle_t mine;
    if (cudaIpcGetMemHandle(&mine, p.window) != cudaSuccess) return "cudaIpcGetMemHandle failed";
    // Every rank's handle, through the communicator that already exists.
    const size_t hb = sizeof(cudaIpcMemHandle_t);
    uint8_t* dev = nullptr;
    if (cudaMalloc(reinterpret_cast<void**>(&dev), hb * (st.size + 1)) != cudaSuccess) return "cudaMalloc failed";
    cudaMemcpy(dev + hb * st.size, &mine, hb, cudaMemcpyHostToDevice);
    std::vector<cudaIpcMemHandle_t> all(st.size);
    const bool ok = n.AllGather(dev + hb * st.size, dev, hb, ncclInt8, st.comm, nullptr) == ncclSuccess &&
                    cudaStreamSynchronize(nullptr) == cudaSuccess &&
                    cudaMemcpy(all.data(), dev, hb * st.size, cudaMemcpyDeviceToHost) == cudaSuccess;
    cudaFree(dev);
    if (!ok) return "exchange of the window handles failed";
    for (int r = 0; r < st.size; r++) {
        if (r == st.rank) {
            p.base[r] = p.window;
            continue;
        }
        void* ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
            return "cudaIpcOpenMemHandle failed (are the ranks' GPUs peers?)";
        p.base[r] = static_cast<uint8_t*>(ptr);
    }
    p.tokens = max_tokens, p.hidden = hidden, p.topk = topk;
    p.on = true;
    st.uni.on = true;  // the dispatch over all ranks' tokens uses the same buffers
    // Nobody stores into a window before every rank has mapped and cleared its own.
    return ep_barrier(st, nullptr);
}

bool ep_peer_applies(const EpState& st, const MoeDims& d, int t) {
    const EpPeer& p = st.peer;
    return p.on && t <= p.tokens && d.hidden == p.hidden && d.topk == p.topk && ep_uniform_applies(st, d, t);
}

const char* ep_forward_peer(EpState& st, EpLayerBuffers& b, const MoeDims& d, const uint16_t* router,
                            const float* bias, const MatrixDev& gate_up, const uint8_t* gate_up_tiled,
                            const MatrixDev& down, const uint8_t* down_tiled, const float* x,
                            const float* norm_w, float eps, int t, float* y, Workspace& ws, int sms,
                            cudaStream_t stream, int* launches, bool one_kernel, unsigned long long* stamps,
                            const PrefillWeights* pw, const PrefillScratch* ps, int prefill_min_avg) {
    EpUniform& u = st.uni;
    EpPeer& p = st.peer;
    const int R = st.size, G = R * t;
    const int nbp = (d.hidden / QK + 7) / 8 * 8;
    if (one_kernel && decode_block_applies(d, gate_up.kind, down.kind, t, R)) {
        // Decode-size batch: the whole block, both exchanges included, is one kernel per rank.
        DecodeEp e;
        e.ranks = R, e.me = st.rank, e.first = b.first, e.local = b.local;
        for (int r = 0; r < R; r++) e.base[r] = p.base[r];
        e.off_xq = p.off_xq, e.off_xs = p.off_xs, e.off_xsum = p.off_xsum, e.off_ids = p.off_ids;
        e.off_out = p.off_out, e.off_flags = p.off_flags;
        e.epoch = p.epoch + 4;
        if (p.mute_next > 0) {
            e.mute = 1;
            p.mute_next--;
        }
        const int n = launch_decode_block(d, gate_up.kind, router, bias, x, norm_w, eps, t, y, gate_up_tiled, down_tiled,
                                          ws, sms, p.wait_limit, stamps, stream, &e, u.hidden_f);
        if (n < 0) return "the one-kernel block does not fit this shape";
        *launches += n;
        return nullptr;
    }
    PeerPlan plan{};
    for (int r = 0; r < R; r++) plan.base[r] = p.base[r];
    plan.off_xq = p.off_xq, plan.off_xs = p.off_xs, plan.off_ids = p.off_ids, plan.off_flags = p.off_flags;
    plan.xq = ws.xq, plan.xs = ws.xs, plan.ids = ws.ids;
    plan.t = t, plan.hidden = d.hidden, plan.nbp = nbp, plan.topk = d.topk, plan.me = st.rank, plan.ranks = R;
    plan.flag_set = 0;
    plan.epoch = p.epoch;
    if (p.mute_next > 0) {
        plan.mute = 1;
        p.mute_next--;
    }
    Workspace rw = ws;
    rw.route_scatter = plan;  // batches of up to one CTA's worth of tokens: sent by the router's last CTA
    *launches += launch_route(d, router, bias, x, norm_w, eps, t, rw, stream);
    if (t > 256) {  // larger ones: sent by kernels of their own (many CTAs copy, one thread announces)
        peer_scatter_rows_kernel<<<2 * sms, 256, 0, stream>>>(plan);
        peer_rows_sent_kernel<<<1, 32, 0, stream>>>(plan);
        *launches += 2;
    }

    Workspace gw = ws;  // the view over every rank's tokens, gathered in this rank's window
    gw.ids = reinterpret_cast<uint32_t*>(p.window + p.off_ids);
    gw.xq = reinterpret_cast<int8_t*>(p.window + p.off_xq);
    gw.xs = reinterpret_cast<float*>(p.window + p.off_xs);
    gw.xsum = u.xsum;
    gw.counts = u.counts;
    gw.offsets = u.offsets;
    gw.perm = u.perm;
    gw.pos = u.pos;
    gw.slot_token = u.slot_token;
    gw.active = u.active;
    gw.block_hist = u.block_hist;
    gw.dispatch_wait.flags = reinterpret_cast<const uint32_t*>(p.window + p.off_flags);
    gw.dispatch_wait.epoch = p.epoch;
    gw.dispatch_wait.ranks = R;
    gw.dispatch_wait.status = ws.status;
    gw.dispatch_wait.limit = p.wait_limit;
    *launches += launch_dispatch(d, G, gw, stream);
    if (gate_up.kind == 2) {
        const size_t want_blocks = (size_t(G) * nbp + 7) / 8;
        block_sums_kernel<<<unsigned(want_blocks < 148 * 16 ? want_blocks : 148 * 16), 256, 0, stream>>>(
            gw.xq, gw.xs, size_t(G), d.hidden, nbp, u.xsum);
        *launches += 1;
    }
    MoeDims ld = d;
    ld.experts = b.local;
    Workspace lw = gw;
    lw.counts = u.counts + b.first;
    lw.offsets = u.offsets + b.first;
    lw.active = nullptr;
    lw.runs = u.runs;  // experts here see several 16-token segments each: spread them over the CTAs
    *launches += launch_build_runs(lw.counts, lw.offsets, b.local, u.runs, stream);
    lw.hidden_f = u.hidden_f;
    lw.out = nullptr;
    float* outs[8] = {};
    for (int r = 0; r < R; r++) outs[r] = reinterpret_cast<float*>(p.base[r] + p.off_out);
    uint32_t* flags2[8] = {};
    for (int r = 0; r < R; r++) flags2[r] = reinterpret_cast<uint32_t*>(p.base[r] + p.off_flags) + 8 + st.rank;
    if (pw && ps && pw->gu_t && (long long)G * d.topk >= (long long)prefill_min_avg * d.experts) {
        // Prefill-size groups: the tcgen05 kernels on this rank's tiles. How many slots this rank
        // gets is only known on the device, so the grids are sized for all of them; the down
        // kernel's epilogue stores each row into its home rank's window, then one thread announces.
        const int slots = G * d.topk;
        *launches += launch_prefill(ld, true, gate_up.kind == 2, *pw, *ps, lw, slots, u.hidden_f, nullptr, stream);
        *launches += launch_prefill(ld, false, down.kind == 2, *pw, *ps, lw, slots, nullptr, u.perm, stream, outs, R,
                                    uint32_t(t) * d.topk);
        PeerFlags pf{};
        for (int r = 0; r < R; r++) pf.p[r] = flags2[r];
        peer_announce_kernel<<<1, 32, 0, stream>>>(p.epoch + 1, pf, R);
        *launches += 1;
    } else {
        *launches += launch_gate_up_fast(ld, gate_up, gate_up_tiled, G, lw, sms, stream);
        *launches += launch_down_fast_rows(ld, down, down_tiled, lw, u.perm, sms, stream, outs, R,
                                           uint32_t(t) * d.topk, flags2, p.epoch + 1, p.epoch + 2);
    }

    Workspace cw = ws;
    cw.out = reinterpret_cast<float*>(p.window + p.off_out);
    cw.pos = u.identity;
    cw.combine_wait.flags = reinterpret_cast<const uint32_t*>(p.window + p.off_flags) + 8;
    cw.combine_wait.epoch = p.epoch + 1;
    cw.combine_wait.ranks = R;
    cw.combine_wait.status = ws.status;
    cw.combine_wait.limit = p.wait_limit;
    *launches += launch_combine(d, t, cw, y, stream);
    return nullptr;
}

// The block over expert-parallel ranks. `gate_up_tiled` / `down_tiled` hold this
// rank's experts only; `local_dims` is the shape with experts = b.local.
const char* ep_forward(EpState& st, EpLayerBuffers& b, const MoeDims& d, const uint16_t* router,
                       const float* bias, const MatrixDev& gate_up, const uint8_t* gate_up_tiled,
                       const MatrixDev& down, const uint8_t* down_tiled, const float* x,
                       const float* norm_w, float eps, int t, float* y, Workspace& ws, int sms,
                       cudaStream_t stream, int* launches, const PrefillWeights* pw,
                       const PrefillScratch* ps, int prefill_min_avg) {
    NcclApi& n = nccl();
    const int R = st.size;
    const int nbp = (d.hidden / QK + 7) / 8 * 8;
    const int slots = t * d.topk;
    *launches += launch_route(d, router, bias, x, norm_w, eps, t, ws, stream);
    gather_rows_kernel<<<min(slots, 148 * 8), 128, 0, stream>>>(ws.xq, ws.xs, ws.slot_token, slots, d.hidden,
                                                               nbp, b.send_xq, b.send_xs);
    *launches += 1;
    // Histograms of every rank, and a copy on the host for the exchange sizes.
    if (st.hist_host_elems < size_t(R) * d.experts) {
        if (st.hist_host) cudaFreeHost(st.hist_host);
        if (cudaHostAlloc(reinterpret_cast<void**>(&st.hist_host), size_t(R) * d.experts * 4, cudaHostAllocDefault) !=
            cudaSuccess)
            return "cudaHostAlloc failed";
        st.hist_host_elems = size_t(R) * d.experts;
    }
    if (n.AllGather(ws.counts, b.hist_all, d.experts, ncclUint32, st.comm, stream) != ncclSuccess)
        return "ncclAllGather failed";
    cudaMemcpyAsync(st.hist_host, b.hist_all, size_t(R) * d.experts * 4, cudaMemcpyDeviceToHost, stream);
    if (cudaStreamSynchronize(stream) != cudaSuccess) return "stream sync failed";

    std::vector<size_t> send_off(R + 1, 0), recv_off(R + 1, 0);
    for (int r = 0; r < R; r++) {
        int first, cnt;
        ep_expert_range(d.experts, r, R, &first, &cnt);
        size_t s = 0;
        for (int e = 0; e < cnt; e++) s += st.hist_host[size_t(st.rank) * d.experts + first + e];
        send_off[r + 1] = send_off[r] + s;
        size_t rc = 0;
        for (int e = 0; e < b.local; e++) rc += st.hist_host[size_t(r) * d.experts + b.first + e];
        recv_off[r + 1] = recv_off[r] + rc;
    }
    const size_t received = recv_off[R];
    if (received > b.capacity) return "more rows received than the layer was sized for";

    // Rows and scales out.
    n.GroupStart();
    for (int r = 0; r < R; r++) {
        const size_t sc = send_off[r + 1] - send_off[r], rc = recv_off[r + 1] - recv_off[r];
        if (sc) {
            n.Send(b.send_xq + send_off[r] * d.hidden, sc * d.hidden, ncclInt8, r, st.comm, stream);
            n.Send(b.send_xs + send_off[r] * nbp, sc * nbp, ncclFloat32, r, st.comm, stream);
        }
        if (rc) {
            n.Recv(b.recv_xq + recv_off[r] * d.hidden, rc * d.hidden, ncclInt8, r, st.comm, stream);
            n.Recv(b.recv_xs + recv_off[r] * nbp, rc * nbp, ncclFloat32, r, st.comm, stream);
        }
    }
    if (n.GroupEnd() != ncclSuccess) return "dispatch all-to-all failed";

    merge_received_kernel<<<1, 256, 0, stream>>>(b.hist_all, R, d.experts, b.first, b.local, b.counts,
                                                 b.offsets, b.active, b.slot_row);
    *launches += 1;
    if (received) {
        MoeDims ld = d;
        ld.experts = b.local;
        Workspace lw = ws;  // the local-expert view: received rows, merged lists
        lw.counts = b.counts;
        lw.offsets = b.offsets;
        lw.active = b.active;
        lw.slot_token = b.slot_row;
        lw.xq = b.recv_xq;
        lw.xs = b.recv_xs;
        if (gate_up.kind == 2) {
            const size_t warps = received * nbp;
            const size_t want_blocks = (warps + 7) / 8;
            block_sums_kernel<<<unsigned(want_blocks < 148 * 16 ? want_blocks : 148 * 16), 256, 0, stream>>>(
                b.recv_xq, b.recv_xs, received, d.hidden, nbp, b.recv_xsum);
            *launches += 1;
            lw.xsum = b.recv_xsum;
        }
        lw.hidden_f = b.hidden_f;
        lw.out = b.out_recv;
        if (pw && ps && pw->gu_t && received >= size_t(prefill_min_avg) * size_t(b.local)) {
            // Prefill-size groups: the tcgen05 kernels, on this rank's tiles.
            *launches += launch_prefill(ld, true, gate_up.kind == 2, *pw, *ps, lw, int(received), b.hidden_f, nullptr,
                                        stream);
            *launches += launch_prefill(ld, false, down.kind == 2, *pw, *ps, lw, int(received), b.out_recv,
                                        b.slot_row, stream);
        } else {
            *launches += launch_gate_up_fast(ld, gate_up, gate_up_tiled, t, lw, sms, stream);
            *launches += launch_down_fast_rows(ld, down, down_tiled, lw, b.slot_row, sms, stream);
        }
    }

    // Outputs back to the ranks the slots came from, into their expert-contiguous order.
    n.GroupStart();
    for (int r = 0; r < R; r++) {
        const size_t sc = send_off[r + 1] - send_off[r], rc = recv_off[r + 1] - recv_off[r];
        if (rc) n.Send(b.out_recv + recv_off[r] * d.hidden, rc * d.hidden, ncclFloat32, r, st.comm, stream);
        if (sc) n.Recv(ws.out + send_off[r] * d.hidden, sc * d.hidden, ncclFloat32, r, st.comm, stream);
    }
    if (n.GroupEnd() != ncclSuccess) return "combine all-to-all failed";
    *launches += launch_combine(d, t, ws, y, stream);
    return nullptr;
}

}  // namespace tc

