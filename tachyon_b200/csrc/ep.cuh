// Expert parallelism: state and entry points shared by ep.cu and the C ABI.
#pragma once

#include <vector>

#include "common.cuh"

struct ncclComm;

namespace tc {

// Buffers of the fixed-size exchange (every rank brings the same number of tokens):
// all ranks' rows gathered here, their dispatch, and the slot-ordered output
// buffer that the reduce-scatter returns to the tokens' home ranks. Shared by the
// context's layers.
struct EpUniform {
    bool on = false;
    int tokens = 0, hidden = 0, experts = 0, topk = 0, inter = 0;  // sized for (tokens = size * per-rank)
    int8_t* xq = nullptr;                  // [G, H]
    float *xs = nullptr, *xsum = nullptr;  // [G, pad8(H/32)]
    uint32_t* ids = nullptr;               // [G, k]
    uint32_t *counts = nullptr, *offsets = nullptr, *perm = nullptr, *pos = nullptr, *slot_token = nullptr;
    int* active = nullptr;
    uint32_t* block_hist = nullptr;
    float *hidden_f = nullptr, *big = nullptr;  // [G*k, I]; [G*k, H]
    uint32_t* identity = nullptr;               // [T*k] = 0, 1, 2, ...
    RunList runs;                               // this rank's slots in runs of up to 16 per expert
    std::vector<void*> allocs;
};

// Expert parallelism over peer memory (one NVSwitch node, up to 8 ranks): each rank
// owns a window that the others map through CUDA IPC. Rows and expert outputs
// are stored straight into the destination rank's window over NVLink and
// announced with flags; no collective library call is made inside a block.
struct EpPeer {
    bool on = false;
    int tokens = 0, hidden = 0, topk = 0;      // per-rank token capacity and row shape
    uint8_t* window = nullptr;                 // this rank's
    uint8_t* base[8] = {};                     // every rank's window as mapped here (base[rank] == window)
    size_t off_xq = 0, off_xs = 0, off_xsum = 0, off_ids = 0, off_out = 0, off_flags = 0, bytes = 0;
    uint32_t wait_limit = 1u << 23;            // polls a kernel spends on another rank's flag before giving up
    int mute_next = 0;                         // testing: this many coming blocks send rows without announcing them
    uint32_t* epoch = nullptr;                 // [0], [1]: this rank's signal counters (rows sent, outputs
                                               // sent); [2]: arrival counter of the down kernel's CTAs;
                                               // [4]: blocks completed by the one-kernel path
};

struct EpState {
    ncclComm* comm = nullptr;
    int rank = 0, size = 1;
    uint32_t* hist_host = nullptr;  // pinned [size * experts]
    size_t hist_host_elems = 0;
    EpUniform uni;
    EpPeer peer;
};

struct EpLayerBuffers {
    int first = 0, local = 0;        // this rank's expert range
    size_t capacity = 0;             // rows the receive side can hold
    int8_t *send_xq = nullptr, *recv_xq = nullptr;
    float *send_xs = nullptr, *recv_xs = nullptr, *recv_xsum = nullptr;
    uint32_t* hist_all = nullptr;    // [size, experts]
    uint32_t *counts = nullptr, *offsets = nullptr, *slot_row = nullptr;
    int* active = nullptr;
    float *hidden_f = nullptr, *out_recv = nullptr;
    std::vector<void*> allocs;
};

// Contiguous expert ranges, the remainder to the low ranks.
void ep_expert_range(int experts, int rank, int size, int* first, int* count);
const char* ep_unique_id(char* out128);
const char* ep_init(EpState& st, const char* id128, int rank, int size);
void ep_destroy(EpState& st);
bool ep_layer_alloc(EpLayerBuffers& b, const EpState& st, const MoeDims& d, int max_tokens);
void ep_layer_free(EpLayerBuffers& b);
// Sizes the fixed-size exchange for blocks of up to max_tokens tokens per rank.
bool ep_uniform_reserve(EpState& st, const MoeDims& d, int max_tokens);
// True if a block of t tokens per rank goes through the fixed-size exchange.
bool ep_uniform_applies(const EpState& st, const MoeDims& d, int t);
const char* ep_forward_uniform(EpState& st, EpLayerBuffers& b, const MoeDims& d, const uint16_t* router,
                               const float* bias, const MatrixDev& gate_up, const uint8_t* gate_up_tiled,
                               const MatrixDev& down, const uint8_t* down_tiled, const float* x,
                               const float* norm_w, float eps, int t, float* y, Workspace& ws, int sms,
                               cudaStream_t stream, int* launches);
// Collective: allocates this rank's window and maps every other rank's.
const char* ep_peer_enable(EpState& st, int hidden, int topk, int max_tokens);
bool ep_peer_applies(const EpState& st, const MoeDims& d, int t);
const char* ep_forward_peer(EpState& st, EpLayerBuffers& b, const MoeDims& d, const uint16_t* router,
                            const float* bias, const MatrixDev& gate_up, const uint8_t* gate_up_tiled,
                            const MatrixDev& down, const uint8_t* down_tiled, const float* x,
                            const float* norm_w, float eps, int t, float* y, Workspace& ws, int sms,
                            cudaStream_t stream, int* launches, bool one_kernel = false,
                            unsigned long long* stamps = nullptr, const PrefillWeights* pw = nullptr,
                            const PrefillScratch* ps = nullptr, int prefill_min_avg = 32);
const char* ep_barrier(EpState& st, cudaStream_t stream);
const char* ep_forward(EpState& st, EpLayerBuffers& b, const MoeDims& d, const uint16_t* router,
                       const float* bias, const MatrixDev& gate_up, const uint8_t* gate_up_tiled,
                       const MatrixDev& down, const uint8_t* down_tiled, const float* x,
                       const float* norm_w, float eps, int t, float* y, Workspace& ws, int sms,
                       cudaStream_t stream, int* launches, const PrefillWeights* pw = nullptr,
                       const PrefillScratch* ps = nullptr, int prefill_min_avg = 32);

}  // namespace tc
