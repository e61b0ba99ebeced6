// Expert parallelism: state and entry points shared by ep.cu and the C ABI.
#pragma once

#include <vector>

#include "common.cuh"

struct ncclComm;

namespace tc {

struct EpState {
    ncclComm* comm = nullptr;
    int rank = 0, size = 1;
    uint32_t* hist_host = nullptr;  // pinned [size * experts]
    size_t hist_host_elems = 0;
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
const char* ep_forward(EpState& st, EpLayerBuffers& b, const MoeDims& d, const uint16_t* router,
                       const float* bias, const MatrixDev& gate_up, const uint8_t* gate_up_tiled,
                       const MatrixDev& down, const uint8_t* down_tiled, const float* x,
                       const float* norm_w, float eps, int t, float* y, Workspace& ws, int sms,
                       cudaStream_t stream, int* launches);

}  // namespace tc
