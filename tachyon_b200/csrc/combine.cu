// Weighted combine / unpermute, fused with the residual add.
//
// The CPU path walks experts in ascending index and, for each token routed to
// the expert, does proj[token] += gate * expert_out (src/model.rs:484,
// 513-519; axpy rounds the product before the add, src/kernels.rs:606-610),
// starting from zeros; its caller then adds proj to the residual stream
// (src/model.rs:681). So a token's k contributions are summed in ascending
// expert order, not in the router's score order: each CTA ranks its token's
// picks by expert index and adds them in that order.
#include "common.cuh"

namespace tc {

namespace {

constexpr int COMBINE_THREADS = 256;

__global__ void __launch_bounds__(COMBINE_THREADS)
combine_kernel(const uint32_t* __restrict__ ids, const float* __restrict__ gates,
               const uint32_t* __restrict__ pos, const float* out, int hidden, int topk,
               float* y, const PeerWait pw) {
    // (`out` without __restrict__: in the peer-memory exchange other GPUs store these rows
    // while this kernel is already resident, up to the wait below.)
    __shared__ uint32_t s_pos[MAX_TOPK];
    __shared__ float s_gate[MAX_TOPK];
    const int token = blockIdx.x, tid = threadIdx.x;
    grid_launch_dependents();
    grid_dependency_wait();
    if (pw.flags) {  // expert outputs arrive from other ranks: all of them have signalled this block
        if (tid < pw.ranks) peer_wait(pw, tid);
        __syncthreads();
    }
    if (tid < topk) {
        const uint32_t mine = ids[size_t(token) * topk + tid];
        int rank = 0;
        for (int j = 0; j < topk; j++) rank += ids[size_t(token) * topk + j] < mine ? 1 : 0;
        s_pos[rank] = pos[size_t(token) * topk + tid];
        s_gate[rank] = gates[size_t(token) * topk + tid];
    }
    __syncthreads();
    float* yr = y + size_t(token) * hidden;
    for (int c = tid * 4; c < hidden; c += COMBINE_THREADS * 4) {
        float4 proj = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
        for (int j = 0; j < topk; j++) {
            const float g = s_gate[j];
            const float4 v = *reinterpret_cast<const float4*>(out + size_t(s_pos[j]) * hidden + c);
            proj.x = proj.x + g * v.x;
            proj.y = proj.y + g * v.y;
            proj.z = proj.z + g * v.z;
            proj.w = proj.w + g * v.w;
        }
        float4 r = *reinterpret_cast<float4*>(yr + c);
        r.x = r.x + proj.x;
        r.y = r.y + proj.y;
        r.z = r.z + proj.z;
        r.w = r.w + proj.w;
        *reinterpret_cast<float4*>(yr + c) = r;
    }
}

}  // namespace

int launch_combine(const MoeDims& d, int t, Workspace& ws, float* y, cudaStream_t stream) {
    launch_overlapped(combine_kernel, dim3(t), dim3(COMBINE_THREADS), size_t(0), stream,
                      static_cast<const uint32_t*>(ws.ids), static_cast<const float*>(ws.gates),
                      static_cast<const uint32_t*>(ws.pos), static_cast<const float*>(ws.out), d.hidden, d.topk, y,
                      ws.combine_wait);
    return 1;
}

}  // namespace tc

