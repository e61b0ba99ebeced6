// Device helpers shared by the expert kernels: the argument block, mbarrier and
// bulk-copy wrappers (every wait bounded), and the small arithmetic pieces that
// restate src/kernels.rs.
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"

namespace tc {

constexpr uint32_t SPIN_LIMIT = 1u << 20;
constexpr int MAX_PEERS = 8;  // ranks of a peer-memory exchange (one NVSwitch node)
constexpr int MAGIC_I = 0x4B400000;  // bits of 12582912.0f = 1.5 * 2^23
constexpr float MAGIC_F = 12582912.0f;

struct ExpertArgs {
    const uint8_t* wdata;     // int8 rows or packed nibbles
    const void* wscales;      // f16 per block, or packed 4-bit words
    int cols;                 // K
    int rows_per_expert;      // 2*inter (gate_up) or hidden (down)
    int experts, topk;
    int units_per_expert;
    const uint32_t* counts;
    const uint32_t* offsets;
    const uint32_t* slot_token;  // gate_up: sorted slot -> token (null for down: rows are slots)
    const int* active;        // experts with tokens, ascending; active[experts] = their number
    RunList runs;             // when runs.expert is set, walked instead of the three lists above
    const int8_t* xq;         // activations [rows, cols]
    const float* xs;          // scales [rows, pad8(cols/32)]
    const float* xsum;        // [rows, pad8(cols/32)] (4-bit offsets)
    const float* xf;          // when set: f32 activation rows [rows, cols] to quantize while staging
    float* out;               // gate_up: hidden_f [slots, inter]; down: out [slots, hidden]
    int out_cols;
    const uint32_t* out_rows;  // when set: output row of sorted slot p (expert parallel: its row in the receive order)
    // Expert parallelism over peer memory: when peer_out[0] is set, output row p (after
    // out_rows) belongs to rank p / peer_rows and is stored into that rank's buffer.
    float* peer_out[MAX_PEERS];
    uint32_t peer_rows;
    // ... and the last CTA to finish announces this rank's outputs: *peer_epoch + 1 into
    // peer_flag[r] (this rank's flag word in rank r's window) for every rank.
    uint32_t* peer_flag[MAX_PEERS];
    uint32_t* peer_epoch;
    uint32_t* peer_ticket;
    int peer_ranks;
    int* status;
};

inline ExpertArgs gate_up_args(const MoeDims& d, const MatrixDev& m, const Workspace& ws) {
    ExpertArgs a{};
    a.wdata = static_cast<const uint8_t*>(m.data);
    a.wscales = m.scales;
    a.cols = d.hidden;
    a.rows_per_expert = 2 * d.inter;
    a.experts = d.experts;
    a.topk = d.topk;
    a.units_per_expert = (d.inter + 7) / 8;  // 8 gate rows + the 8 matching up rows
    a.counts = ws.counts;
    a.offsets = ws.offsets;
    a.slot_token = ws.slot_token;
    a.active = ws.active;
    a.runs = ws.runs;
    a.xq = ws.xq;
    a.xs = ws.xs;
    a.xsum = ws.xsum;
    a.out = ws.hidden_f;
    a.out_cols = d.inter;
    a.status = ws.status;
    return a;
}

inline ExpertArgs down_args(const MoeDims& d, const MatrixDev& m, const Workspace& ws) {
    ExpertArgs a{};
    a.wdata = static_cast<const uint8_t*>(m.data);
    a.wscales = m.scales;
    a.cols = d.inter;
    a.rows_per_expert = d.hidden;
    a.experts = d.experts;
    a.topk = d.topk;
    a.units_per_expert = (d.hidden + 15) / 16;
    a.counts = ws.counts;
    a.offsets = ws.offsets;
    a.slot_token = nullptr;
    a.active = ws.active;
    a.runs = ws.runs;
    a.xq = ws.hq;
    a.xs = ws.hs;
    a.xsum = ws.hsum;
    a.out = ws.out;
    a.out_cols = d.hidden;
    a.status = ws.status;
    return a;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return uint32_t(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    // The last operand is a suspend-time hint in nanoseconds: the thread may
    // sleep in hardware until the phase completes or that much time passes.
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity), "r"(4000u)
        : "memory");
    return ok != 0;
}

// Waits for a stage with a spin limit. Returns false if the limit ran out
// (2^20 probes of up to 4 us each, with a short sleep between them so that
// waiting warps leave the issue slots to the ones that have data).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(100);
    }
    return false;
}

// The same for waits on a kernel's critical path: plain probes a few tens of nanoseconds
// apart. (A suspended try_wait was seen to return microseconds after the phase had
// completed.) Bounded: about a second of probing.
__device__ __forceinline__ bool mbar_wait_poll(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < (SPIN_LIMIT << 4); i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_addr(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        __nanosleep(20);
    }
    return false;
}

__device__ __forceinline__ void bulk_copy(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                          uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_addr(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}

// The same for data that is read once (the weight stream): the lines are marked to be
// evicted first from L2, so that they do not push out what is read again and again
// between them (the activations, the routing, the kernel's own instructions).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_copy_once(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar,
                                               uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_addr(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
        : "memory");
}

// Exact int -> float for |v| < 2^22: the dp4a accumulates onto the bit pattern
// of 1.5*2^23, whose float value is then 1.5*2^23 + v.
__device__ __forceinline__ float lane_sum(int w, int x) {
    return __int_as_float(__dp4a(w, x, MAGIC_I)) - MAGIC_F;
}

// (q - 8) in every byte of a word of nibbles 0..15, as signed bytes.
__device__ __forceinline__ int nibbles_minus8(uint32_t v) {
    uint32_t t = v ^ 0x08080808u;          // q>=8: q-8; q<8: q+8
    uint32_t neg = t & 0x08080808u;        // set where the result is negative
    return int(t | (neg * 30u));           // q+8 with 0xF0 on top = q-8 as a signed byte
}

__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}

// src/kernels.rs:544-564
__device__ __forceinline__ float exp_poly(float x) {
    x = x < -87.33655f ? -87.33655f : x;
    x = x > 88.7f ? 88.7f : x;
    const float n = roundf(x * 1.44269504088896340736f);
    const float r = x - n * 0.6933594f - n * -2.1219444e-4f;
    float y = 1.9875692e-4f;
    y = y * r + 1.3981999e-3f;
    y = y * r + 8.333452e-3f;
    y = y * r + 4.1665796e-2f;
    y = y * r + 0.16666665f;
    y = y * r + 0.5f;
    y = y * (r * r) + r + 1.0f;
    return __int_as_float(__float_as_int(y) + (int(n) << 23));
}

// sum_b c[row,b] * xsum[token,b]: eight lanes (one per block of a super-block)
// fma'd over super-blocks, then ((a0+a4)+(a1+a5))+((a2+a6)+(a3+a7)).
__device__ __forceinline__ float offset_dot(const uint32_t* words, const float* sums, int supers) {
    float acc[SUPER];
#pragma unroll
    for (int j = 0; j < SUPER; j++) acc[j] = 0.0f;
    for (int k = 0; k < supers; k++) {
        const uint32_t* w = words + k * SUPER_WORDS;
        const float step = f16_bits_to_f32(uint16_t(w[0] >> 16));
        const uint32_t o01 = w[3], o23 = w[4];
#pragma unroll
        for (int j = 0; j < SUPER; j++) {
            const uint32_t word = j < 4 ? o01 : o23;
            const float c = step * float(int(int8_t(uint8_t(word >> (8 * (j & 3))))));
            acc[j] = fmaf(c, sums[k * SUPER + j], acc[j]);
        }
    }
    return ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
}

// Two IEEE f32 operations per instruction (the results are those of the
// scalar forms): a - m, a * b, fma(a, b, c) on register pairs.
__device__ __forceinline__ float2 sub2(float2 a, float2 m) {
    float2 r;
    asm("{\n\t.reg .b64 ra, rm, rr;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rm, {%4, %5};\n\t"
        "sub.rn.f32x2 rr, ra, rm;\n\t"
        "mov.b64 {%0, %1}, rr;\n\t}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a.x), "f"(a.y), "f"(m.x), "f"(m.y));
    return r;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 r;
    asm("{\n\t.reg .b64 ra, rb, rr;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rr, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rr;\n\t}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 r;
    asm("{\n\t.reg .b64 ra, rb, rc, rr;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rr, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rr;\n\t}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return r;
}

}  // namespace tc
