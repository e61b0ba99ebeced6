/* tachyon_cuda.h: C ABI of the B200 (sm_100a) backend for Tachyon's Granite
 * mixture-of-experts block.
 *
 * This is the interface a `src/gpu/cuda/mod.rs` in Tachyon binds with
 * `extern "C"`, the way `src/gpu/mod.rs:115-145` binds the Metal shim
 * (`src/gpu/shim.m`). Plain pointers and sizes only. One thread drives a
 * context at a time (Tachyon's `Backend` is `Send`, not `Sync`:
 * src/engine.rs:8, src/gpu/mod.rs:440-442), so nothing here locks.
 *
 * Status codes: 0 = ok, negative = failure; the message is kept per context
 * and read with tc_last_error(). There is no CPU fallback: every entry point
 * that computes runs CUDA kernels or fails.
 */
#ifndef TACHYON_CUDA_H
#define TACHYON_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tc_ctx tc_ctx;
typedef struct tc_matrix tc_matrix;
typedef struct tc_moe_layer tc_moe_layer;
typedef struct tc_graph tc_graph;

/* Storage kinds of Tachyon's `Matrix` enum (src/weights.rs:58-79). */
enum { TC_BF16 = 0, TC_Q8 = 1, TC_Q4 = 2 };

/* ---- context: replaces tm_create / tm_destroy / tm_device_name
 *      (src/gpu/mod.rs:116-124, src/gpu/shim.m:33-70). */
tc_ctx *tc_create(int device_ordinal, char *err, size_t errlen);
void tc_destroy(tc_ctx *ctx);
void tc_device_name(tc_ctx *ctx, char *out, size_t len);
/* Copies the context's last error message into `out`; returns its length. */
size_t tc_last_error(tc_ctx *ctx, char *out, size_t len);
/* Waits for the context's stream; also reports a kernel's bounded wait that
 * ran out (replaces tm_end's error return, src/gpu/mod.rs:144, 1049-1053). */
int tc_sync(tc_ctx *ctx);
/* The context's stream as a cudaStream_t, for callers that enqueue their own work. */
void *tc_stream(tc_ctx *ctx);

/* How the expert products add up a row's 32-element blocks (src/kernels_x86.rs:79-129).
 * TC_ARITH_FAST (default): one fma chain per output over the exact integer
 *   block sums, blocks in order; the same on every kernel, so a token's result
 *   does not depend on its batch. Differs from the CPU path by float rounding only.
 * TC_ARITH_CPU_LANES: the CPU path's own eight-lane order and hsum tree:
 *   bit-identical to Tachyon's AVX2 kernels, at about five times the instructions. */
enum { TC_ARITH_FAST = 0, TC_ARITH_CPU_LANES = 1 };
int tc_set_arithmetic(tc_ctx *ctx, int mode);

/* Overlap of consecutive kernels of a block (programmatic dependent launch:
 * a kernel's weight prefetch runs under the previous kernel's tail). Process-wide,
 * on by default; results do not depend on it. */
int tc_set_launch_overlap(tc_ctx *ctx, int on);

/* From how many tokens per expert (batch tokens x experts per token / experts,
 * on average) a block's expert products run on the tcgen05 tensor-core kernels
 * instead of the bandwidth-oriented ones. Default 32; 0 = always; a huge value
 * = never. Both give the same values (same fma chain per output). */
int tc_set_prefill_threshold(tc_ctx *ctx, int avg_tokens_per_expert);

/* Decode-size blocks (8-bit or 4-bit experts, default arithmetic) run as ONE kernel whose
 * CTAs meet at grid-wide counters (no counterpart in the reference, whose Metal backend
 * encodes a dispatch per step: src/gpu/mod.rs:651-702): up to 32 tokens directly, and up to
 * 128 tokens with an expert's tokens walked in runs of up to 32. on = 1: the default; on = 0: the four-kernel path;
 * on > 1: one kernel up to that many tokens (at most 128). All give the same values. */
int tc_set_decode_block(tc_ctx *ctx, int on);

/* ---- device buffers: replace tm_buffer / tm_buffer_contents / tm_buffer_free
 *      (src/gpu/mod.rs:125-127). HBM is not host-visible, hence the copies. */
void *tc_malloc(tc_ctx *ctx, size_t bytes);
void tc_free(tc_ctx *ctx, void *dev);
int tc_upload(tc_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
int tc_download(tc_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes);
int tc_memset(tc_ctx *ctx, void *dst_dev, int value, size_t bytes);
/* Device-to-device copy on the context's stream (not waited for). */
int tc_copy(tc_ctx *ctx, void *dst_dev, const void *src_dev, size_t bytes);
/* Page-locked host memory, so uploads and downloads run at full PCIe rate. */
void *tc_host_alloc(tc_ctx *ctx, size_t bytes);
void tc_host_free(tc_ctx *ctx, void *host);

/* ---- weights: replaces GpuMatrix::upload (src/gpu/mod.rs:222-251). Takes the
 * buffers of a `Matrix` byte for byte:
 *   TC_BF16: scales = NULL;                       data = u16[rows*cols]
 *   TC_Q8:   scales = u16 f16 [rows*cols/32];     data = i8[rows*cols]
 *   TC_Q4:   scales = u32 [rows*ceil(cols/256)*5]; data = u8[rows*cols/2]
 * cols must be a multiple of 32 (as src/gpu/mod.rs:241-243 requires). */
tc_matrix *tc_matrix_upload(tc_ctx *ctx, int kind, size_t rows, size_t cols, const void *scales,
                            size_t scales_bytes, const void *data, size_t data_bytes);
/* The same from f32 values: Matrix::from_f32 (src/weights.rs:82-105) on the device.
 * Uploads data_host (f32[rows*cols]) and quantizes it there with Tachyon's own
 * quantizers (f32_to_bf16 src/kernels.rs:21-28; quantize_q8_weights 135-149;
 * quantize_q4_packed 180-242 with fit_q4_offset 438-495, no importance matrix):
 * the bytes are those the host loader would have produced. */
tc_matrix *tc_matrix_quantize(tc_ctx *ctx, int kind, size_t rows, size_t cols, const float *data_host);
/* Copies a matrix's buffers back to the host (sizes as for tc_matrix_upload). */
int tc_matrix_download(const tc_matrix *m, void *scales_host, size_t scales_bytes, void *data_host,
                       size_t data_bytes);
void tc_matrix_free(tc_matrix *m);

/* ---- the MoE block: replaces GpuBackend::moe (src/gpu/mod.rs:651-702) with
 * the arithmetic of the CPU path (src/model.rs:462-521).
 * router: TC_BF16 [experts, hidden]; gate_up: [experts*2*inter, hidden];
 * down: [experts*hidden, inter]; both TC_Q8 or TC_Q4. max_tokens bounds `t`
 * of later forwards (scratch is sized from it, here, not during a forward). */
tc_moe_layer *tc_moe_layer_create(tc_ctx *ctx, int hidden, int experts, int experts_per_token,
                                  int inter, const tc_matrix *router, const tc_matrix *gate_up,
                                  const tc_matrix *down, int max_tokens);
void tc_moe_layer_free(tc_moe_layer *layer);
/* A layer keeps its own re-tiled copies of the expert matrices; the matrices as uploaded are
 * only read again by TC_ARITH_CPU_LANES. After this call the layer no longer refers to them, so
 * the caller may tc_matrix_free gate_up and down (a third of the layer's expert memory); blocks
 * in TC_ARITH_CPU_LANES are then refused for this layer. (The Metal backend keeps one copy,
 * src/gpu/mod.rs:222-251; no counterpart there.) */
int tc_moe_layer_detach_experts(tc_moe_layer *layer);
/* A bias added to every token's router logits before top-k (NULL clears it).
 * Tachyon's router has none (src/model.rs:473); the routing-skew workload
 * adds one on both the CPU and the GPU side. bias_host: f32[experts]. */
int tc_moe_set_router_bias(tc_moe_layer *layer, const float *bias_host);
/* y[t,hidden] += moe(x[t,hidden]); x is the normed input (`s.xb`), y the
 * residual stream (`s.x`): src/model.rs:671-681. Device pointers; enqueued on
 * the context's stream, returns without waiting. */
int tc_moe_forward(tc_moe_layer *layer, const float *x_dev, int t, float *y_dev);
/* The whole MLP block of a MoE layer on the residual stream, as
 * src/model.rs:662-681 runs it: y[t,hidden] += moe(rmsnorm(y, norm_weight, eps)).
 * The norm is fused into the router kernel (same arithmetic as tc_rmsnorm). */
int tc_moe_block(tc_moe_layer *layer, const float *norm_weight_dev, float eps, int t, float *y_dev);
/* The same through host buffers: copies x and y in, runs, copies y back, waits. */
int tc_moe_forward_host(tc_moe_layer *layer, const float *x_host, int t, float *y_host);
/* Routing of the last forward, copied to the host (any pointer may be NULL):
 * ids u32[t*k] and gates f32[t*k] in descending score order per token
 * (src/model.rs:448-457), counts u32[experts] = tokens per expert
 * (src/model.rs:474-482), logits f32[t*experts]. Waits for the stream. */
int tc_moe_last_routing(tc_moe_layer *layer, uint32_t *ids, float *gates, uint32_t *counts,
                        float *logits);

/* Dispatch of the last forward, copied to the host (either may be NULL):
 * offsets u32[experts+1] = first expert-contiguous slot of each expert, and
 * perm u32[t*k] = for each expert-contiguous slot, token*k + pick. Within an
 * expert, slots are in ascending token order: the per-expert lists of
 * src/model.rs:474-482. Waits for the stream. */
int tc_moe_last_dispatch(tc_moe_layer *layer, uint32_t *offsets, uint32_t *perm);

/* The token -> expert dispatch on its own, for callers that must not allocate.
 * It has no counterpart in the reference. Tachyon's scheduler thread drives the
 * backend inside its step loop (src/scheduler.rs:567-722) and a backend sized to
 * fill the device with KV-cache blocks at start-up has no memory left to ask
 * for later; cudaMalloc and cudaFree also stall the whole device while they
 * run. This entry point therefore allocates and frees nothing: the one piece
 * of scratch the three-pass dispatch needs (per-CTA histograms, 64 KiB) lives
 * in an array inside the library, held by every GPU that loads it until the
 * process exits.
 *   ids_dev u32[t*k]: each token's experts (what tc_moe_last_routing returns).
 *   Outputs (device, all required): counts u32[experts], offsets
 *   u32[experts+1], perm u32[t*k], pos u32[t*k], slot_token u32[t*k], active
 *   i32[experts+1] (experts with tokens, ascending; [experts] = their number).
 * Limits: t <= 16384, experts <= 256; anything beyond is refused with a
 * message. The first call on a device looks the array's address up: make it
 * before any stream capture. All calls on a device share the array, so two
 * calls whose kernels overlap on the GPU race; calls on one stream do not. */
int tc_dispatch_static(tc_ctx *ctx, const uint32_t *ids_dev, int t, int experts, int experts_per_token,
                       uint32_t *counts_dev, uint32_t *offsets_dev, uint32_t *perm_dev, uint32_t *pos_dev,
                       uint32_t *slot_token_dev, int32_t *active_dev);

/* ---- expert parallelism over the GPUs of one node (no counterpart in the
 * reference, which is single-device). Experts are sharded in contiguous ranges,
 * the remainder to the low ranks (tc_ep_expert_range); the router is
 * replicated; each rank keeps its own tokens; one process drives one GPU.
 * Rank 0 makes an id (tc_ep_unique_id, 128 bytes), the host passes it to every
 * rank, each calls tc_ep_init (collective). A layer made with
 * tc_moe_ep_layer_create takes the full router and THIS rank's rows of gate_up
 * and down; tc_moe_forward / tc_moe_block on it exchange rows with two NCCL
 * all-to-alls per block and give the same values as one GPU would. */
int tc_ep_unique_id(char *out128);
int tc_ep_init(tc_ctx *ctx, const char *id128, int rank, int size);
int tc_ep_expert_range(int experts, int rank, int size, int *first, int *count);
/* Promise that every rank calls each block with the SAME number of tokens. Layers
 * created afterwards then run decode-size blocks (ranks x tokens x experts-per-
 * token x hidden x 4 bytes <= 64 MiB) through a fixed-size exchange: one grouped
 * all-gather of the 8-bit rows and expert ids, the dispatch over all ranks'
 * tokens, this rank's experts, one reduce-scatter of the slot-ordered outputs.
 * Nothing is read on the host, so such a block can be captured in a CUDA graph;
 * same values as one GPU. Larger blocks keep the all-to-all-v exchange. Create
 * every layer before capturing. */
int tc_ep_set_uniform_batch(tc_ctx *ctx, int on);
/* Collective, up to 8 ranks of one NVSwitch node, before the layers are created;
 * implies tc_ep_set_uniform_batch(ctx, 1). Blocks of up to max_tokens tokens per
 * rank with this hidden size and experts-per-token then exchange over peer memory:
 * each rank allocates a window, the others map it (CUDA IPC), rows and expert
 * outputs are stored straight into the destination rank's window over NVLink and
 * announced with flags that the consuming kernels wait for (bounded: a rank that
 * never signals leaves an error status for tc_sync, not a hang). No collective
 * library call runs inside a block; same values as one GPU. */
int tc_ep_enable_peer_exchange(tc_ctx *ctx, int hidden, int experts_per_token, int max_tokens);
/* How long a kernel of the peer-memory exchange polls another rank's flag before it
 * gives up, leaves an error status for tc_sync and goes on (default 2^23 polls,
 * about ten seconds). Applies to blocks enqueued (or captured) afterwards. */
int tc_ep_set_wait_limit(tc_ctx *ctx, uint32_t polls);
/* Testing hook: the next `blocks` blocks store this rank's rows into the windows but
 * do not announce them, as if the rank never signalled; the kernels waiting for it
 * then run into the limit above. No fault is injected and nothing hangs. */
int tc_ep_test_mute_signals(tc_ctx *ctx, int blocks);
/* Collective: returns when every rank has reached it (host-side barrier). */
int tc_ep_barrier(tc_ctx *ctx);
tc_moe_layer *tc_moe_ep_layer_create(tc_ctx *ctx, int hidden, int experts, int experts_per_token, int inter,
                                     const tc_matrix *router, const tc_matrix *gate_up_local,
                                     const tc_matrix *down_local, int max_tokens);

/* Self-check of the tcgen05 path's encodings (no counterpart in the reference):
 * one 128 x n x 32 int8 MMA (n = 64 or 128) through tensor memory.
 * a_rows_host: i8[128*32], b_rows_host: i8[n*32], row-major; d_out_host:
 * i32[128*n] = a_rows x b_rows^T. Allocates and frees its own scratch. */
int tc_umma_selftest(tc_ctx *ctx, const int8_t *a_rows_host, const int8_t *b_rows_host, int n,
                     int32_t *d_out_host);

/* The dense int8 rate of the tensor cores, measured (no counterpart in the reference):
 * every SM issues `batches` batches of 32 tcgen05 MMAs (128 x 256 x 32, int8 -> int32,
 * accumulating in tensor memory) from operands resident in shared memory. Returns the
 * integer operations performed (multiply and add counted separately) and the kernel's
 * duration in milliseconds (CUDA events): the denominator of the prefill-size kernels'
 * tensor-pipe fraction. Allocates and frees one status word. */
int tc_int8_peak(tc_ctx *ctx, int batches, double *ops_out, float *ms_out);

/* ---- the pre-MoE norm: kernels::rmsnorm (src/kernels.rs:522-528) per row,
 * as src/model.rs:662-667 applies it. out may alias x. */
int tc_rmsnorm(tc_ctx *ctx, const float *x_dev, const float *weight_dev, float eps, int t, int n,
               float *out_dev);

/* ---- stream capture: one launch for a whole stack of blocks at a fixed
 * batch size. Everything enqueued on the context's stream between begin and
 * end is recorded, not run. */
int tc_capture_begin(tc_ctx *ctx);
tc_graph *tc_capture_end(tc_ctx *ctx);
int tc_graph_launch(tc_graph *g);
void tc_graph_free(tc_graph *g);

/* ---- timing on the context's stream with CUDA events. */
int tc_timer_start(tc_ctx *ctx);
/* Records the stop event, waits for it, returns milliseconds (negative on error). */
float tc_timer_stop_ms(tc_ctx *ctx);

/* ---- per-kernel timing. While enabled (and outside a capture), every kernel
 * the library enqueues is bracketed by CUDA events on the context's stream.
 * tc_profile_read() waits, then adds up milliseconds and launches per stage
 * since the last read: stage 0 route, 1 dispatch, 2 gate_up, 3 quantize
 * hidden, 4 down, 5 combine, 6 rmsnorm, 7 the one-kernel decode block
 * (TC_PROFILE_STAGES entries each). */
#define TC_PROFILE_STAGES 8
int tc_profile_enable(tc_ctx *ctx, int on);
int tc_profile_read(tc_ctx *ctx, float *ms, uint64_t *launches);

/* Phase timing inside the one-kernel decode block. While on, CTA 0 of every such
 * kernel stores the GPU's wall clock (ns) at: entry, after its wait for the previous
 * kernel, after the router phase, after gate_up, after down, at exit.
 * tc_profile_read_phases() waits for the stream and returns the six stamps of the
 * last block that ran (also from a replayed graph captured while this was on). */
int tc_profile_phases(tc_ctx *ctx, int on);
int tc_profile_read_phases(tc_ctx *ctx, uint64_t *ns6);

/* Number of kernel launches this context has enqueued so far. */
uint64_t tc_launch_count(tc_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* TACHYON_CUDA_H */
