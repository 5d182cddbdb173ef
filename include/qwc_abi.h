/*
 * C ABI of the sm_100a decode-step kernels.
 *
 * Every `qwc_*` launcher below that carries a reference citation has exactly the
 * signature the reference's Rust FFI declares in crates/qwc-cuda/src/ffi.rs, so the
 * shared library can be linked in place of the reference's libqwc_kernels.a:
 *   - all pointers are DEVICE pointers unless the comment says "host";
 *   - shapes are `int`, the CUDA stream is always the last argument;
 *   - the return value is a cudaError_t carried as `int` (0 = success); bad, NULL or
 *     out-of-range arguments give cudaErrorInvalidValue (1) before anything is launched;
 *   - the callee never allocates, frees, retains a pointer or synchronises, and every
 *     launcher is legal inside cudaStreamBeginCapture (ThreadLocal).
 *
 * `qwc_stream` is a cudaStream_t.  The header has no CUDA include on purpose: it is
 * what a cgo / Rust-bindgen / ctypes binding reads.
 */
#ifndef QWC_ABI_H
#define QWC_ABI_H

#include <stddef.h>
#include <stdint.h>

#include "qwc_exchange.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void* qwc_stream;

/* ------------------------------------------------------------------ */
/* Shape selection (additive; no reference counterpart)                 */
/* ------------------------------------------------------------------ */

/*
 * The reference bakes its model dimensions in as constexpr
 * (cuda/delta_net.cu:36-38 value heads 48, cuda/paged_attention.cu:21 page 64).
 * The legacy-signature launchers below read the two dimensions that differ between
 * the reference checkpoint and the synthetic 27B-shaped model from this process-wide
 * setting.  Defaults reproduce the reference: 48 value heads, 64-token pages.
 * Supported: delta_value_heads in {32, 48}; kv_page_size in {16, 64}.
 * Host call; not thread-safe against concurrent launches.
 */
typedef struct qwc_shape {
    int delta_value_heads;
    int kv_page_size;
} qwc_shape;

int qwc_configure(const qwc_shape* shape);
void qwc_get_shape(qwc_shape* shape);

/* Sticky device-side status word: 0, or the code of the first bounded wait that gave up
 * (see qwc_device_status_reset).  Host call; synchronises the device. */
int qwc_device_status(void);
int qwc_device_status_reset(void);
/* After code 0x106 (a wait for a peer's words gave up): the tag the first such wait looked for and the
 * tag it found instead (epoch << 10 | exchange number; 0 = never written).  Host-side, synchronising. */
int qwc_device_status_detail(uint32_t* expected_and_found);
/* Host-side fault injection: stores `code` in the status word as a bounded wait that gave up
 * would (every kernel that waits then returns at once and skips its stores).  Synchronises. */
int qwc_device_status_set(int code);
/* Copies the status word to `destination` (device memory, 4 bytes) in stream order: no sync,
 * capture-legal.  A step that ends with this copy lets its caller read the word together with
 * the step's results instead of synchronising for it. */
int qwc_device_status_copy(void* destination, qwc_stream stream);

/* ------------------------------------------------------------------ */
/* NVFP4 W4A16 projections                                              */
/* ------------------------------------------------------------------ */

/*
 * Y[b, n] = sum_k e2m1(W[n, k]) * e4m3(S[n, k / 16]) / weight_global_scale * X[b, k].
 * Replaces crates/qwc-cuda/src/ffi.rs:352-362 (cuda/nvfp4.cu:489-537).
 * packed: u8[out, in/2], low nibble = even k.  scales: e4m3 in the 128x4 swizzled
 * block-scale layout of cuda/nvfp4.cu:33-39 (rows padded to 128, groups to 4).
 * input bf16[batch, in], output bf16[batch, out].  in_features % 256 == 0.
 * batch 1..32 (the reference stops at 8), one pass over the weights for all rows.
 */
int qwc_nvfp4_w4a16(const void* packed, const void* scales, const void* input, void* output,
                    int out_features, int in_features, int batch, float weight_global_scale,
                    qwc_stream stream);

/*
 * H[b, n] = silu(gate(x))[n] * up(x)[n], two NVFP4 matrices sharing one input.
 * Replaces crates/qwc-cuda/src/ffi.rs:383-396 (cuda/nvfp4.cu:585-643).  batch 1..32.
 */
int qwc_nvfp4_swiglu_w4a16(const void* gate_packed, const void* gate_scales, const void* up_packed,
                           const void* up_scales, const void* input, void* output,
                           int out_features, int in_features, int batch, float gate_global_scale,
                           float up_global_scale, qwc_stream stream);

/*
 * Additive (no reference counterpart).  Names the weights of the projection that the calling
 * thread's stream will run AFTER the next qwc_nvfp4_w4a16 / qwc_nvfp4_swiglu_w4a16 /
 * qwc_fp8_lm_head* call it makes: that launch then asks L2 for the first stages of the named
 * matrix once its own last bytes are on their way, so HBM keeps streaming across the kernel
 * boundary.  kind: 0 = NVFP4 matrix (packed0, scales0), 1 = SwiGLU pair (packed0/scales0 = gate,
 * packed1/scales1 = up), 2 = e4m3 rows of the vocabulary head (packed0 = table; no scales),
 * 3 = an NVFP4 matrix that will run through qwc_nvfp4_w4a16_split (or qwc_nvfp4_w4a16_exchange),
 * 4 = a SwiGLU pair that will run through qwc_nvfp4_swiglu_w4a16_exchange.
 * Pure hint: host-side only (no launch, no sync, capture-legal), good for one launch of this
 * thread, ignored when that launch does not take the tcgen05 path; wrong or stale hints cost
 * bandwidth, never correctness (prefetches do not fault on valid device memory and write nothing).
 * The pointers must be device memory of the shapes given, 16-byte aligned, and must stay mapped
 * until the projection call that consumes the hint has run on the device (a call that is refused
 * for bad arguments consumes the hint without launching anything).
 * Returns cudaErrorInvalidValue for a null matrix, non-positive or misaligned shapes, or an unknown kind.
 */
int qwc_nvfp4_prefetch_next(const void* packed0, const void* scales0, const void* packed1,
                            const void* scales1, int out_features, int in_features, int kind);

/*
 * Additive (no reference counterpart): the same projections on STAGED activations, for a caller
 * that chains them (the decode executor).  "Staged" is f16 in the layout the tensor core reads its
 * B operand in: [features / 8][rows padded to 16 (batch <= 16) or 32][8], so that a 128-element
 * chunk of every row is one contiguous block (qwc_staged_activation_bytes gives the size;
 * qwc_stage_activations converts bf16 rows; values are the bf16 values, |x| > 65504 saturates).
 * The kernels that produce activations can store this layout directly (the `_staged` variants of
 * the RMSNorm, gated RMSNorm and attention entry points below, and `staged_output` here), so no
 * projection converts its input.  The work of a launch is cut into equal shares for every SM; tiles
 * whose K range is split between CTAs are summed through `workspace` (qwc_streamk_workspace_bytes()
 * bytes of device memory, 16-byte aligned, cleared once with qwc_streamk_workspace_init and then
 * left to the library; launches that overlap on the device must not share one).  Sums are taken in
 * a fixed order: results are bit-reproducible.  `output` (bf16 [batch][out]) and `staged_output`
 * (the same values staged for a following projection) may each be NULL, not both.
 * out_features % 8 == 0, in_features % 256 == 0, batch 1..32, all pointers 16-byte aligned.
 * A launch in which a bounded wait gave up (qwc_device_status) leaves the workspace dirty: clear it
 * again before the next use.  qwc_nvfp4_prefetch_next applies to these calls as well.
 */
size_t qwc_streamk_workspace_bytes(void);
int qwc_streamk_workspace_init(void* workspace, qwc_stream stream);
size_t qwc_staged_activation_bytes(int batch, int features);
int qwc_stage_activations(const void* input, void* staged, int batch, int in_features, qwc_stream stream);
int qwc_nvfp4_w4a16_staged(const void* packed, const void* scales, const void* staged_input, void* output,
                           void* staged_output, int out_features, int in_features, int batch,
                           float weight_global_scale, void* workspace, qwc_stream stream);
int qwc_nvfp4_swiglu_w4a16_staged(const void* gate_packed, const void* gate_scales, const void* up_packed,
                                  const void* up_scales, const void* staged_input, void* output,
                                  void* staged_output, int out_features, int in_features, int batch,
                                  float gate_global_scale, float up_global_scale, void* workspace,
                                  qwc_stream stream);
/*
 * Additive: a projection whose output feeds a residual RMSNorm and has too few rows for the SMs
 * (5120 outputs = 20 tile pairs on 148 SMs) runs as a regular K split and leaves the sum to the norm:
 * qwc_nvfp4_w4a16_split stores fp32 partial rows [qwc_nvfp4_split_count(out, in)][batch][out]
 * (unscaled: the global scale is applied after the sum) and ends with plain stores, no reduction
 * between CTAs; qwc_rmsnorm_bf16_split_staged sums the slices in slice order (bit-reproducible),
 * rounds the sum / weight_global_scale to bf16 as the projection would have (and stores those rows
 * in `projection_output`, bf16 [batch][hidden], when it is not NULL), and continues as
 * qwc_rmsnorm_bf16_staged on those values.  hidden <= 10240.
 */
int qwc_nvfp4_split_count(int out_features, int in_features);
int qwc_nvfp4_w4a16_split(const void* packed, const void* scales, const void* staged_input, float* partial_sums,
                          int out_features, int in_features, int batch, qwc_stream stream);
int qwc_rmsnorm_bf16_split_staged(const float* partial_sums, int splits, float weight_global_scale,
                                  void* projection_output, void* residual, const void* weight, void* output,
                                  void* staged_output, int batch, int hidden, float epsilon, qwc_stream stream);

/* Consumers of a K-split projection other than the residual norm: the DeltaNet prepare step and the
 * gated RMSNorm on a split mixer in-projection (same arithmetic as qwc_delta_prepare_decode and
 * qwc_delta_gated_rmsnorm_staged; a, b and the gate z are columns a_column, b_column, gate_column of
 * the in-projection's rows of `width` outputs), and the plain sum to bf16 rows [batch][width]. */
int qwc_delta_prepare_decode_split(const float* partial_sums, int slices, int width, float weight_global_scale,
                                   int a_column, int b_column, const void* conv_weight, const void* a_log,
                                   const void* dt_bias, void* conv_state, const void* state_slots, void* query,
                                   void* key, void* value, void* alpha, void* beta, void* kq, int state_capacity,
                                   int batch, qwc_stream stream);
int qwc_delta_gated_rmsnorm_split(const float* input, const float* partial_sums, int slices, int width,
                                  float weight_global_scale, int gate_column, const void* weight, void* output,
                                  void* staged_output, int batch, float epsilon, qwc_stream stream);
int qwc_nvfp4_sum_slices(const float* partial_sums, int slices, float weight_global_scale, void* rows, int batch,
                         int width, qwc_stream stream);
/* The recurrent update in the step's own form: as qwc_delta_decode_int8, but the state slots and the
 * state tiles are fetched before the kernel waits for its predecessor on the stream (so neither may be
 * written by the kernels just before it: in a decode step they are not), and - when every head is one
 * CTA, which qwc_delta_decode_fuses_norm(batch) tells - the gated RMSNorm (qwc_delta_gated_rmsnorm*)
 * runs in the same CTA: `staged_output` (not NULL) receives its result staged for the output
 * projection and `out` is left alone.  The gate z is column `gate_column` of the in-projection's rows
 * of `width` outputs, given as K-split slices (gate_sums, slices, gate_global_scale) or bf16 rows. */
int qwc_delta_decode_fuses_norm(int batch);
int qwc_delta_decode_int8_step(void* state, float* state_scales, const void* state_slots, const void* q,
                               const void* k, const void* v, const void* alpha, const void* beta, const void* kq,
                               void* out, int state_capacity, int batch, const float* gate_sums, int slices,
                               float gate_global_scale, const void* gate_rows, int width, int gate_column,
                               const void* norm_weight, float epsilon, void* staged_output, qwc_stream stream);

/*
 * The FP8 vocabulary head (see qwc_fp8_lm_head_batched) on staged activations, with greedy sampling
 * folded in: `logits` (f32 [batch][vocab]) may be NULL when only the tokens are wanted, `sampled`
 * (u32 [batch], argmax with ties to the smaller index, cuda/sampling.cu:11-14) may be NULL when only
 * the logits are.  With `sampled`, `status_out` (u32, may be NULL) receives the device status word.
 */
int qwc_fp8_lm_head_staged(const void* weights, const void* row_scales, const void* staged_input, void* logits,
                           void* sampled, void* status_out, int batch, int hidden_size, int vocab,
                           void* workspace, qwc_stream stream);

/*
 * Additive: latency mode.  The weight rows of every projection are split over the ranks of one node
 * and a single sequence is decoded (batch 1).  Where the reference gathers each projection's output
 * with ncclAllGather, these entry points fuse the exchange into the kernels on both sides of it:
 *
 *  - qwc_nvfp4_w4a16_exchange / qwc_nvfp4_swiglu_w4a16_exchange run this rank's rows as a regular K
 *    split and store every partial sum into EVERY rank's copy of the row
 *    ([qwc_nvfp4_exchange_slices(...)][row->width] words of 8 bytes at row->offset of each block):
 *    columns rank * out_features .. of the row; for the SwiGLU pair the row is [gate | up], each half
 *    ranks * out_features wide, unscaled and uncombined;
 *  - the consumers (qwc_rmsnorm_bf16_exchanged, qwc_delta_prepare_decode_exchanged,
 *    qwc_delta_gated_rmsnorm_exchanged, qwc_nvfp4_sum_exchanged, qwc_swiglu_combine_exchanged) sum
 *    the slices of their own rank's copy in slice order, exactly as their one-GPU forms do, after a
 *    bounded wait for the words of this step (status code 0x106 in the device status word when a
 *    peer's words do not come; the step's tokens must then be discarded);
 *  - qwc_fp8_lm_head_exchange scans this rank's vocabulary rows and hands every rank its best
 *    candidates; the token stored in `sampled` is the same on all ranks (ties to the smaller index;
 *    `sampled` NULL: the candidates are stored and no token is picked; `logits`, f32 [vocab_local],
 *    may be NULL and receives this rank's columns only).
 *
 * All ranks must issue the same sequence of steps (qwc_exchange_advance first in each) with the same
 * instance numbers.  Every rank of a row must use the same slice count, which holds when they call
 * with the same shapes.  One activation row only.
 */
int qwc_exchange_advance(void* epoch, qwc_stream stream);
size_t qwc_exchange_row_bytes(int width);
size_t qwc_exchange_candidate_bytes(int ranks);
int qwc_nvfp4_exchange_slices(int out_features, int in_features, int swiglu);
int qwc_nvfp4_w4a16_exchange(const void* packed, const void* scales, const void* staged_input,
                             const qwc_exchange_row* row, int out_features, int in_features, qwc_stream stream);
int qwc_nvfp4_swiglu_w4a16_exchange(const void* gate_packed, const void* gate_scales, const void* up_packed,
                                    const void* up_scales, const void* staged_input, const qwc_exchange_row* row,
                                    int out_features, int in_features, qwc_stream stream);
int qwc_rmsnorm_bf16_exchanged(const qwc_exchange_row* row, int slices, float weight_global_scale,
                               void* projection_output, void* residual, const void* weight, void* output,
                               void* staged_output, int hidden, float epsilon, qwc_stream stream);
int qwc_delta_prepare_decode_exchanged(const qwc_exchange_row* row, int slices, float weight_global_scale,
                                       int a_column, int b_column, const void* conv_weight, const void* a_log,
                                       const void* dt_bias, void* conv_state, const void* state_slots,
                                       void* query, void* key, void* value, void* alpha, void* beta, void* kq,
                                       int state_capacity, qwc_stream stream);
int qwc_delta_gated_rmsnorm_exchanged(const float* input, const qwc_exchange_row* row, int slices,
                                      float weight_global_scale, int gate_column, const void* weight,
                                      void* output, void* staged_output, float epsilon, qwc_stream stream);
int qwc_nvfp4_sum_exchanged(const qwc_exchange_row* row, int slices, float weight_global_scale, void* rows,
                            qwc_stream stream);
int qwc_swiglu_combine_exchanged(const qwc_exchange_row* row, int slices, float gate_global_scale,
                                 float up_global_scale, void* output, void* staged_output, int intermediate,
                                 qwc_stream stream);
int qwc_fp8_lm_head_exchange(const void* weights, const void* row_scales, const void* staged_input,
                             void* logits, const qwc_exchange_row* candidates, void* sampled, void* status_out,
                             int hidden_size, int vocab_local, void* workspace, qwc_stream stream);

/*
 * Additive: the producers of activations with a staged output beside (or instead of) their bf16
 * rows.  Same arguments and arithmetic as qwc_rmsnorm_bf16, qwc_delta_gated_rmsnorm and
 * qwc_paged_attention_packed_fp8_scaled below; `output` and `staged_output` may each be NULL, not
 * both; with a staged output the batch (row_base + rows for attention) is at most 32.
 */
int qwc_rmsnorm_bf16_staged(const void* input, void* residual, const void* weight, void* output,
                            void* staged_output, int batch, int hidden, float epsilon, qwc_stream stream);
int qwc_delta_gated_rmsnorm_staged(const float* input, const void* gate, const void* weight, void* output,
                                   void* staged_output, int batch, float epsilon, int gate_stride,
                                   qwc_stream stream);
int qwc_paged_attention_packed_fp8_staged(const void* query, const void* query_gate_projection,
                                          const void* key_cache, const void* value_cache,
                                          const void* block_tables, const void* context_lengths,
                                          const float* key_scales, const float* value_scales, void* output,
                                          void* staged_output, void* workspace, size_t workspace_bytes, int rows,
                                          int row_base, int max_blocks, int page_size, int gate_stride,
                                          int partitions, float softmax_scale, qwc_stream stream);

/* ------------------------------------------------------------------ */
/* Packed paged FP8 attention                                           */
/* ------------------------------------------------------------------ */

/*
 * Decode attention for `rows` query rows (row_base .. row_base + rows), 24 query heads
 * packed six to a KV head, head_dim 256, e4m3 K/V pages u8[num_blocks, 4, PAGE, 256].
 * Replaces crates/qwc-cuda/src/ffi.rs:520-537 (cuda/paged_attention.cu:1913-1958).
 * query bf16[*, 24, 256]; query_gate_projection bf16[*, 24, 512] or NULL (sigmoid gate
 * from the second half of each head); block_tables u32[*, max_blocks];
 * context_lengths u32[*]; output bf16[*, 24, 256].
 * workspace holds split-context partials: per (row, head, partition) max f32, sum f32 and
 * 256 f16 values = rows * 24 * partitions * 520 bytes; ignored when partitions == 1,
 * too small -> cudaErrorInvalidValue.  tile_size must be 6 (one decode row per tile);
 * larger tiles (segments of one sequence) are prefill shapes -> cudaErrorNotSupported.
 */
int qwc_paged_attention_packed_fp8(const void* query, const void* query_gate_projection,
                                   const void* key_cache, const void* value_cache,
                                   const void* block_tables, const void* context_lengths,
                                   void* output, void* workspace, size_t workspace_bytes, int rows,
                                   int row_base, int max_blocks, int tile_size, int partitions,
                                   float softmax_scale, qwc_stream stream);

/*
 * Same, with per-KV-head dequantisation scales f32[4] for K and V (device pointers, either
 * may be NULL = 1.0), an explicit page size, and the row stride (in elements) of
 * query_gate_projection so that [q; gate] may sit inside a wider fused projection row
 * (0 = 24 * 512, the reference layout).  No reference counterpart: the reference cache is
 * unscaled (cuda/attention_prepare.cu:139-142).
 */
int qwc_paged_attention_packed_fp8_scaled(const void* query, const void* query_gate_projection,
                                          const void* key_cache, const void* value_cache,
                                          const void* block_tables, const void* context_lengths,
                                          const float* key_scales, const float* value_scales,
                                          void* output, void* workspace, size_t workspace_bytes,
                                          int rows, int row_base, int max_blocks, int page_size,
                                          int gate_stride, int partitions, float softmax_scale,
                                          qwc_stream stream);

/*
 * Packed attention for callers that cannot allocate device memory.  No counterpart in the
 * reference, whose wrappers always own a workspace buffer.
 *
 * Same arithmetic and arguments as qwc_paged_attention_packed_fp8_scaled, without the workspace
 * pair: the split-context partials go to a scratch array built into the library (6 389 760 bytes
 * of device memory per GPU that loads it, held until the process exits).  Intended for a caller
 * that gave its whole memory budget away at start-up, a language binding with no allocator of
 * its own, or a tool attached to a running server.  The call itself performs no cudaMalloc,
 * cudaFree or other allocating call.
 *
 * Limit: rows * partitions <= qwc_paged_attention_packed_noalloc_max_pairs() (512); anything
 * larger is refused with cudaErrorInvalidValue before a launch.  The first call on a device
 * looks the scratch address up (cudaGetSymbolAddress with that device current) and should
 * therefore be made before any stream capture begins.  All calls share the one array: it keeps
 * whatever the previous call left (every slot a call reads it has written first, so nothing has
 * to be cleared), and two calls whose kernels overlap on the GPU - different streams, or
 * different host threads - race on it.  Callers that need concurrency pass their own workspace
 * to the _scaled entry point instead.
 */
int qwc_paged_attention_packed_fp8_noalloc(const void* query, const void* query_gate_projection,
                                           const void* key_cache, const void* value_cache,
                                           const void* block_tables, const void* context_lengths,
                                           const float* key_scales, const float* value_scales,
                                           void* output, int rows, int row_base, int max_blocks,
                                           int page_size, int gate_stride, int partitions,
                                           float softmax_scale, qwc_stream stream);
int qwc_paged_attention_packed_noalloc_max_pairs(void);

/* Host helper: bytes of split-context workspace for (rows, partitions). */
size_t qwc_paged_attention_packed_workspace_bytes(int rows, int partitions);

/* ------------------------------------------------------------------ */
/* Gated DeltaNet, int8 state                                           */
/* ------------------------------------------------------------------ */

/*
 * One recurrent step for `batch` slots: state i8[capacity, Hv, 128, 128] with per-row
 * scales f32[capacity, Hv, 128], addressed through state_slots u32[batch] (NULL = slot b).
 * q, k f32[batch, 16, 128]; v f32[batch, Hv, 128]; alpha, beta f32[batch, Hv];
 * kq f32[batch, 16]; out f32[batch, Hv, 128].  Hv from qwc_configure.
 * Replaces crates/qwc-cuda/src/ffi.rs:164-178 (cuda/delta_net.cu:1220-1237).
 */
int qwc_delta_decode_int8(void* state, float* state_scales, const void* state_slots, const void* q,
                          const void* k, const void* v, const void* alpha, const void* beta,
                          const void* kq, void* out, int state_capacity, int batch,
                          qwc_stream stream);

/*
 * conv1d update + SiLU + q/k/v split, then L2 normalisation, k.q, alpha and beta.
 * Replaces crates/qwc-cuda/src/ffi.rs:284-304 (cuda/delta_prepare.cu:249-316).
 */
int qwc_delta_prepare_decode(const void* mixed_qkv, const void* a_projection,
                             const void* b_projection, const void* conv_weight, const void* a_log,
                             const void* dt_bias, void* conv_state, const void* state_slots,
                             void* query, void* key, void* value, void* alpha, void* beta, void* kq,
                             int state_capacity, int batch, int mixed_stride, int gate_stride,
                             qwc_stream stream);

/*
 * RMSNormGated over 128-wide value heads: bf16(out) -> norm -> * weight -> * silu(z).
 * Replaces crates/qwc-cuda/src/ffi.rs:339-348 (cuda/delta_output.cu:68-91).
 */
int qwc_delta_gated_rmsnorm(const float* input, const void* gate, const void* weight, void* output,
                            int batch, float epsilon, int gate_stride, qwc_stream stream);

/* ------------------------------------------------------------------ */
/* Step glue                                                            */
/* ------------------------------------------------------------------ */

/*
 * QK-norm (1 + w), partial RoPE on the first 64 dims, query -> bf16, K/V of the new token
 * -> e4m3 at (physical_blocks[b], block_offsets[b]).
 * Replaces crates/qwc-cuda/src/ffi.rs:588-604 (cuda/attention_prepare.cu:199-228).
 */
int qwc_prepare_attention_decode_fp8(const void* query_gate_projection, const void* key_projection,
                                     const void* value_projection, const void* query_norm_weight,
                                     const void* key_norm_weight, const void* cosine,
                                     const void* sine, const void* physical_blocks,
                                     const void* block_offsets, void* query, void* key_cache,
                                     void* value_cache, int batch, float epsilon,
                                     qwc_stream stream);

/* Same with per-KV-head scales (values are divided by the scale before the fp8 store) and an
 * explicit page size and projection row strides.  No reference counterpart. */
int qwc_prepare_attention_decode_fp8_scaled(
    const void* query_gate_projection, const void* key_projection, const void* value_projection,
    const void* query_norm_weight, const void* key_norm_weight, const void* cosine,
    const void* sine, const void* physical_blocks, const void* block_offsets,
    const float* key_scales, const float* value_scales, void* query, void* key_cache,
    void* value_cache, int batch, int page_size, int query_stride, int key_stride,
    int value_stride, float epsilon, qwc_stream stream);

/*
 * residual <- bf16(residual + input) when residual != NULL; output = x * rsqrt(mean x^2 + eps)
 * * (1 + w), bf16.  Replaces crates/qwc-cuda/src/ffi.rs:440-449 (cuda/rmsnorm.cu:220-241).
 */
int qwc_rmsnorm_bf16(const void* input, void* residual, const void* weight, void* output, int batch,
                     int hidden, float epsilon, qwc_stream stream);

/* Replaces crates/qwc-cuda/src/ffi.rs:71-80 (cuda/vocab_fp8.cu:702-722). */
int qwc_fp8_embedding_gather(const void* table, const void* row_scales, const void* token_ids,
                             void* output, int batch, int cols, int vocab, qwc_stream stream);

/* logits f32[batch, vocab] = (e4m3 W . bf16 hidden) * row_scale.
 * Replaces crates/qwc-cuda/src/ffi.rs:94-103 and :131-140 (cuda/vocab_fp8.cu:746,823).
 * Both entry points accept batch 1..qwc_fp8_max_batched_logits(). */
int qwc_fp8_lm_head(const void* weights, const void* row_scales, const void* hidden, void* logits,
                    int batch, int hidden_size, int vocab, qwc_stream stream);
int qwc_fp8_lm_head_batched(const void* weights, const void* row_scales, const void* hidden,
                            void* logits, int batch, int hidden_size, int vocab, qwc_stream stream);
/* bf16 rows [rows][cols] -> e4m3 rows with one fp32 scale per row (scale = max|x| / 448, 1 for a zero
 * row), written at rows first_row .. of `output` and `row_scales`: the weight loader's conversion of
 * the vocabulary tables, chunk by chunk.  Replaces crates/qwc-cuda/src/ffi.rs:60-68
 * (cuda/vocab_fp8.cu:681-700). */
int qwc_fp8_quantize_rows(const void* input, void* output, void* row_scales, int rows, int cols,
                          int first_row, qwc_stream stream);
int qwc_fp8_max_logits_batch(void);    /* crates/qwc-cuda/src/ffi.rs:142 */
int qwc_fp8_max_batched_logits(void);  /* crates/qwc-cuda/src/ffi.rs:144 */

/* Greedy argmax, ties -> lower index, NaN never wins.
 * Replaces crates/qwc-cuda/src/ffi.rs:625-634 (cuda/sampling.cu:94-118) behind its signature.  The
 * reference runs two launches through the caller's partial arrays; here one launch (a cluster of
 * eight CTAs per row) does it and partial_values / partial_indices / parts are checked but unused. */
int qwc_argmax(const float* logits, float* partial_values, uint32_t* partial_indices,
               uint32_t* output, int vocab, int batch, int parts, qwc_stream stream);

/* ------------------------------------------------------------------ */
/* Device-side ragged-batch packing (additive; replaces host loops)     */
/* ------------------------------------------------------------------ */

/*
 * Persistent device tables, one entry per state slot:
 *   seq_tokens u32[capacity]            tokens held, including the one this step appends
 *   seq_blocks u32[capacity, max_blocks] physical page ids in logical order
 *
 * qwc_page_table_apply applies `count` host-decided edits (device array of
 * {slot, index, value, kind}: kind 0 sets seq_blocks[slot][index] = value,
 * kind 1 sets seq_tokens[slot] = value, kind 2 adds value to seq_tokens[slot]).
 * It does on the device what CacheManager::append_token / release do to the host maps
 * (crates/qwc-runtime/src/cache.rs:411-449).
 */
typedef struct qwc_table_edit {
    uint32_t slot;
    uint32_t index;
    uint32_t value;
    uint32_t kind;
} qwc_table_edit;

int qwc_page_table_apply(uint32_t* seq_tokens, uint32_t* seq_blocks, const qwc_table_edit* edits,
                         int count, int capacity, int max_blocks, qwc_stream stream);

/*
 * Builds every per-row array the decode step reads, on the device, from the tables above:
 * what BatchLayout::build (crates/qwc-runtime/src/layout.rs:54-152) and
 * Executor::upload_layout_decode (crates/qwc-engine/src/executor.rs:1939-1990) build on the
 * host and upload with eight blocking copies.
 *
 * Row selection: row_slots u32[rows] gives the batch order; or row_slots == NULL and
 * slot_active u8[capacity] != NULL, in which case the rows are the active slots in ascending
 * order (prefix-sum compaction) and *row_count receives their number (<= rows).
 *
 * Outputs (all device): state_slots u32[rows], positions u32[rows], context_lengths u32[rows],
 * physical_blocks u32[rows], block_offsets u32[rows], block_tables u32[rows, max_blocks]
 * (zero padded), block_table_offsets u32[rows + 1] (exclusive prefix sum of page counts),
 * block_ids u32[sum pages] (may be NULL), cosine / sine bf16[rows, 64] gathered from
 * rope_table bf16[max_positions, 2, 64].  status u32[1] receives 0 or the first error
 * (1 slot out of range or empty, 2 duplicate slot, 4 missing pages, 8 position beyond table).
 */
int qwc_pack_decode_batch(const uint32_t* row_slots, const uint8_t* slot_active,
                          const uint32_t* seq_tokens, const uint32_t* seq_blocks,
                          const void* rope_table, int max_positions, uint32_t* row_count,
                          uint32_t* state_slots, uint32_t* positions, uint32_t* context_lengths,
                          uint32_t* physical_blocks, uint32_t* block_offsets,
                          uint32_t* block_tables, uint32_t* block_table_offsets,
                          uint32_t* block_ids, void* cosine, void* sine, uint32_t* status,
                          int rows, int capacity, int max_blocks, int page_size,
                          qwc_stream stream);

#ifdef __cplusplus
}
#endif

#endif /* QWC_ABI_H */
