/*
 * C API of the host side that sits above the kernel ABI (qwc_abi.h): the runtime
 * (cache manager, scheduler, batch layout) and the decode executor.
 *
 * These are the C++ counterparts of the reference's Rust host crates, exposed with plain
 * pointers and integers so that tests, the benchmark and foreign callers can drive them:
 *   qwc_cache_*      crates/qwc-runtime/src/cache.rs      (CacheManager, KvPool, StatePool)
 *   qwc_scheduler_*  crates/qwc-runtime/src/scheduler.rs  (Scheduler)
 *   qwc_layout_*     crates/qwc-runtime/src/layout.rs     (BatchLayout::build)
 *   qwc_engine_*     crates/qwc-engine/src/executor.rs    (Executor: decode path, :878-1112)
 * Error codes are the enum discriminants documented at each function; 0 is success.
 */
#ifndef QWC_ENGINE_H
#define QWC_ENGINE_H

#include <stddef.h>
#include <stdint.h>

#include "qwc_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------------------------- */
/* Cache manager (crates/qwc-runtime/src/cache.rs:300-449,571-594)                     */
/* Rejected: 1 NoStateSlot, 2 NoKvBlocks, 3 AlreadyAdmitted, 4 UnknownSequence,         */
/*           5 NothingToRollback                                                        */
/* ---------------------------------------------------------------------------------- */
typedef struct qwc_cache qwc_cache;

qwc_cache* qwc_cache_new(size_t state_slots, size_t kv_blocks, size_t block_size);
void qwc_cache_free(qwc_cache* cache);
int qwc_cache_admit(qwc_cache* cache, uint32_t id, size_t prompt_tokens);
int qwc_cache_append_token(qwc_cache* cache, uint32_t id);
int qwc_cache_rollback_token(qwc_cache* cache, uint32_t id);
void qwc_cache_release(qwc_cache* cache, uint32_t id);
/* Returns 0 and fills the outputs, or 4 when the sequence is unknown.  `blocks` receives at
 * most `max_blocks` page ids; *num_blocks the real count. */
int qwc_cache_sequence(const qwc_cache* cache, uint32_t id, uint32_t* state_slot, size_t* tokens,
                       uint32_t* blocks, size_t max_blocks, size_t* num_blocks);
/* Prefix cache, bookkeeping only (crates/qwc-runtime/src/cache.rs:193-310, :328-365, :451-569): an
 * entry is a snapshot NUMBER plus references to the KV pages that cover a prompt prefix; the state
 * snapshots themselves would be the executor's.  admit_prompt continues the longest cached proper
 * prefix of at least one page: full pages are shared by reference, an incomplete last page is to be
 * copied (copy_from -> copy_to), the entry stays pinned until finish_restore.  reserve_snapshot
 * returns a free snapshot number (evicting the least valuable unpinned entry when none is free) or
 * -1; commit_snapshot records sequence `id`'s first `num_tokens` tokens under it. */
typedef struct qwc_admission {
    size_t reused;
    int has_restore;
    uint32_t snapshot;
    int copy;
    uint32_t copy_from;
    uint32_t copy_to;
} qwc_admission;
void qwc_cache_enable_prefix_cache(qwc_cache* cache, size_t snapshots);
int qwc_cache_admit_prompt(qwc_cache* cache, uint32_t id, const uint32_t* prompt, size_t prompt_tokens,
                           qwc_admission* admission);
void qwc_cache_finish_restore(qwc_cache* cache, uint32_t snapshot);
long long qwc_cache_reserve_snapshot(qwc_cache* cache);
void qwc_cache_cancel_snapshot(qwc_cache* cache, uint32_t snapshot);
void qwc_cache_commit_snapshot(qwc_cache* cache, uint32_t snapshot, uint32_t id, const uint32_t* tokens,
                               size_t num_tokens);
size_t qwc_cache_prefix_entries(const qwc_cache* cache);
void qwc_cache_prefix_stats(const qwc_cache* cache, uint64_t* lookups_hits_reused_evictions);
size_t qwc_cache_free_blocks(const qwc_cache* cache);
size_t qwc_cache_states_in_use(const qwc_cache* cache);
size_t qwc_cache_active(const qwc_cache* cache);
/* need / free of the last NoKvBlocks rejection */
void qwc_cache_last_shortage(const qwc_cache* cache, size_t* need, size_t* free_blocks);
/* Moves the table edits recorded since the last call into `edits` (at most `max_edits`);
 * returns how many were pending. */
size_t qwc_cache_drain_edits(qwc_cache* cache, qwc_table_edit* edits, size_t max_edits);

/* ---------------------------------------------------------------------------------- */
/* Scheduler (crates/qwc-runtime/src/scheduler.rs:190-668)                              */
/* SubmitError: 1 Duplicate, 2 EmptyPrompt, 3 NoOutputTokens, 4 NoStateCapacity,         */
/*              5 ContextTooLong                                                         */
/* SchedulerError: 1 BatchInFlight, 2 NoBatchInFlight, 3 SequenceInFlight,               */
/*                 4 InvalidStopped, 5 DuplicateStopped, 6 Invariant, 7 Cache            */
/* ---------------------------------------------------------------------------------- */
typedef struct qwc_scheduler qwc_scheduler;

typedef struct qwc_prefill_chunk {
    uint32_t id;
    uint32_t offset;
    uint32_t tokens;
} qwc_prefill_chunk;

typedef struct qwc_completion {
    uint32_t id;
    uint32_t generated_tokens;
    uint32_t reason; /* 0 Length, 1 Stopped */
} qwc_completion;

qwc_scheduler* qwc_scheduler_new(size_t max_num_seqs, size_t max_num_batched_tokens, size_t state_slots,
                                 size_t kv_blocks, size_t block_size);
void qwc_scheduler_free(qwc_scheduler* scheduler);
int qwc_scheduler_submit(qwc_scheduler* scheduler, uint32_t id, size_t prompt_tokens, size_t max_new_tokens);
/* Plans the next batch.  Returns 0 with the batch (possibly empty: *num_decode == 0 and
 * *num_prefill == 0 means nothing to run), or a SchedulerError.  Buffers must hold
 * max_num_seqs entries. */
int qwc_scheduler_next_batch(qwc_scheduler* scheduler, uint32_t* decode_ids, size_t* num_decode,
                             qwc_prefill_chunk* prefill, size_t* num_prefill);
int qwc_scheduler_complete_batch(qwc_scheduler* scheduler, const uint32_t* stopped, size_t num_stopped,
                                 qwc_completion* completed, size_t max_completed, size_t* num_completed);
/* The same for steps in which decode sequences may have produced more than one token
 * (Scheduler::complete_batch_multi, crates/qwc-runtime/src/scheduler.rs:392-500): `produced_tokens[i]`
 * tokens for sequence `produced_ids[i]`; sequences not named count one; zero tokens -> Invariant, a
 * sequence that is not in the batch's decode list -> InvalidStopped. */
int qwc_scheduler_complete_batch_multi(qwc_scheduler* scheduler, const uint32_t* stopped, size_t num_stopped,
                                       const uint32_t* produced_ids, const uint32_t* produced_tokens,
                                       size_t num_produced, qwc_completion* completed, size_t max_completed,
                                       size_t* num_completed);
/* Prefix cache through the scheduler (crates/qwc-runtime/src/scheduler.rs:52-68, :226-261).  A request
 * submitted with its prompt tokens can continue a cached prefix and leave its own: the prefill chunk is
 * cut at `snapshot_at` (the history boundary), and the batch then carries a save op; an admitted request
 * that continues a prefix carries a restore op with its first chunk.  prompt_tokens must equal the
 * request's prompt length and snapshot_at must not exceed it (SubmitError 2 otherwise). */
typedef struct qwc_prefix_restore_op {
    uint32_t id;
    uint32_t state_slot;
    uint32_t snapshot;
    uint32_t copy; /* 1: copy page copy_from into copy_to before the step (the prefix ends inside a page) */
    uint32_t copy_from;
    uint32_t copy_to;
} qwc_prefix_restore_op;

typedef struct qwc_prefix_save_op {
    uint32_t id;
    uint32_t state_slot;
    uint32_t snapshot;
} qwc_prefix_save_op;

void qwc_scheduler_enable_prefix_cache(qwc_scheduler* scheduler, size_t snapshots);
int qwc_scheduler_submit_prompt(qwc_scheduler* scheduler, uint32_t id, const uint32_t* prompt, size_t prompt_tokens,
                                size_t max_new_tokens, size_t snapshot_at);
/* The prefix work of the batch in flight (restore before the pass, capture inside it after the chunk's
 * scan).  Buffers must hold max_num_seqs entries; SchedulerError 2 when no batch is in flight. */
int qwc_scheduler_batch_prefix_ops(const qwc_scheduler* scheduler, qwc_prefix_restore_op* restores,
                                   size_t* num_restores, qwc_prefix_save_op* saves, size_t* num_saves);
int qwc_scheduler_abort_batch(qwc_scheduler* scheduler);
/* *removed receives 1 when the request existed. */
int qwc_scheduler_cancel(qwc_scheduler* scheduler, uint32_t id, int* removed);
/* -1 when the request is not active */
long long qwc_scheduler_remaining_tokens(const qwc_scheduler* scheduler, uint32_t id);
size_t qwc_scheduler_waiting(const qwc_scheduler* scheduler);
size_t qwc_scheduler_active(const qwc_scheduler* scheduler);
size_t qwc_scheduler_committed_kv_blocks(const qwc_scheduler* scheduler);
/* The scheduler's own cache manager (borrowed; do not free). */
qwc_cache* qwc_scheduler_cache(qwc_scheduler* scheduler);

/* ---------------------------------------------------------------------------------- */
/* Batch layout (crates/qwc-runtime/src/layout.rs:54-152)                               */
/* LayoutError: 1 MissingSequence, 2 DuplicateSequence, 3 InvalidPrefillRange,           */
/*              4 MissingKvBlocks, 5 IntegerOverflow                                     */
/* ---------------------------------------------------------------------------------- */
/* Builds the CSR metadata of a batch on the host.  Output arrays must hold num_decode +
 * num_prefill (+1 for the two offset arrays) entries; block_ids `max_block_ids`.
 * *offender receives the sequence id an error refers to. */
int qwc_layout_build(const qwc_cache* cache, const uint32_t* decode_ids, size_t num_decode,
                     const qwc_prefill_chunk* prefill, size_t num_prefill, uint32_t* seq_ids,
                     uint32_t* state_slots, uint32_t* position_starts, uint32_t* context_lens,
                     uint32_t* token_offsets, uint32_t* block_table_offsets, uint32_t* block_ids,
                     size_t max_block_ids, uint32_t* offender);

/* ---------------------------------------------------------------------------------- */
/* Decode executor (crates/qwc-engine/src/executor.rs:395-546,878-1112,1774-1990)        */
/* ---------------------------------------------------------------------------------- */
typedef struct qwc_engine qwc_engine;

typedef struct qwc_engine_config {
    int num_layers;              /* 64; every `full_attention_interval`-th layer is full attention */
    int full_attention_interval; /* 4 */
    int hidden;                  /* 5120 */
    int intermediate;            /* 17408 */
    int vocab;                   /* 151936 */
    int delta_value_heads;       /* 32 (reference checkpoint: 48) */
    int kv_page_size;            /* 16 (reference: 64) */
    int max_batch;               /* rows of the largest step; one CUDA graph per batch size */
    int max_context;             /* per-sequence context cap; sets the block-table width */
    int kv_pool_blocks;          /* physical KV pages shared by all sequences */
    int state_slots;             /* DeltaNet state slots */
    unsigned long long seed;     /* synthetic weights and caches */
    int split_rank;              /* column split of every projection (latency mode): this rank */
    int split_size;              /* ... of this many; 1 = off.  Needs max_batch == 1. */
    int use_graph;               /* 1: replay a captured graph per batch size (default path) */
    int attention_partitions;    /* 0 = choose from max_batch and max_context */
    int write_logits;            /* 1: the vocabulary head also stores fp32 logits (tensor "logits"); 0: tokens only */
    int exchange;                /* latency mode: 0 = every projection's output gathered by ncclAllGather
                                    (qwc_engine_init_split), 1 = fused: projections store their partial sums
                                    into every rank's memory and the consumers sum them
                                    (qwc_engine_exchange_handle / qwc_engine_open_peers).  Needs max_batch == 1;
                                    with split_size 1 the rank exchanges with itself (tests). */
    unsigned long long memory_limit; /* ceiling in bytes for the engine's device allocations, 0 = none
                                    (set_memory_limit, crates/qwc-cuda/src/memory.rs:31-58): clipped to the
                                    device's free memory less 512 MiB; an allocation that would pass it is
                                    refused BEFORE cudaMalloc with cudaErrorMemoryAllocation (2) and
                                    qwc_engine_create frees what it had taken */
} qwc_engine_config;

/* ---- memory plan (crates/qwc-core/src/memory.rs:99-218, crates/qwc-runtime/src/cache.rs:360-378,
 *      :596-622): what a sequence costs, what a GPU has left for the two pools, pools sized for a
 *      target context.  Host arithmetic only. ---- */
typedef struct qwc_cache_geometry {
    uint64_t kv_bytes_per_token;   /* e4m3 K and V of every full-attention layer */
    uint64_t state_bytes_per_slot; /* int8 state rows + fp32 row scales + fp32 convolution window */
    size_t block_size;             /* tokens per KV page */
} qwc_cache_geometry;

typedef struct qwc_budget {
    uint64_t total_vram;
    uint64_t reserved;  /* context, driver, other processes */
    uint64_t weights;
    uint64_t workspace; /* activations, exchange blocks, graphs */
} qwc_budget;

void qwc_cache_geometry_for(const qwc_engine_config* config, qwc_cache_geometry* geometry);
/* Resident weight bytes of the engine this config describes (this rank's share under a column split):
 * NVFP4 nibbles and block scales of every projection, the two e4m3 vocabulary tables with their row
 * scales, the bf16 norms and gates. */
uint64_t qwc_engine_weight_bytes(const qwc_engine_config* config);
/* One B200: 183 359 MiB, 1 GiB reserved. */
void qwc_budget_b200(uint64_t weights, uint64_t workspace, qwc_budget* budget);
uint64_t qwc_budget_cache_available(const qwc_budget* budget);
size_t qwc_budget_max_concurrency(const qwc_budget* budget, const qwc_cache_geometry* geometry, size_t context);
size_t qwc_budget_max_context(const qwc_budget* budget, const qwc_cache_geometry* geometry, size_t concurrency);
int qwc_budget_fits(const qwc_budget* budget, const qwc_cache_geometry* geometry, size_t concurrency,
                    size_t context);
size_t qwc_cache_geometry_crossover_tokens(const qwc_cache_geometry* geometry);
/* CacheManager::from_budget: as many state slots as sequences of `target_context` fit, the rest as
 * KV pages.  Free with qwc_cache_free. */
qwc_cache* qwc_cache_from_budget(const qwc_budget* budget, const qwc_cache_geometry* geometry,
                                 size_t target_context);
size_t qwc_cache_state_capacity(const qwc_cache* cache);
size_t qwc_cache_kv_capacity(const qwc_cache* cache);
/* Utilisation of the two pools in [0, 1]; the larger one is the bottleneck (Pressure). */
void qwc_cache_pressure(const qwc_cache* cache, double* states, double* kv);

/* Fills `config` with the synthetic 27B-shaped model of the benchmark. */
void qwc_engine_default_config(qwc_engine_config* config);

/* Allocates every resident buffer, generates seeded synthetic weights, KV pages and
 * DeltaNet state on the device.  Returns a cudaError_t. */
int qwc_engine_create(const qwc_engine_config* config, qwc_engine** engine);
void qwc_engine_destroy(qwc_engine* engine);
/* Bytes the engine asked for so far and its ceiling, 0 when it has none (memory_usage,
 * crates/qwc-cuda/src/memory.rs:73-78; requested bytes, not what the driver rounded them to). */
void qwc_engine_memory_usage(const qwc_engine* engine, size_t* used, size_t* limit);

/* Joins a NCCL communicator for the column-split mode.  `unique_id` is the 128-byte
 * ncclUniqueId made by rank 0 (qwc_engine_nccl_unique_id) and distributed by the caller.
 * Returns 0, or a negative code when libnccl cannot be loaded / initialised. */
int qwc_engine_nccl_unique_id(void* unique_id_128);
int qwc_engine_init_split(qwc_engine* engine, const void* unique_id_128);

/* Fused latency mode (config.exchange = 1): every rank exports the 64-byte inter-process handle of
 * its exchange block, the caller distributes them (any host channel), and every rank maps the
 * others' blocks with `handles` = split_size handles in rank order (its own entry is ignored).  The
 * ranks must be processes on one node whose GPUs have peer access.  Until the peers are open a step
 * returns cudaErrorNotReady.  In this mode the step uses no library collective; every rank stores the
 * same sampled token; "logits" holds this rank's vocab / split_size columns only. */
int qwc_engine_exchange_handle(qwc_engine* engine, void* handle_64);
int qwc_engine_open_peers(qwc_engine* engine, const void* handles, int count);
/* Measurement aid of the fused latency mode: for each exchange of the step (in step order; 1024
 * entries) the longest time, in nanoseconds, that a consumer thread of this rank has waited for a
 * peer's word since the last call; reads and clears (synchronises the engine's stream). */
int qwc_engine_exchange_waits(qwc_engine* engine, unsigned long long* nanoseconds, int capacity);
/* Turns that bookkeeping on or off (off by default: it costs an atomic per word that was waited for,
 * enough to lengthen the waits; never on in a timed run).  Captured graphs are dropped and rebuilt. */
int qwc_engine_profile_waits(qwc_engine* engine, int enable);

/* Device pointer and size of a named resident tensor, for tests that read weights and
 * caches back.  Layer-indexed names take the layer number; others ignore it.  Returns 0 or 1. */
int qwc_engine_tensor(qwc_engine* engine, const char* name, int layer, void** device_ptr, size_t* bytes);

/* Test aid: with `enable` != 0 every later step also copies, per layer, the mixer's output
 * projection and the residual stream after the MLP into the tensor "trace"
 * (bf16 [num_layers][2][max_batch][hidden]); 0 turns it off again.  Captured graphs are dropped
 * either way (the next step of each batch size is captured anew). */
int qwc_engine_trace_layers(qwc_engine* engine, int enable);

/* Synchronous copies of a named tensor to / from host memory (`bytes` must equal its size). */
/* The fp32 global divisor of an NVFP4 matrix ("gate", "up", "down", "in_proj", "la_out", "qkv", "o"):
 * synthetic weights carry 1; a weight loader sets the checkpoint's weight_global_scale
 * (crates/qwc-engine/src/weights.rs:470-476).  Setting it drops the captured graphs. */
int qwc_engine_set_weight_global_scale(qwc_engine* engine, const char* name, int layer, float value);
int qwc_engine_weight_global_scale(qwc_engine* engine, const char* name, int layer, float* value);
int qwc_engine_read(qwc_engine* engine, const char* name, int layer, void* host, size_t bytes);
int qwc_engine_write(qwc_engine* engine, const char* name, int layer, const void* host, size_t bytes);

/* Bytes the decode step must move for `rows` rows with the given total context tokens:
 * weights, DeltaNet state read+write, KV read.  The roofline numerator. */
typedef struct qwc_step_traffic {
    double weight_bytes;
    double state_bytes;
    double kv_bytes;
    double gemv_bytes_per_step; /* NVFP4 projection weights only (the dominant kernel) */
    int gemv_launches_per_step;
    int kernel_launches_per_step;
} qwc_step_traffic;
void qwc_engine_traffic(const qwc_engine* engine, int rows, double context_tokens, qwc_step_traffic* out);

/* Applies table edits (host array) to the device page table: one H2D copy and one kernel.  The edits
 * are bounded on the host first (here and in qwc_engine_decode): a slot beyond the state pool, a table
 * index beyond max_context, a page id beyond the KV pool or an unknown kind is refused with
 * cudaErrorInvalidValue and nothing of the drain is applied - every page id the attention kernels
 * follow came through here. */
int qwc_engine_apply_edits(qwc_engine* engine, const qwc_table_edit* edits, size_t count);

/* Copies KV page `from` onto page `to` in every full-attention layer, asynchronously on the engine's
 * stream (Executor::copy_kv_block, crates/qwc-engine/src/executor.rs:825-835): a sequence that
 * continues a cached prefix ending inside a page appends to a copy of that page
 * (qwc_prefix_restore_op.copy_from / copy_to).  cudaErrorInvalidValue for a page outside the pool. */
int qwc_engine_copy_kv_block(qwc_engine* engine, uint32_t from, uint32_t to);

/*
 * One decode step for `rows` rows.  Host inputs: row_slots u32[rows] (batch order),
 * tokens u32[rows], optional table edits to apply first.  Copies them to the device, packs
 * the ragged batch on the device, runs the 64-layer step (graph replay), and copies the
 * greedy tokens back into sampled u32[rows].  Synchronous.  Mirrors
 * Executor::execute_layout for a pure-decode layout (executor.rs:878-905,947-951).
 * Returns a cudaError_t; a packing error (status word of qwc_pack_decode_batch) is returned
 * as 0x1000 + status, and a bounded device-side wait that gave up or a state slot beyond the
 * pool (the sticky word of qwc_device_status, which the step copies back with its tokens) as
 * 0x4000 + status: such a step has skipped stores and its tokens must not be committed
 * (qwc_worker_step rolls the batch back).
 */
int qwc_engine_decode(qwc_engine* engine, const uint32_t* row_slots, const uint32_t* tokens,
                      const qwc_table_edit* edits, size_t num_edits, int rows, uint32_t* sampled);

/* Same step with inputs already resident (the arrays of the previous call are reused) and no
 * copies: only the graph replay.  For device-only timing. */
int qwc_engine_replay(qwc_engine* engine, int rows);
/* The stream the engine works on (cudaStream_t), for event timing by the caller. */
qwc_stream qwc_engine_stream(qwc_engine* engine);

/* Event timeline of one eager (un-captured) step, as Timeline / Executor::mark
 * (crates/qwc-cuda/src/timeline.rs:17-77, executor.rs:586-591): per phase label the summed
 * milliseconds and launch count.  Returns the number of phases written. */
typedef struct qwc_phase_time {
    char label[24];
    float milliseconds;
    int launches;
} qwc_phase_time;
int qwc_engine_profile_step(qwc_engine* engine, int rows, qwc_phase_time* phases, int max_phases);

/* Graph-timed cost of a subset of the step: captures a CUDA graph of only the phases whose label
 * starts with `label_prefix` ("gemm.", "attn.decode", "delta.scan", "norm", ...; "" = the whole
 * step), on the buffers the last real step left on the device, replays it `replays` times between
 * two events and returns the mean milliseconds per replay and the phases it launched.  The eager
 * timeline above includes host launch gaps; this does not.  The selected kernels run on stale
 * activations, so the recurrent state and the KV pages they write are garbage afterwards: call it
 * after the measurements that need them.  Needs one real step of `rows` rows beforehand. */
int qwc_engine_time_phases(qwc_engine* engine, int rows, const char* label_prefix, int replays,
                           float* milliseconds, int* launches);

/*
 * One iteration of the serving worker loop (crates/qwc-engine/src/bin/serve.rs:806-1074,
 * decode part): scheduler.next_batch -> layout check -> table edits -> decode step ->
 * scheduler.complete_batch.  Prefill chunks are accounted but not computed (the synthetic
 * caches already hold data for the prompt).  On any error before or at the launch the batch
 * is rolled back with abort_batch.  *num_decoded receives the rows decoded, `completed` the
 * finished requests.  Returns 0, 0x2000 + SchedulerError, 0x3000 + LayoutError or a
 * cudaError_t.
 */
int qwc_worker_step(qwc_engine* engine, qwc_scheduler* scheduler, uint32_t eos_token, size_t* num_decoded,
                    qwc_completion* completed, size_t max_completed, size_t* num_completed);

/* ---------------------------------------------------------------------------------- */
/* Worker loop at token level (crates/qwc-engine/src/bin/serve.rs:777-1074, :1133-1156,  */
/* :1339-1368, :1438-1442): commands in, plan, layout, one executor call per step, token  */
/* emission with the stop rules, completion, rollback and fail-all on an error,           */
/* cancellation of abandoned jobs.  Text (tokenizer, stop strings) and the speculative    */
/* branch are the caller's: the token callback's return value says "stop here".           */
/* ---------------------------------------------------------------------------------- */
typedef struct qwc_worker qwc_worker;

/* What a step hands to its executor.  Layout arrays as BatchLayout (layout.rs:54-152): decode rows
 * first; tokens[token_offsets[i] .. token_offsets[i+1]) are the input tokens of sequence i (a decode
 * row: the token sampled by the previous step; a prefill chunk: its slice of the prompt). */
typedef struct qwc_step_view {
    size_t num_sequences;
    size_t num_decode;
    const uint32_t* seq_ids;
    const uint32_t* state_slots;
    const uint32_t* position_starts;
    const uint32_t* context_lens;
    const uint32_t* token_offsets;       /* num_sequences + 1 */
    const uint32_t* block_table_offsets; /* num_sequences + 1 */
    const uint32_t* block_ids;
    size_t num_block_ids;
    const uint32_t* tokens;
    size_t num_tokens;
    const qwc_table_edit* edits; /* page-table edits the plan produced, to apply before the step */
    size_t num_edits;
    const qwc_prefix_restore_op* restores;
    size_t num_restores;
    const qwc_prefix_save_op* saves;
    size_t num_saves;
} qwc_step_view;

/* Runs the step and writes one sampled token per sequence, layout order.  0, or an error code with
 * which the worker fails: nothing of such a step is committed (the plan is rolled back). */
typedef int (*qwc_execute_fn)(void* user, const qwc_step_view* step, uint32_t* sampled);
/* kind 0 Token (value = token; a non-zero return stops the sequence after it), 1 Done (value = tokens
 * emitted, reason 0 Length / 1 Stopped), 2 Error (value = the code the worker failed with, or
 * 0x5000 + SubmitError for a refused request). */
typedef int (*qwc_event_fn)(void* user, uint32_t id, uint32_t kind, uint32_t value, uint32_t reason);

qwc_worker* qwc_worker_new(qwc_scheduler* scheduler, qwc_execute_fn execute, void* execute_user, qwc_event_fn event,
                           void* event_user, const uint32_t* eos_ids, size_t num_eos);
/* Free only after qwc_worker_run has returned (and no other thread still calls into the worker); the
 * scheduler is borrowed and outlives the worker. */
void qwc_worker_free(qwc_worker* worker);
/* Thread-safe: queue a request / tell the worker that nobody listens to a request any more / tell it
 * that no more commands will come (qwc_worker_run then returns once its jobs are finished). */
void qwc_worker_submit(qwc_worker* worker, uint32_t id, const uint32_t* prompt, size_t prompt_tokens,
                       size_t max_new_tokens, size_t history_tokens, int ignore_eos);
void qwc_worker_abandon(qwc_worker* worker, uint32_t id);
void qwc_worker_shutdown(qwc_worker* worker);
/* One pass of the loop body (*progressed = 1 when a step ran) / the loop itself.  0, or the code the
 * worker failed with: 0x2000 + SchedulerError, 0x3000 + LayoutError, 0x5100 a decode row without a
 * sampled token, 0x5101 a prefill chunk without its prompt, 0x5102 an executor that returned too few
 * tokens, or the executor's own code.  A failed worker has sent Error to every job and stays failed. */
int qwc_worker_iterate(qwc_worker* worker, int* progressed);
int qwc_worker_run(qwc_worker* worker);
size_t qwc_worker_jobs(const qwc_worker* worker);
uint64_t qwc_worker_steps(const qwc_worker* worker);
uint64_t qwc_worker_aborted_steps(const qwc_worker* worker);

/* A qwc_execute_fn over the GPU engine (`user` = the qwc_engine*): decode rows run the decode step
 * (qwc_engine_decode); a prefill chunk is accounted, not computed (the synthetic caches already hold
 * data for the prompt) and samples a token derived from its sequence id; of the prefix ops the page
 * copies of the restores are executed (qwc_engine_copy_kv_block), the state snapshots, which belong to
 * the prefill pass, are not.  Error codes as qwc_engine_decode. */
int qwc_engine_execute_step(void* engine, const qwc_step_view* step, uint32_t* sampled);

#ifdef __cplusplus
}
#endif

#endif /* QWC_ENGINE_H */
