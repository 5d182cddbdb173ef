// C entry points of the host runtime (include/qwc_engine.h, cache / scheduler / layout part).
#include <algorithm>
#include <cstring>

#include "../../../include/qwc_engine.h"
#include "runtime.h"
#include "runtime_handles.h"

using namespace qwc::runtime;

extern "C" {

qwc_cache* qwc_cache_new(size_t state_slots, size_t kv_blocks, size_t block_size) {
    if (block_size == 0) {
        return nullptr;
    }
    auto* handle = new qwc_cache;
    handle->owned.reset(new CacheManager(state_slots, kv_blocks, block_size));
    handle->cache = handle->owned.get();
    return handle;
}

void qwc_cache_free(qwc_cache* cache) {
    if (cache != nullptr && cache->owned) {
        delete cache;
    }
}

int qwc_cache_admit(qwc_cache* cache, uint32_t id, size_t prompt_tokens) {
    return static_cast<int>(cache->cache->admit(id, prompt_tokens));
}

int qwc_cache_append_token(qwc_cache* cache, uint32_t id) { return static_cast<int>(cache->cache->append_token(id)); }

int qwc_cache_rollback_token(qwc_cache* cache, uint32_t id) {
    return static_cast<int>(cache->cache->rollback_token(id));
}

void qwc_cache_release(qwc_cache* cache, uint32_t id) { cache->cache->release(id); }

int qwc_cache_sequence(const qwc_cache* cache, uint32_t id, uint32_t* state_slot, size_t* tokens, uint32_t* blocks,
                       size_t max_blocks, size_t* num_blocks) {
    const Sequence* seq = cache->cache->sequence(id);
    if (seq == nullptr) {
        return static_cast<int>(Rejected::UnknownSequence);
    }
    if (state_slot != nullptr) {
        *state_slot = seq->state_slot;
    }
    if (tokens != nullptr) {
        *tokens = seq->tokens;
    }
    if (num_blocks != nullptr) {
        *num_blocks = seq->blocks.size();
    }
    if (blocks != nullptr) {
        std::copy_n(seq->blocks.begin(), std::min(max_blocks, seq->blocks.size()), blocks);
    }
    return 0;
}

// ---- prefix cache (cache.rs:328-365, :451-569) ----
void qwc_cache_enable_prefix_cache(qwc_cache* cache, size_t snapshots) { cache->cache->enable_prefix_cache(snapshots); }

int qwc_cache_admit_prompt(qwc_cache* cache, uint32_t id, const uint32_t* prompt, size_t prompt_tokens,
                           qwc_admission* admission) {
    Admission result;
    const Rejected rejected =
        cache->cache->admit_prompt(id, std::vector<uint32_t>(prompt, prompt + prompt_tokens), &result);
    if (admission != nullptr) {
        admission->reused = result.reused;
        admission->has_restore = result.has_restore ? 1 : 0;
        admission->snapshot = result.restore.snapshot;
        admission->copy = result.restore.copy ? 1 : 0;
        admission->copy_from = result.restore.copy_from;
        admission->copy_to = result.restore.copy_to;
    }
    return static_cast<int>(rejected);
}

void qwc_cache_finish_restore(qwc_cache* cache, uint32_t snapshot) { cache->cache->finish_restore(snapshot); }

long long qwc_cache_reserve_snapshot(qwc_cache* cache) {
    const std::optional<uint32_t> snapshot = cache->cache->reserve_snapshot();
    return snapshot ? static_cast<long long>(*snapshot) : -1;
}

void qwc_cache_cancel_snapshot(qwc_cache* cache, uint32_t snapshot) { cache->cache->cancel_snapshot(snapshot); }

void qwc_cache_commit_snapshot(qwc_cache* cache, uint32_t snapshot, uint32_t id, const uint32_t* tokens,
                               size_t num_tokens) {
    cache->cache->commit_snapshot(snapshot, id, std::vector<uint32_t>(tokens, tokens + num_tokens));
}

size_t qwc_cache_prefix_entries(const qwc_cache* cache) { return cache->cache->prefix_entries(); }

void qwc_cache_prefix_stats(const qwc_cache* cache, uint64_t* lookups_hits_reused_evictions) {
    const PrefixStats& stats = cache->cache->prefix_stats();
    lookups_hits_reused_evictions[0] = stats.lookups;
    lookups_hits_reused_evictions[1] = stats.hits;
    lookups_hits_reused_evictions[2] = stats.reused_tokens;
    lookups_hits_reused_evictions[3] = stats.evictions;
}

size_t qwc_cache_free_blocks(const qwc_cache* cache) { return cache->cache->kv().free_blocks(); }
size_t qwc_cache_states_in_use(const qwc_cache* cache) { return cache->cache->states().in_use(); }
size_t qwc_cache_active(const qwc_cache* cache) { return cache->cache->active(); }

void qwc_cache_last_shortage(const qwc_cache* cache, size_t* need, size_t* free_blocks) {
    *need = cache->cache->last_need();
    *free_blocks = cache->cache->last_free();
}

size_t qwc_cache_drain_edits(qwc_cache* cache, qwc_table_edit* edits, size_t max_edits) {
    static_assert(sizeof(qwc_table_edit) == sizeof(TableEdit), "edit layouts must match");
    const std::vector<TableEdit> pending = cache->cache->drain_edits();
    const size_t n = std::min(max_edits, pending.size());
    if (n > 0 && edits != nullptr) {
        std::memcpy(edits, pending.data(), n * sizeof(TableEdit));
    }
    return pending.size();
}

namespace {

CacheGeometry geometry_of(const qwc_cache_geometry* g) {
    CacheGeometry geometry;
    geometry.kv_bytes_per_token = g->kv_bytes_per_token;
    geometry.state_bytes_per_slot = g->state_bytes_per_slot;
    geometry.block_size = g->block_size ? g->block_size : 1;
    return geometry;
}

Budget budget_of(const qwc_budget* b) { return Budget{b->total_vram, b->reserved, b->weights, b->workspace}; }

// NVFP4 matrix as the engine keeps it: nibbles, and e4m3 block scales in the 128 x 4 swizzle (rows
// padded to 128, 16-wide blocks padded to 4).
uint64_t nvfp4_bytes(uint64_t rows, uint64_t cols) {
    const uint64_t padded_rows = (rows + 127) / 128 * 128;
    const uint64_t padded_blocks = (cols / 16 + 3) / 4 * 4;
    return rows * cols / 2 + padded_rows * padded_blocks;
}

}  // namespace

void qwc_cache_geometry_for(const qwc_engine_config* config, qwc_cache_geometry* out) {
    const size_t attention = static_cast<size_t>(config->num_layers / config->full_attention_interval);
    const CacheGeometry geometry =
        CacheGeometry::for_model(static_cast<size_t>(config->num_layers) - attention, attention,
                                 static_cast<size_t>(config->delta_value_heads), static_cast<size_t>(config->kv_page_size));
    *out = {geometry.kv_bytes_per_token, geometry.state_bytes_per_slot, geometry.block_size};
}

uint64_t qwc_engine_weight_bytes(const qwc_engine_config* c) {
    const uint64_t split = static_cast<uint64_t>(c->split_size > 0 ? c->split_size : 1);
    const uint64_t hidden = c->hidden, inter = c->intermediate, heads = c->delta_value_heads, vocab = c->vocab;
    const uint64_t attention = c->num_layers / c->full_attention_interval;
    const uint64_t linear = c->num_layers - attention;
    const uint64_t channels = 2 * 16 * 128 + heads * 128;
    const uint64_t mixer_width = channels + heads * 128 + 2 * heads;  // q|k|v, z, a, b
    const uint64_t qkv_width = 24 * 2 * 256 + 2 * 4 * 256;
    // a column split keeps N / split rows of every projection on a rank; the K-side matrices
    // (down, out, o) are split the same way
    uint64_t per_layer = 2 * nvfp4_bytes(inter / split, hidden) + nvfp4_bytes(hidden / split, inter) + 2 * hidden * 2;
    uint64_t per_linear = nvfp4_bytes(mixer_width / split, hidden) + nvfp4_bytes(hidden / split, heads * 128) +
                          (channels * 4 + 2 * heads + 128) * 2;
    uint64_t per_attention = nvfp4_bytes(qkv_width / split, hidden) + nvfp4_bytes(hidden / split, 24 * 256) +
                             2 * 256 * 2 + 2 * 4 * 4;
    const uint64_t tables = vocab * hidden + 4 * vocab + (vocab / split) * hidden + 4 * (vocab / split);
    return c->num_layers * per_layer + linear * per_linear + attention * per_attention + tables + hidden * 2;
}

void qwc_budget_b200(uint64_t weights, uint64_t workspace, qwc_budget* out) {
    const Budget budget = Budget::b200(weights, workspace);
    *out = {budget.total_vram, budget.reserved, budget.weights, budget.workspace};
}

uint64_t qwc_budget_cache_available(const qwc_budget* budget) { return budget_of(budget).cache_available(); }

size_t qwc_budget_max_concurrency(const qwc_budget* budget, const qwc_cache_geometry* geometry, size_t context) {
    return budget_of(budget).max_concurrency(geometry_of(geometry), context);
}

size_t qwc_budget_max_context(const qwc_budget* budget, const qwc_cache_geometry* geometry, size_t concurrency) {
    return budget_of(budget).max_context(geometry_of(geometry), concurrency);
}

int qwc_budget_fits(const qwc_budget* budget, const qwc_cache_geometry* geometry, size_t concurrency,
                    size_t context) {
    return budget_of(budget).fits(geometry_of(geometry), concurrency, context) ? 1 : 0;
}

size_t qwc_cache_geometry_crossover_tokens(const qwc_cache_geometry* geometry) {
    return geometry_of(geometry).crossover_tokens();
}

qwc_cache* qwc_cache_from_budget(const qwc_budget* budget, const qwc_cache_geometry* geometry,
                                 size_t target_context) {
    auto* handle = new qwc_cache;
    handle->owned = std::make_unique<CacheManager>(
        CacheManager::from_budget(budget_of(budget), geometry_of(geometry), target_context));
    handle->cache = handle->owned.get();
    return handle;
}

size_t qwc_cache_state_capacity(const qwc_cache* cache) { return cache->cache->states().capacity(); }
size_t qwc_cache_kv_capacity(const qwc_cache* cache) { return cache->cache->kv().capacity(); }

void qwc_cache_pressure(const qwc_cache* cache, double* states, double* kv) {
    const Pressure pressure = cache->cache->pressure();
    *states = pressure.states;
    *kv = pressure.kv;
}

qwc_scheduler* qwc_scheduler_new(size_t max_num_seqs, size_t max_num_batched_tokens, size_t state_slots,
                                 size_t kv_blocks, size_t block_size) {
    if (max_num_seqs == 0 || max_num_batched_tokens == 0 || block_size == 0) {
        return nullptr;  // SchedulerConfig::new asserts both limits are positive
    }
    auto* handle = new qwc_scheduler{
        Scheduler(SchedulerConfig{max_num_seqs, max_num_batched_tokens}, CacheManager(state_slots, kv_blocks, block_size)),
        {}};
    handle->cache_view.cache = &handle->scheduler.cache_mut();
    return handle;
}

void qwc_scheduler_free(qwc_scheduler* scheduler) { delete scheduler; }

int qwc_scheduler_submit(qwc_scheduler* scheduler, uint32_t id, size_t prompt_tokens, size_t max_new_tokens) {
    return static_cast<int>(scheduler->scheduler.submit(Request{id, prompt_tokens, max_new_tokens}));
}

int qwc_scheduler_next_batch(qwc_scheduler* scheduler, uint32_t* decode_ids, size_t* num_decode,
                             qwc_prefill_chunk* prefill, size_t* num_prefill) {
    Batch batch;
    bool has_batch = false;
    *num_decode = 0;
    *num_prefill = 0;
    const SchedulerError error = scheduler->scheduler.next_batch(&batch, &has_batch);
    if (error != SchedulerError::None || !has_batch) {
        return static_cast<int>(error);
    }
    *num_decode = batch.decode.size();
    *num_prefill = batch.prefill.size();
    std::copy(batch.decode.begin(), batch.decode.end(), decode_ids);
    for (size_t i = 0; i < batch.prefill.size(); ++i) {
        prefill[i] = {batch.prefill[i].id, static_cast<uint32_t>(batch.prefill[i].offset),
                      static_cast<uint32_t>(batch.prefill[i].tokens)};
    }
    return 0;
}

int qwc_scheduler_complete_batch(qwc_scheduler* scheduler, const uint32_t* stopped, size_t num_stopped,
                                 qwc_completion* completed, size_t max_completed, size_t* num_completed) {
    std::vector<SeqId> stopped_ids(stopped, stopped + num_stopped);
    std::vector<Completion> done;
    const SchedulerError error = scheduler->scheduler.complete_batch(stopped_ids, &done);
    *num_completed = done.size();
    for (size_t i = 0; i < done.size() && i < max_completed; ++i) {
        completed[i] = {done[i].id, static_cast<uint32_t>(done[i].generated_tokens),
                        static_cast<uint32_t>(done[i].reason)};
    }
    return static_cast<int>(error);
}

int qwc_scheduler_complete_batch_multi(qwc_scheduler* scheduler, const uint32_t* stopped, size_t num_stopped,
                                       const uint32_t* produced_ids, const uint32_t* produced_tokens,
                                       size_t num_produced, qwc_completion* completed, size_t max_completed,
                                       size_t* num_completed) {
    std::vector<SeqId> stopped_ids(stopped, stopped + num_stopped);
    std::vector<std::pair<SeqId, size_t>> produced;
    for (size_t i = 0; i < num_produced; ++i) {
        produced.emplace_back(produced_ids[i], static_cast<size_t>(produced_tokens[i]));
    }
    std::vector<Completion> done;
    const SchedulerError error = scheduler->scheduler.complete_batch_multi(stopped_ids, produced, &done);
    *num_completed = done.size();
    for (size_t i = 0; i < done.size() && i < max_completed; ++i) {
        completed[i] = {done[i].id, static_cast<uint32_t>(done[i].generated_tokens),
                        static_cast<uint32_t>(done[i].reason)};
    }
    return static_cast<int>(error);
}

void qwc_scheduler_enable_prefix_cache(qwc_scheduler* scheduler, size_t snapshots) {
    scheduler->scheduler.enable_prefix_cache(snapshots);
}

int qwc_scheduler_submit_prompt(qwc_scheduler* scheduler, uint32_t id, const uint32_t* prompt, size_t prompt_tokens,
                                size_t max_new_tokens, size_t snapshot_at) {
    return static_cast<int>(scheduler->scheduler.submit_prompt(
        Request{id, prompt_tokens, max_new_tokens}, std::vector<uint32_t>(prompt, prompt + prompt_tokens), snapshot_at));
}

int qwc_scheduler_batch_prefix_ops(const qwc_scheduler* scheduler, qwc_prefix_restore_op* restores,
                                   size_t* num_restores, qwc_prefix_save_op* saves, size_t* num_saves) {
    *num_restores = 0;
    *num_saves = 0;
    const Batch* batch = scheduler->scheduler.in_flight();
    if (batch == nullptr) {
        return static_cast<int>(SchedulerError::NoBatchInFlight);
    }
    *num_restores = batch->restores.size();
    *num_saves = batch->saves.size();
    for (size_t i = 0; i < batch->restores.size(); ++i) {
        const PrefixRestoreOp& op = batch->restores[i];
        restores[i] = {op.id, op.state_slot, op.snapshot, op.copy ? 1u : 0u, op.copy_from, op.copy_to};
    }
    for (size_t i = 0; i < batch->saves.size(); ++i) {
        saves[i] = {batch->saves[i].id, batch->saves[i].state_slot, batch->saves[i].snapshot};
    }
    return 0;
}

int qwc_scheduler_abort_batch(qwc_scheduler* scheduler) { return static_cast<int>(scheduler->scheduler.abort_batch()); }

int qwc_scheduler_cancel(qwc_scheduler* scheduler, uint32_t id, int* removed) {
    bool was = false;
    const SchedulerError error = scheduler->scheduler.cancel(id, &was);
    *removed = was ? 1 : 0;
    return static_cast<int>(error);
}

long long qwc_scheduler_remaining_tokens(const qwc_scheduler* scheduler, uint32_t id) {
    const auto remaining = scheduler->scheduler.remaining_tokens(id);
    return remaining ? static_cast<long long>(*remaining) : -1;
}

size_t qwc_scheduler_waiting(const qwc_scheduler* scheduler) { return scheduler->scheduler.waiting(); }
size_t qwc_scheduler_active(const qwc_scheduler* scheduler) { return scheduler->scheduler.active(); }
size_t qwc_scheduler_committed_kv_blocks(const qwc_scheduler* scheduler) {
    return scheduler->scheduler.committed_kv_blocks();
}
qwc_cache* qwc_scheduler_cache(qwc_scheduler* scheduler) { return &scheduler->cache_view; }

int qwc_layout_build(const qwc_cache* cache, const uint32_t* decode_ids, size_t num_decode,
                     const qwc_prefill_chunk* prefill, size_t num_prefill, uint32_t* seq_ids, uint32_t* state_slots,
                     uint32_t* position_starts, uint32_t* context_lens, uint32_t* token_offsets,
                     uint32_t* block_table_offsets, uint32_t* block_ids, size_t max_block_ids, uint32_t* offender) {
    Batch batch;
    batch.decode.assign(decode_ids, decode_ids + num_decode);
    for (size_t i = 0; i < num_prefill; ++i) {
        batch.prefill.push_back({prefill[i].id, prefill[i].offset, prefill[i].tokens});
    }
    BatchLayout layout;
    SeqId bad = 0;
    const LayoutError error = BatchLayout::build(batch, *cache->cache, &layout, &bad);
    if (error != LayoutError::None) {
        if (offender != nullptr) {
            *offender = bad;
        }
        return static_cast<int>(error);
    }
    if (layout.block_ids.size() > max_block_ids) {
        return static_cast<int>(LayoutError::IntegerOverflow);
    }
    std::copy(layout.seq_ids.begin(), layout.seq_ids.end(), seq_ids);
    std::copy(layout.state_slots.begin(), layout.state_slots.end(), state_slots);
    std::copy(layout.position_starts.begin(), layout.position_starts.end(), position_starts);
    std::copy(layout.context_lens.begin(), layout.context_lens.end(), context_lens);
    std::copy(layout.token_offsets.begin(), layout.token_offsets.end(), token_offsets);
    std::copy(layout.block_table_offsets.begin(), layout.block_table_offsets.end(), block_table_offsets);
    std::copy(layout.block_ids.begin(), layout.block_ids.end(), block_ids);
    return 0;
}

}  // extern "C"
