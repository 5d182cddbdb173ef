// Host-side runtime: two-resource cache manager, continuous-batching scheduler and the
// CSR batch layout.  C++ restatement of the reference's CUDA-free `qwc-runtime` crate
// (crates/qwc-runtime/src/{cache,scheduler,layout}.rs) with the same names, argument
// meaning and error behaviour, so that the decode step keeps the scheduler / KV-cache /
// slot API it is driven by.  The prefix cache (cache.rs:193-310, :451-569) is the bookkeeping only:
// which pages an entry shares and which snapshot number it holds; the snapshots themselves (DeltaNet
// state at a prefix boundary) would be the executor's, and the prefill path that takes them is not
// part of this library.
#pragma once

#include <cstddef>
#include <cstdint>
#include <deque>
#include <optional>
#include <unordered_map>
#include <utility>
#include <vector>

namespace qwc {
namespace runtime {

using SeqId = uint32_t;

// crates/qwc-runtime/src/cache.rs:33-45
enum class Rejected : int {
    None = 0,
    NoStateSlot = 1,
    NoKvBlocks = 2,
    AlreadyAdmitted = 3,
    UnknownSequence = 4,
    NothingToRollback = 5,
};

// crates/qwc-runtime/src/cache.rs:64-104: identical, indivisible slots; LIFO free list that
// hands out 0, 1, 2, ... first.
class StatePool {
public:
    explicit StatePool(size_t capacity);
    std::optional<uint32_t> acquire();
    void release(uint32_t slot);
    size_t capacity() const { return capacity_; }
    size_t in_use() const { return capacity_ - free_.size(); }
    double utilization() const { return static_cast<double>(in_use()) / static_cast<double>(capacity_ ? capacity_ : 1); }
    bool empty() const { return free_.empty(); }

private:
    size_t capacity_;
    std::vector<uint32_t> free_;
};

// crates/qwc-runtime/src/cache.rs:112-182: paged KV pool with reference counts.
class KvPool {
public:
    KvPool(size_t capacity, size_t block_size);
    size_t blocks_for(size_t tokens) const { return (tokens + block_size_ - 1) / block_size_; }
    size_t free_blocks() const { return free_.size(); }
    size_t capacity() const { return capacity_; }
    size_t block_size() const { return block_size_; }
    double utilization() const {
        return static_cast<double>(capacity_ - free_.size()) / static_cast<double>(capacity_ ? capacity_ : 1);
    }
    bool acquire(size_t n, std::vector<uint32_t>* out);
    void retain(const std::vector<uint32_t>& blocks);
    void release(const std::vector<uint32_t>& blocks);
    uint32_t refs(uint32_t block) const { return refs_[block]; }

private:
    size_t block_size_;
    size_t capacity_;
    std::vector<uint32_t> free_;
    std::vector<uint32_t> refs_;
};

// crates/qwc-runtime/src/cache.rs:185-191
struct Sequence {
    uint32_t state_slot = 0;
    std::vector<uint32_t> blocks;
    size_t tokens = 0;
};

// crates/qwc-runtime/src/cache.rs:193-210: how to continue a cached prefix.
struct PrefixRestore {
    uint32_t snapshot = 0;
    bool copy = false;  // the prefix ends inside a page: copy page `copy_from` into `copy_to`
    uint32_t copy_from = 0;
    uint32_t copy_to = 0;
};

struct Admission {
    size_t reused = 0;  // prompt tokens that are already computed
    bool has_restore = false;
    PrefixRestore restore;
};

// crates/qwc-runtime/src/cache.rs:231-238
struct PrefixStats {
    uint64_t lookups = 0;
    uint64_t hits = 0;
    uint64_t reused_tokens = 0;
    uint64_t evictions = 0;
};

// One change of the device-resident tables caused by a cache operation
// (same layout as qwc_table_edit in the kernel ABI).
struct TableEdit {
    uint32_t slot;
    uint32_t index;
    uint32_t value;
    uint32_t kind;  // 0 set block, 1 set tokens, 2 add tokens
};

// What one sequence costs in device memory (crates/qwc-core/src/memory.rs:99-157): a recurrent-state
// slot of constant size (int8 rows with an fp32 scale per row of 128, plus the fp32 convolution window)
// and KV pages that grow with the context (e4m3, K and V, every full-attention layer).  Below
// crossover_tokens() a sequence's state is the larger part, above it its KV pages are.
struct CacheGeometry {
    uint64_t kv_bytes_per_token = 0;
    uint64_t state_bytes_per_slot = 0;
    size_t block_size = 1;

    // The decode engine's shape: `linear_layers` DeltaNet layers of `value_heads` heads (16 key heads,
    // 128 x 128 state per value head), `attention_layers` layers of 4 KV heads x 256.
    static CacheGeometry for_model(size_t linear_layers, size_t attention_layers, size_t value_heads, size_t block_size);
    uint64_t kv_bytes_per_block() const { return kv_bytes_per_token * block_size; }
    uint64_t bytes_per_seq(size_t context) const {
        return state_bytes_per_slot + (context + block_size - 1) / block_size * kv_bytes_per_block();
    }
    size_t crossover_tokens() const {
        return static_cast<size_t>(state_bytes_per_slot / (kv_bytes_per_token ? kv_bytes_per_token : 1));
    }
};

// crates/qwc-core/src/memory.rs:163-207: what is left for the two pools once the context, the weights
// and the workspace (activations, exchange blocks, graphs) are taken.
struct Budget {
    uint64_t total_vram = 0;
    uint64_t reserved = 0;
    uint64_t weights = 0;
    uint64_t workspace = 0;

    // One B200: 183 359 MiB as the driver reports it, 1 GiB for the context and the library.
    static Budget b200(uint64_t weights, uint64_t workspace);
    uint64_t cache_available() const;
    size_t max_concurrency(const CacheGeometry& geometry, size_t context) const;
    size_t max_context(const CacheGeometry& geometry, size_t concurrency) const;
    bool fits(const CacheGeometry& geometry, size_t concurrency, size_t context) const;
};

// crates/qwc-runtime/src/cache.rs:604-622: which pool is closer to exhaustion.
struct Pressure {
    double states = 0.0;
    double kv = 0.0;
    bool states_bind() const { return states >= kv; }
    double worst() const { return states > kv ? states : kv; }
};

// crates/qwc-runtime/src/cache.rs:300-449,571-594.  Every mutation is also recorded as table
// edits so the device copy of (tokens, blocks) per slot can follow without a rebuild.
class CacheManager {
public:
    CacheManager(size_t state_slots, size_t kv_blocks, size_t block_size);
    // Pools sized for a target context (cache.rs:360-378): as many state slots as sequences of that
    // length fit, the rest of the budget as KV pages - a slot without pages is as useless as pages
    // without a slot.
    static CacheManager from_budget(const Budget& budget, const CacheGeometry& geometry, size_t target_context);
    Pressure pressure() const { return Pressure{states_.utilization(), kv_.utilization()}; }
    Rejected admit(SeqId id, size_t prompt_tokens);
    Rejected append_token(SeqId id);
    Rejected rollback_token(SeqId id);
    void release(SeqId id);
    const Sequence* sequence(SeqId id) const;
    size_t active() const { return seqs_.size(); }
    const StatePool& states() const { return states_; }
    const KvPool& kv() const { return kv_; }
    // need / free of the last NoKvBlocks rejection (cache.rs:37)
    size_t last_need() const { return last_need_; }
    size_t last_free() const { return last_free_; }
    // Edits accumulated since the last drain, in order.
    std::vector<TableEdit> drain_edits();

    // ---- prefix cache (cache.rs:328-365, :451-569) ----
    void enable_prefix_cache(size_t snapshots);
    size_t prefix_capacity() const { return prefix_capacity_; }
    size_t prefix_entries() const { return entries_.size(); }
    const PrefixStats& prefix_stats() const { return prefix_stats_; }
    Rejected admit_prompt(SeqId id, const std::vector<uint32_t>& prompt, Admission* admission);
    void finish_restore(uint32_t snapshot);
    std::optional<uint32_t> reserve_snapshot();
    void cancel_snapshot(uint32_t snapshot);
    void commit_snapshot(uint32_t snapshot, SeqId id, std::vector<uint32_t> tokens);

private:
    struct PrefixEntry {
        std::vector<uint32_t> tokens;
        std::vector<uint32_t> blocks;
        uint32_t snapshot;
        uint64_t last_used;
        uint32_t pins;  // admitted sequences waiting to restore this snapshot: not evictable
    };
    bool acquire_blocks(size_t n, std::vector<uint32_t>* out);
    bool evict_one(bool for_pages);
    std::optional<size_t> entry_position(uint32_t snapshot) const;
    std::optional<uint32_t> best_match(const std::vector<uint32_t>& prompt, size_t min_tokens) const;
    void record_admission(uint32_t slot, const std::vector<uint32_t>& blocks, size_t tokens);

    StatePool states_;
    KvPool kv_;
    std::unordered_map<SeqId, Sequence> seqs_;
    std::vector<TableEdit> edits_;
    size_t last_need_ = 0;
    size_t last_free_ = 0;
    std::vector<PrefixEntry> entries_;
    std::vector<uint32_t> free_snapshots_;
    size_t prefix_capacity_ = 0;
    uint64_t prefix_clock_ = 0;
    PrefixStats prefix_stats_;
};

// crates/qwc-runtime/src/scheduler.rs:12-35
struct SchedulerConfig {
    size_t max_num_seqs;
    size_t max_num_batched_tokens;
};

struct Request {
    SeqId id;
    size_t prompt_tokens;
    size_t max_new_tokens;
};

struct PrefillChunk {
    SeqId id;
    size_t offset;
    size_t tokens;
};

// crates/qwc-runtime/src/scheduler.rs:52-68: prefix-cache work of a step.  The executor restores before
// the pass and captures inside it, after the chunk's scan.
struct PrefixRestoreOp {
    SeqId id;
    uint32_t state_slot;
    uint32_t snapshot;
    bool copy;  // the prefix's incomplete page must be copied before the step: copy_from -> copy_to
    uint32_t copy_from;
    uint32_t copy_to;
};

struct PrefixSaveOp {
    SeqId id;
    uint32_t state_slot;
    uint32_t snapshot;
};

struct Batch {
    std::vector<PrefillChunk> prefill;
    std::vector<SeqId> decode;
    std::vector<PrefixRestoreOp> restores;
    std::vector<PrefixSaveOp> saves;
    size_t num_seqs() const { return prefill.size() + decode.size(); }
    size_t num_tokens() const;
    bool empty() const { return prefill.empty() && decode.empty(); }
};

enum class FinishReason : int { Length = 0, Stopped = 1 };

struct Completion {
    SeqId id;
    size_t generated_tokens;
    FinishReason reason;
};

// crates/qwc-runtime/src/scheduler.rs:105-112
enum class SubmitError : int {
    None = 0,
    Duplicate = 1,
    EmptyPrompt = 2,
    NoOutputTokens = 3,
    NoStateCapacity = 4,
    ContextTooLong = 5,
};

// crates/qwc-runtime/src/scheduler.rs:135-144
enum class SchedulerError : int {
    None = 0,
    BatchInFlight = 1,
    NoBatchInFlight = 2,
    SequenceInFlight = 3,
    InvalidStopped = 4,
    DuplicateStopped = 5,
    Invariant = 6,
    Cache = 7,
};

// crates/qwc-runtime/src/scheduler.rs:190-668: FIFO admission, round-robin decode, one batch
// in flight, full rollback of a batch that was planned but not executed.
class Scheduler {
public:
    Scheduler(SchedulerConfig config, CacheManager cache);
    SubmitError submit(Request request);
    // The same with the prompt tokens themselves: only such a request can continue a cached prefix and
    // leave its own.  `snapshot_at`: the length of the prefix worth caching (for chat, the history
    // boundary before the generation prompt); the prefill chunk is cut there (scheduler.rs:237-261).
    void enable_prefix_cache(size_t snapshots) { cache_.enable_prefix_cache(snapshots); }
    SubmitError submit_prompt(Request request, std::vector<uint32_t> prompt, size_t snapshot_at);
    // Returns None with *has_batch == false when there is nothing to run.
    SchedulerError next_batch(Batch* batch, bool* has_batch);
    SchedulerError complete_batch(const std::vector<SeqId>& stopped, std::vector<Completion>* completed);
    SchedulerError complete_batch_multi(const std::vector<SeqId>& stopped,
                                        const std::vector<std::pair<SeqId, size_t>>& produced,
                                        std::vector<Completion>* completed);
    SchedulerError abort_batch();
    SchedulerError cancel(SeqId id, bool* removed);
    std::optional<size_t> remaining_tokens(SeqId id) const;
    size_t waiting() const { return waiting_.size(); }
    size_t active() const { return active_.size(); }
    size_t committed_kv_blocks() const { return committed_kv_blocks_; }
    const CacheManager& cache() const { return cache_; }
    CacheManager& cache_mut() { return cache_; }
    const Batch* in_flight() const { return in_flight_ ? &*in_flight_ : nullptr; }

private:
    enum class Phase { PrefillReady, PrefillInFlight, DecodeReady, DecodeInFlight };
    struct ActiveRequest {
        Request request;
        size_t reserved_blocks;
        size_t prefilled;
        size_t generated;
        Phase phase;
        bool has_restore = false;  // the prefix snapshot has not been restored yet
        PrefixRestore restore;
    };
    struct PromptTokens {
        std::vector<uint32_t> tokens;
        size_t snapshot_at;
    };
    SchedulerError admit_one(std::optional<SeqId>* admitted);
    SchedulerError set_phase(SeqId id, Phase expected, Phase next);

    SchedulerConfig config_;
    CacheManager cache_;
    std::deque<Request> waiting_;
    std::deque<SeqId> prefill_ready_;
    std::deque<SeqId> decode_ready_;
    std::unordered_map<SeqId, ActiveRequest> active_;
    std::unordered_map<SeqId, PromptTokens> prompts_;
    size_t committed_kv_blocks_ = 0;
    std::optional<Batch> in_flight_;
};

// crates/qwc-runtime/src/layout.rs:11-17
enum class LayoutError : int {
    None = 0,
    MissingSequence = 1,
    DuplicateSequence = 2,
    InvalidPrefillRange = 3,
    MissingKvBlocks = 4,
    IntegerOverflow = 5,
};

// crates/qwc-runtime/src/layout.rs:37-52: struct-of-arrays, u32, decode rows first.
struct BatchLayout {
    uint32_t num_decode = 0;
    std::vector<SeqId> seq_ids;
    std::vector<uint32_t> state_slots;
    std::vector<uint32_t> position_starts;
    std::vector<uint32_t> context_lens;
    std::vector<uint32_t> token_offsets;
    std::vector<uint32_t> block_table_offsets;
    std::vector<uint32_t> block_ids;

    static LayoutError build(const Batch& batch, const CacheManager& cache, BatchLayout* out, SeqId* offender);
    size_t num_seqs() const { return seq_ids.size(); }
    size_t num_tokens() const { return token_offsets.empty() ? 0 : token_offsets.back(); }
};

}  // namespace runtime
}  // namespace qwc
