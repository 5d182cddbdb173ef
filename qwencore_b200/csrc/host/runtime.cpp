// See runtime.h.  Behaviour follows crates/qwc-runtime/src/{cache,scheduler,layout}.rs.
#include "runtime.h"

#include <algorithm>
#include <tuple>
#include <unordered_map>
#include <limits>
#include <unordered_set>

namespace qwc {
namespace runtime {

// ---- pools ---------------------------------------------------------------------------

StatePool::StatePool(size_t capacity) : capacity_(capacity) {
    // cache.rs:79: (0..capacity).rev() so that pop() hands out 0 first
    free_.reserve(capacity);
    for (size_t i = capacity; i > 0; --i) {
        free_.push_back(static_cast<uint32_t>(i - 1));
    }
}

std::optional<uint32_t> StatePool::acquire() {
    if (free_.empty()) {
        return std::nullopt;
    }
    const uint32_t slot = free_.back();
    free_.pop_back();
    return slot;
}

void StatePool::release(uint32_t slot) { free_.push_back(slot); }

KvPool::KvPool(size_t capacity, size_t block_size) : block_size_(block_size), capacity_(capacity), refs_(capacity, 0) {
    free_.reserve(capacity);
    for (size_t i = capacity; i > 0; --i) {
        free_.push_back(static_cast<uint32_t>(i - 1));
    }
}

bool KvPool::acquire(size_t n, std::vector<uint32_t>* out) {
    if (free_.size() < n) {
        return false;
    }
    out->clear();
    for (size_t i = 0; i < n; ++i) {
        const uint32_t block = free_.back();
        free_.pop_back();
        refs_[block] = 1;
        out->push_back(block);
    }
    return true;
}

void KvPool::retain(const std::vector<uint32_t>& blocks) {
    for (uint32_t block : blocks) {
        refs_[block] += 1;
    }
}

void KvPool::release(const std::vector<uint32_t>& blocks) {
    for (uint32_t block : blocks) {
        if (refs_[block] > 0 && --refs_[block] == 0) {
            free_.push_back(block);
        }
    }
}

// ---- cache manager -------------------------------------------------------------------

CacheGeometry CacheGeometry::for_model(size_t linear_layers, size_t attention_layers, size_t value_heads,
                                       size_t block_size) {
    constexpr uint64_t kStateDim = 128, kKeyHeads = 16, kKvHeads = 4, kHeadDim = 256, kConvWindow = 3;
    CacheGeometry geometry;
    geometry.block_size = block_size ? block_size : 1;
    geometry.kv_bytes_per_token = attention_layers * kKvHeads * kHeadDim * 2;  // e4m3: one byte each
    const uint64_t state_elements = linear_layers * value_heads * kStateDim * kStateDim;
    const uint64_t channels = 2 * kKeyHeads * kStateDim + value_heads * kStateDim;
    geometry.state_bytes_per_slot = state_elements + state_elements / kStateDim * 4  // codes + row scales
                                    + linear_layers * channels * kConvWindow * 4;      // fp32 conv history
    return geometry;
}

Budget Budget::b200(uint64_t weights, uint64_t workspace) {
    constexpr uint64_t kMiB = 1024ull * 1024ull;
    return Budget{183359ull * kMiB, 1024ull * kMiB, weights, workspace};
}

uint64_t Budget::cache_available() const {
    uint64_t left = total_vram;
    for (const uint64_t taken : {reserved, weights, workspace}) {
        left = left > taken ? left - taken : 0;
    }
    return left;
}

size_t Budget::max_concurrency(const CacheGeometry& geometry, size_t context) const {
    const uint64_t per_seq = geometry.bytes_per_seq(context);
    return per_seq == 0 ? 0 : static_cast<size_t>(cache_available() / per_seq);
}

size_t Budget::max_context(const CacheGeometry& geometry, size_t concurrency) const {
    if (concurrency == 0 || geometry.kv_bytes_per_token == 0) {
        return 0;
    }
    const uint64_t per_seq = cache_available() / concurrency;
    const uint64_t for_kv = per_seq > geometry.state_bytes_per_slot ? per_seq - geometry.state_bytes_per_slot : 0;
    return static_cast<size_t>(for_kv / geometry.kv_bytes_per_token);
}

bool Budget::fits(const CacheGeometry& geometry, size_t concurrency, size_t context) const {
    return geometry.bytes_per_seq(context) * concurrency <= cache_available();
}

CacheManager CacheManager::from_budget(const Budget& budget, const CacheGeometry& geometry, size_t target_context) {
    const uint64_t available = budget.cache_available();
    const uint64_t per_seq = std::max<uint64_t>(geometry.bytes_per_seq(target_context), 1);
    const size_t slots = static_cast<size_t>(available / per_seq);
    const uint64_t state_bytes = slots * geometry.state_bytes_per_slot;
    const uint64_t kv_bytes = available > state_bytes ? available - state_bytes : 0;
    const size_t blocks = static_cast<size_t>(kv_bytes / std::max<uint64_t>(geometry.kv_bytes_per_block(), 1));
    return CacheManager(slots, blocks, geometry.block_size);
}

CacheManager::CacheManager(size_t state_slots, size_t kv_blocks, size_t block_size)
    : states_(state_slots), kv_(kv_blocks, block_size) {}

Rejected CacheManager::admit(SeqId id, size_t prompt_tokens) {
    if (seqs_.count(id)) {
        return Rejected::AlreadyAdmitted;
    }
    const size_t need = kv_.blocks_for(prompt_tokens);
    // cache.rs:386-390: the slot is checked before the blocks are taken
    if (states_.empty()) {
        return Rejected::NoStateSlot;
    }
    std::vector<uint32_t> blocks;
    if (!acquire_blocks(need, &blocks)) {
        last_need_ = need;
        last_free_ = kv_.free_blocks();
        return Rejected::NoKvBlocks;
    }
    const uint32_t slot = *states_.acquire();
    record_admission(slot, blocks, prompt_tokens);
    Sequence seq;
    seq.state_slot = slot;
    seq.blocks = std::move(blocks);
    seq.tokens = prompt_tokens;
    seqs_.emplace(id, std::move(seq));
    return Rejected::None;
}

void CacheManager::record_admission(uint32_t slot, const std::vector<uint32_t>& blocks, size_t tokens) {
    for (size_t i = 0; i < blocks.size(); ++i) {
        edits_.push_back({slot, static_cast<uint32_t>(i), blocks[i], 0});
    }
    edits_.push_back({slot, 0, static_cast<uint32_t>(tokens), 1});
}

// ---- prefix cache (crates/qwc-runtime/src/cache.rs:240-310, :328-365, :451-569) ----------------

void CacheManager::enable_prefix_cache(size_t snapshots) {
    prefix_capacity_ = snapshots;
    free_snapshots_.clear();
    for (size_t i = snapshots; i > 0; --i) {
        free_snapshots_.push_back(static_cast<uint32_t>(i - 1));  // popped from the back: 0, 1, 2, ...
    }
}

std::optional<size_t> CacheManager::entry_position(uint32_t snapshot) const {
    for (size_t i = 0; i < entries_.size(); ++i) {
        if (entries_[i].snapshot == snapshot) {
            return i;
        }
    }
    return std::nullopt;
}

// The longest entry that is a proper prefix of the prompt (one prompt token at least must be run to
// have logits for the first response token) and at least `min_tokens` long.
std::optional<uint32_t> CacheManager::best_match(const std::vector<uint32_t>& prompt, size_t min_tokens) const {
    const PrefixEntry* best = nullptr;
    for (const PrefixEntry& entry : entries_) {
        const size_t length = entry.tokens.size();
        if (length < min_tokens || length >= prompt.size() ||
            !std::equal(entry.tokens.begin(), entry.tokens.end(), prompt.begin())) {
            continue;
        }
        if (best == nullptr || length >= best->tokens.size()) {  // max_by_key keeps the last of equal keys
            best = &entry;
        }
    }
    return best == nullptr ? std::nullopt : std::optional<uint32_t>(best->snapshot);
}

// Evicts the least valuable unpinned entry: entries nested in a longer one first, then entries no
// live sequence holds pages of, then by age.  `for_pages`: the caller wants KV pages, so an entry all
// of whose pages live sequences hold is left alone (it would free nothing and be lost).
bool CacheManager::evict_one(bool for_pages) {
    std::vector<uint32_t> holders(kv_.capacity(), 0);
    for (const PrefixEntry& entry : entries_) {
        for (uint32_t block : entry.blocks) {
            holders[block] += 1;
        }
    }
    const auto live = [&](uint32_t block) { return kv_.refs(block) > holders[block]; };
    std::optional<size_t> chosen;
    bool chosen_not_superseded = false, chosen_in_use = false;
    uint64_t chosen_age = 0;
    for (size_t i = 0; i < entries_.size(); ++i) {
        const PrefixEntry& entry = entries_[i];
        if (entry.pins != 0) {
            continue;
        }
        const bool all_live = std::all_of(entry.blocks.begin(), entry.blocks.end(), live);
        if (for_pages && all_live) {
            continue;
        }
        bool superseded = false;
        for (const PrefixEntry& other : entries_) {
            if (other.tokens.size() > entry.tokens.size() &&
                std::equal(entry.tokens.begin(), entry.tokens.end(), other.tokens.begin())) {
                superseded = true;
                break;
            }
        }
        const bool in_use = std::any_of(entry.blocks.begin(), entry.blocks.end(), live);
        const bool not_superseded = !superseded;
        // min_by_key over (not superseded, in use, last used); the first of equal keys wins
        const bool smaller = !chosen || std::make_tuple(not_superseded, in_use, entry.last_used) <
                                            std::make_tuple(chosen_not_superseded, chosen_in_use, chosen_age);
        if (smaller) {
            chosen = i;
            chosen_not_superseded = not_superseded;
            chosen_in_use = in_use;
            chosen_age = entry.last_used;
        }
    }
    if (!chosen) {
        return false;
    }
    PrefixEntry entry = std::move(entries_[*chosen]);
    entries_[*chosen] = std::move(entries_.back());  // swap_remove
    entries_.pop_back();
    kv_.release(entry.blocks);
    free_snapshots_.push_back(entry.snapshot);
    prefix_stats_.evictions += 1;
    return true;
}

// Blocks from the pool; when short, at the cost of prefix-cache entries (live sequences matter more).
bool CacheManager::acquire_blocks(size_t n, std::vector<uint32_t>* out) {
    for (;;) {
        if (kv_.free_blocks() >= n) {
            return kv_.acquire(n, out);
        }
        if (!evict_one(true)) {
            return false;
        }
    }
}

Rejected CacheManager::admit_prompt(SeqId id, const std::vector<uint32_t>& prompt, Admission* admission) {
    *admission = Admission{};
    if (seqs_.count(id)) {
        return Rejected::AlreadyAdmitted;
    }
    prefix_stats_.lookups += 1;
    const std::optional<uint32_t> snapshot = best_match(prompt, kv_.block_size());
    if (!snapshot) {
        return admit(id, prompt.size());
    }
    if (states_.empty()) {
        return Rejected::NoStateSlot;
    }
    const size_t index = *entry_position(*snapshot);
    entries_[index].pins += 1;
    const size_t reused = entries_[index].tokens.size();
    const size_t full = reused / kv_.block_size();
    std::vector<uint32_t> shared(entries_[index].blocks.begin(), entries_[index].blocks.begin() + full);
    const bool has_tail = reused % kv_.block_size() != 0;
    const uint32_t tail = has_tail ? entries_[index].blocks[full] : 0;
    // the prompt is longer than the prefix, so there is always a page of its own; with an incomplete
    // tail the first own page is a copy of the shared one
    const size_t need = kv_.blocks_for(prompt.size()) - shared.size();
    std::vector<uint32_t> fresh;
    if (!acquire_blocks(need, &fresh)) {
        finish_restore(*snapshot);
        last_need_ = need;
        last_free_ = kv_.free_blocks();
        return Rejected::NoKvBlocks;
    }
    const uint32_t slot = *states_.acquire();
    kv_.retain(shared);
    Sequence seq;
    seq.state_slot = slot;
    seq.blocks = shared;
    seq.blocks.insert(seq.blocks.end(), fresh.begin(), fresh.end());
    seq.tokens = prompt.size();
    record_admission(slot, seq.blocks, seq.tokens);
    seqs_.emplace(id, std::move(seq));

    const uint64_t now = ++prefix_clock_;
    if (const std::optional<size_t> again = entry_position(*snapshot)) {  // eviction above may have moved entries
        entries_[*again].last_used = now;
    }
    prefix_stats_.hits += 1;
    prefix_stats_.reused_tokens += reused;
    admission->reused = reused;
    admission->has_restore = true;
    admission->restore.snapshot = *snapshot;
    admission->restore.copy = has_tail;
    admission->restore.copy_from = tail;
    admission->restore.copy_to = has_tail ? fresh[0] : 0;
    return Rejected::None;
}

void CacheManager::finish_restore(uint32_t snapshot) {
    if (const std::optional<size_t> index = entry_position(snapshot)) {
        if (entries_[*index].pins > 0) {
            entries_[*index].pins -= 1;
        }
    }
}

std::optional<uint32_t> CacheManager::reserve_snapshot() {
    if (prefix_capacity_ == 0) {
        return std::nullopt;
    }
    if (free_snapshots_.empty() && !evict_one(false)) {
        return std::nullopt;
    }
    const uint32_t snapshot = free_snapshots_.back();
    free_snapshots_.pop_back();
    return snapshot;
}

void CacheManager::cancel_snapshot(uint32_t snapshot) { free_snapshots_.push_back(snapshot); }

void CacheManager::commit_snapshot(uint32_t snapshot, SeqId id, std::vector<uint32_t> tokens) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) {
        cancel_snapshot(snapshot);
        return;
    }
    const uint64_t now = ++prefix_clock_;
    for (PrefixEntry& existing : entries_) {
        if (existing.tokens == tokens) {
            existing.last_used = now;
            free_snapshots_.push_back(snapshot);
            return;
        }
    }
    const size_t covered = kv_.blocks_for(tokens.size());
    std::vector<uint32_t> blocks(it->second.blocks.begin(), it->second.blocks.begin() + covered);
    kv_.retain(blocks);
    entries_.push_back({std::move(tokens), std::move(blocks), snapshot, now, 0});
}

Rejected CacheManager::append_token(SeqId id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) {
        return Rejected::UnknownSequence;
    }
    Sequence& seq = it->second;
    const size_t need = kv_.blocks_for(seq.tokens + 1);
    if (need > seq.blocks.size()) {
        const size_t extra = need - seq.blocks.size();
        std::vector<uint32_t> more;
        if (!acquire_blocks(extra, &more)) {
            last_need_ = extra;
            last_free_ = kv_.free_blocks();
            return Rejected::NoKvBlocks;
        }
        for (uint32_t block : more) {
            edits_.push_back({seq.state_slot, static_cast<uint32_t>(seq.blocks.size()), block, 0});
            seq.blocks.push_back(block);
        }
    }
    seq.tokens += 1;
    edits_.push_back({seq.state_slot, 0, static_cast<uint32_t>(seq.tokens), 1});
    return Rejected::None;
}

Rejected CacheManager::rollback_token(SeqId id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) {
        return Rejected::UnknownSequence;
    }
    Sequence& seq = it->second;
    if (seq.tokens == 0) {
        return Rejected::NothingToRollback;
    }
    seq.tokens -= 1;
    const size_t keep = kv_.blocks_for(seq.tokens);
    std::vector<uint32_t> released(seq.blocks.begin() + keep, seq.blocks.end());
    seq.blocks.resize(keep);
    kv_.release(released);
    edits_.push_back({seq.state_slot, 0, static_cast<uint32_t>(seq.tokens), 1});
    return Rejected::None;
}

void CacheManager::release(SeqId id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) {
        return;
    }
    states_.release(it->second.state_slot);
    kv_.release(it->second.blocks);
    edits_.push_back({it->second.state_slot, 0, 0, 1});
    seqs_.erase(it);
}

const Sequence* CacheManager::sequence(SeqId id) const {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? nullptr : &it->second;
}

// The device applies one drain with a thread per edit and no order between them, so a drain
// never carries two edits of the same word: the last one wins here, at the place of the first.
// (A released slot goes straight to the next admission, and a rollback follows an append, so
// "tokens = 0" and "tokens = prompt" for one slot do meet in one drain.)
std::vector<TableEdit> CacheManager::drain_edits() {
    std::vector<TableEdit> out;
    out.reserve(edits_.size());
    std::unordered_map<uint64_t, size_t> place;  // (slot, kind, index) -> position in `out`
    for (const TableEdit& edit : edits_) {
        if (edit.kind == 2) {
            // a relative edit cannot be merged with an absolute one; the host emits none
            out.push_back(edit);
            continue;
        }
        const uint64_t key = (static_cast<uint64_t>(edit.slot) << 33) | (static_cast<uint64_t>(edit.kind & 1u) << 32) |
                             (edit.kind == 0 ? edit.index : 0u);
        const auto found = place.find(key);
        if (found == place.end()) {
            place.emplace(key, out.size());
            out.push_back(edit);
        } else {
            out[found->second] = edit;
        }
    }
    edits_.clear();
    return out;
}

// ---- scheduler -------------------------------------------------------------------------

size_t Batch::num_tokens() const {
    size_t total = decode.size();
    for (const PrefillChunk& chunk : prefill) {
        total += chunk.tokens;
    }
    return total;
}

Scheduler::Scheduler(SchedulerConfig config, CacheManager cache) : config_(config), cache_(std::move(cache)) {}

SubmitError Scheduler::submit(Request request) {
    const bool queued =
        std::any_of(waiting_.begin(), waiting_.end(), [&](const Request& r) { return r.id == request.id; });
    if (active_.count(request.id) || queued) {
        return SubmitError::Duplicate;
    }
    if (request.prompt_tokens == 0) {
        return SubmitError::EmptyPrompt;
    }
    if (request.max_new_tokens == 0) {
        return SubmitError::NoOutputTokens;
    }
    if (cache_.states().capacity() == 0) {
        return SubmitError::NoStateCapacity;
    }
    size_t context = request.prompt_tokens + request.max_new_tokens;
    if (context < request.prompt_tokens) {
        context = std::numeric_limits<size_t>::max();  // saturating_add
    }
    if (cache_.kv().blocks_for(context) > cache_.kv().capacity()) {
        return SubmitError::ContextTooLong;
    }
    waiting_.push_back(request);
    return SubmitError::None;
}

SubmitError Scheduler::submit_prompt(Request request, std::vector<uint32_t> prompt, size_t snapshot_at) {
    if (prompt.size() != request.prompt_tokens || snapshot_at > prompt.size()) {
        return SubmitError::EmptyPrompt;  // the reference asserts; a C caller gets an error instead
    }
    const SubmitError submitted = submit(request);
    if (submitted != SubmitError::None) {
        return submitted;
    }
    prompts_[request.id] = PromptTokens{std::move(prompt), snapshot_at};
    return SubmitError::None;
}

SchedulerError Scheduler::set_phase(SeqId id, Phase expected, Phase next) {
    auto it = active_.find(id);
    if (it == active_.end() || it->second.phase != expected) {
        return SchedulerError::Invariant;
    }
    it->second.phase = next;
    return SchedulerError::None;
}

SchedulerError Scheduler::admit_one(std::optional<SeqId>* admitted) {
    admitted->reset();
    const size_t candidates = waiting_.size();
    for (size_t i = 0; i < candidates; ++i) {
        const Request request = waiting_.front();
        waiting_.pop_front();
        const size_t lifetime = request.prompt_tokens + request.max_new_tokens;
        const size_t reserved = cache_.kv().blocks_for(lifetime);
        // scheduler.rs:615-620: lifetime commitment prevents a decode deadlock
        if (reserved > cache_.kv().capacity() - committed_kv_blocks_) {
            waiting_.push_back(request);
            continue;
        }
        Admission admission;
        const auto prompt = prompts_.find(request.id);
        const Rejected outcome = prompt != prompts_.end()
                                     ? cache_.admit_prompt(request.id, prompt->second.tokens, &admission)
                                     : cache_.admit(request.id, request.prompt_tokens);
        switch (outcome) {
            case Rejected::None: {
                committed_kv_blocks_ += reserved;
                ActiveRequest active{request, reserved, admission.reused, 0, Phase::PrefillReady};
                active.has_restore = admission.has_restore;
                active.restore = admission.restore;
                active_.emplace(request.id, active);
                *admitted = request.id;
                return SchedulerError::None;
            }
            case Rejected::NoStateSlot:
                waiting_.push_front(request);
                return SchedulerError::None;
            case Rejected::NoKvBlocks:
                waiting_.push_back(request);
                break;
            default:
                return SchedulerError::Cache;
        }
    }
    return SchedulerError::None;
}

SchedulerError Scheduler::next_batch(Batch* out, bool* has_batch) {
    *has_batch = false;
    if (in_flight_) {
        return SchedulerError::BatchInFlight;
    }
    Batch batch;
    const size_t decode_candidates = decode_ready_.size();
    for (size_t i = 0; i < decode_candidates; ++i) {
        if (batch.num_seqs() == config_.max_num_seqs || batch.num_tokens() == config_.max_num_batched_tokens) {
            break;
        }
        const SeqId id = decode_ready_.front();
        decode_ready_.pop_front();
        const Rejected outcome = cache_.append_token(id);
        if (outcome == Rejected::None) {
            const SchedulerError phase = set_phase(id, Phase::DecodeReady, Phase::DecodeInFlight);
            if (phase != SchedulerError::None) {
                return phase;
            }
            batch.decode.push_back(id);
        } else if (outcome == Rejected::NoKvBlocks) {
            decode_ready_.push_back(id);
        } else {
            return SchedulerError::Cache;
        }
    }

    while (batch.num_seqs() < config_.max_num_seqs && batch.num_tokens() < config_.max_num_batched_tokens) {
        SeqId id;
        if (!prefill_ready_.empty()) {
            id = prefill_ready_.front();
            prefill_ready_.pop_front();
        } else {
            std::optional<SeqId> admitted;
            const SchedulerError err = admit_one(&admitted);
            if (err != SchedulerError::None) {
                return err;
            }
            if (!admitted) {
                break;
            }
            id = *admitted;
        }
        auto it = active_.find(id);
        if (it == active_.end() || it->second.phase != Phase::PrefillReady) {
            return SchedulerError::Invariant;
        }
        const size_t remaining = it->second.request.prompt_tokens - it->second.prefilled;
        const size_t budget = config_.max_num_batched_tokens - batch.num_tokens();
        size_t tokens = std::min(remaining, budget);
        const size_t offset = it->second.prefilled;
        // the snapshot point is inside the chunk: the chunk ends at it, the rest of the prompt goes in
        // the next step (scheduler.rs:339-349)
        std::optional<size_t> snapshot_at;
        const auto prompt = prompts_.find(id);
        if (prompt != prompts_.end() && cache_.prefix_capacity() > 0 && prompt->second.snapshot_at > offset &&
            prompt->second.snapshot_at <= offset + tokens) {
            snapshot_at = prompt->second.snapshot_at;
            tokens = *snapshot_at - offset;
        }
        const Sequence* sequence = cache_.sequence(id);
        if (sequence == nullptr) {
            return SchedulerError::Invariant;
        }
        const uint32_t state_slot = sequence->state_slot;
        if (it->second.has_restore) {
            const PrefixRestore& restore = it->second.restore;
            batch.restores.push_back({id, state_slot, restore.snapshot, restore.copy, restore.copy_from, restore.copy_to});
        }
        // the next turn of the same dialog will start with this whole history
        if (snapshot_at && *snapshot_at >= cache_.kv().block_size()) {
            if (const std::optional<uint32_t> snapshot = cache_.reserve_snapshot()) {
                batch.saves.push_back({id, state_slot, *snapshot});
            }
        }
        const SchedulerError phase = set_phase(id, Phase::PrefillReady, Phase::PrefillInFlight);
        if (phase != SchedulerError::None) {
            return phase;
        }
        batch.prefill.push_back({id, offset, tokens});
    }

    if (batch.empty()) {
        return SchedulerError::None;
    }
    in_flight_ = batch;
    *out = std::move(batch);
    *has_batch = true;
    return SchedulerError::None;
}

SchedulerError Scheduler::complete_batch(const std::vector<SeqId>& stopped, std::vector<Completion>* completed) {
    return complete_batch_multi(stopped, {}, completed);
}

// The same, for steps in which a decode sequence may have produced more than one token (speculative
// verification accepts 1 .. k + 1): sequences missing from `produced` count one token
// (crates/qwc-runtime/src/scheduler.rs:392-500).
SchedulerError Scheduler::complete_batch_multi(const std::vector<SeqId>& stopped,
                                               const std::vector<std::pair<SeqId, size_t>>& produced,
                                               std::vector<Completion>* completed) {
    completed->clear();
    if (!in_flight_) {
        return SchedulerError::NoBatchInFlight;
    }
    for (const auto& entry : produced) {
        if (entry.second == 0) {
            return SchedulerError::Invariant;
        }
        if (std::find(in_flight_->decode.begin(), in_flight_->decode.end(), entry.first) == in_flight_->decode.end()) {
            return SchedulerError::InvalidStopped;
        }
    }
    std::unordered_set<SeqId> stopped_set;
    for (SeqId id : stopped) {
        if (!stopped_set.insert(id).second) {
            return SchedulerError::DuplicateStopped;
        }
        if (std::find(in_flight_->decode.begin(), in_flight_->decode.end(), id) == in_flight_->decode.end()) {
            return SchedulerError::InvalidStopped;
        }
    }
    Batch batch = std::move(*in_flight_);
    in_flight_.reset();
    for (const PrefixRestoreOp& op : batch.restores) {
        auto it = active_.find(op.id);
        if (it != active_.end()) {
            it->second.has_restore = false;
        }
        cache_.finish_restore(op.snapshot);
    }
    for (const PrefixSaveOp& op : batch.saves) {
        const auto prompt = prompts_.find(op.id);
        if (prompt != prompts_.end()) {
            cache_.commit_snapshot(op.snapshot, op.id,
                                   std::vector<uint32_t>(prompt->second.tokens.begin(),
                                                         prompt->second.tokens.begin() + prompt->second.snapshot_at));
        } else {
            cache_.cancel_snapshot(op.snapshot);
        }
    }
    for (const PrefillChunk& chunk : batch.prefill) {
        auto it = active_.find(chunk.id);
        if (it == active_.end() || it->second.phase != Phase::PrefillInFlight) {
            return SchedulerError::Invariant;
        }
        it->second.prefilled += chunk.tokens;
        if (it->second.prefilled == it->second.request.prompt_tokens) {
            it->second.phase = Phase::DecodeReady;
            decode_ready_.push_back(chunk.id);
        } else {
            it->second.phase = Phase::PrefillReady;
            prefill_ready_.push_back(chunk.id);
        }
    }
    for (SeqId id : batch.decode) {
        auto it = active_.find(id);
        if (it == active_.end() || it->second.phase != Phase::DecodeInFlight) {
            return SchedulerError::Invariant;
        }
        ActiveRequest& active = it->second;
        size_t tokens = 1;
        for (const auto& entry : produced) {
            if (entry.first == id) {
                tokens = entry.second;
                break;  // the first entry of a sequence counts, as in the reference's `find`
            }
        }
        active.generated = std::min(active.generated + tokens, active.request.max_new_tokens);
        const bool was_stopped = stopped_set.count(id) != 0;
        if (was_stopped || active.generated >= active.request.max_new_tokens) {
            completed->push_back({id, active.generated, was_stopped ? FinishReason::Stopped : FinishReason::Length});
            committed_kv_blocks_ -= active.reserved_blocks;
            cache_.release(id);
            prompts_.erase(id);
            active_.erase(it);
        } else {
            active.phase = Phase::DecodeReady;
            decode_ready_.push_back(id);
        }
    }
    return SchedulerError::None;
}

SchedulerError Scheduler::abort_batch() {
    if (!in_flight_) {
        return SchedulerError::NoBatchInFlight;
    }
    Batch batch = std::move(*in_flight_);
    in_flight_.reset();
    // restores stay with their sequences and go with the next chunk; snapshots were not captured: their
    // slots are free again (scheduler.rs:536-540)
    for (const PrefixSaveOp& op : batch.saves) {
        cache_.cancel_snapshot(op.snapshot);
    }
    for (auto it = batch.prefill.rbegin(); it != batch.prefill.rend(); ++it) {
        const SchedulerError phase = set_phase(it->id, Phase::PrefillInFlight, Phase::PrefillReady);
        if (phase != SchedulerError::None) {
            return phase;
        }
        prefill_ready_.push_front(it->id);
    }
    for (auto it = batch.decode.rbegin(); it != batch.decode.rend(); ++it) {
        if (cache_.rollback_token(*it) != Rejected::None) {
            return SchedulerError::Cache;
        }
        const SchedulerError phase = set_phase(*it, Phase::DecodeInFlight, Phase::DecodeReady);
        if (phase != SchedulerError::None) {
            return phase;
        }
        decode_ready_.push_front(*it);
    }
    return SchedulerError::None;
}

SchedulerError Scheduler::cancel(SeqId id, bool* removed) {
    *removed = false;
    if (in_flight_) {
        const bool decoding =
            std::find(in_flight_->decode.begin(), in_flight_->decode.end(), id) != in_flight_->decode.end();
        const bool prefilling = std::any_of(in_flight_->prefill.begin(), in_flight_->prefill.end(),
                                            [&](const PrefillChunk& c) { return c.id == id; });
        if (decoding || prefilling) {
            return SchedulerError::SequenceInFlight;
        }
    }
    auto queued = std::find_if(waiting_.begin(), waiting_.end(), [&](const Request& r) { return r.id == id; });
    if (queued != waiting_.end()) {
        waiting_.erase(queued);
        prompts_.erase(id);
        *removed = true;
        return SchedulerError::None;
    }
    auto it = active_.find(id);
    if (it != active_.end()) {
        prefill_ready_.erase(std::remove(prefill_ready_.begin(), prefill_ready_.end(), id), prefill_ready_.end());
        decode_ready_.erase(std::remove(decode_ready_.begin(), decode_ready_.end(), id), decode_ready_.end());
        committed_kv_blocks_ -= it->second.reserved_blocks;
        if (it->second.has_restore) {
            cache_.finish_restore(it->second.restore.snapshot);
        }
        cache_.release(id);
        prompts_.erase(id);
        active_.erase(it);
        *removed = true;
    }
    return SchedulerError::None;
}

std::optional<size_t> Scheduler::remaining_tokens(SeqId id) const {
    auto it = active_.find(id);
    if (it == active_.end()) {
        return std::nullopt;
    }
    return it->second.request.max_new_tokens - it->second.generated;
}

// ---- batch layout ----------------------------------------------------------------------

namespace {

LayoutError push_sequence(BatchLayout* layout, SeqId id, uint32_t state_slot, size_t position, size_t context,
                          size_t tokens, const CacheManager& cache) {
    const Sequence* seq = cache.sequence(id);
    if (seq == nullptr) {
        return LayoutError::MissingSequence;
    }
    const size_t blocks = cache.kv().blocks_for(context);
    if (blocks > seq->blocks.size()) {
        return LayoutError::MissingKvBlocks;
    }
    constexpr size_t kMax = std::numeric_limits<uint32_t>::max();
    const size_t total_tokens = layout->num_tokens() + tokens;
    if (position > kMax || context > kMax || total_tokens > kMax || layout->block_ids.size() + blocks > kMax) {
        return LayoutError::IntegerOverflow;
    }
    layout->seq_ids.push_back(id);
    layout->state_slots.push_back(state_slot);
    layout->position_starts.push_back(static_cast<uint32_t>(position));
    layout->context_lens.push_back(static_cast<uint32_t>(context));
    layout->token_offsets.push_back(static_cast<uint32_t>(total_tokens));
    layout->block_ids.insert(layout->block_ids.end(), seq->blocks.begin(), seq->blocks.begin() + blocks);
    layout->block_table_offsets.push_back(static_cast<uint32_t>(layout->block_ids.size()));
    return LayoutError::None;
}

}  // namespace

LayoutError BatchLayout::build(const Batch& batch, const CacheManager& cache, BatchLayout* out, SeqId* offender) {
    BatchLayout layout;
    layout.num_decode = static_cast<uint32_t>(batch.decode.size());
    layout.token_offsets.push_back(0);
    layout.block_table_offsets.push_back(0);
    std::unordered_set<SeqId> seen;
    auto fail = [&](LayoutError error, SeqId id) {
        if (offender != nullptr) {
            *offender = id;
        }
        return error;
    };
    for (SeqId id : batch.decode) {
        if (!seen.insert(id).second) {
            return fail(LayoutError::DuplicateSequence, id);
        }
        const Sequence* seq = cache.sequence(id);
        if (seq == nullptr) {
            return fail(LayoutError::MissingSequence, id);
        }
        if (seq->tokens == 0) {
            return fail(LayoutError::IntegerOverflow, id);  // checked_sub(1) on the decode position
        }
        const LayoutError pushed = push_sequence(&layout, id, seq->state_slot, seq->tokens - 1, seq->tokens, 1, cache);
        if (pushed != LayoutError::None) {
            return fail(pushed, id);
        }
    }
    for (const PrefillChunk& chunk : batch.prefill) {
        if (!seen.insert(chunk.id).second) {
            return fail(LayoutError::DuplicateSequence, chunk.id);
        }
        const Sequence* seq = cache.sequence(chunk.id);
        if (seq == nullptr) {
            return fail(LayoutError::MissingSequence, chunk.id);
        }
        const size_t context = chunk.offset + chunk.tokens;
        if (chunk.tokens == 0 || context > seq->tokens) {
            return fail(LayoutError::InvalidPrefillRange, chunk.id);
        }
        const LayoutError pushed =
            push_sequence(&layout, chunk.id, seq->state_slot, chunk.offset, context, chunk.tokens, cache);
        if (pushed != LayoutError::None) {
            return fail(pushed, chunk.id);
        }
    }
    *out = std::move(layout);
    return LayoutError::None;
}

}  // namespace runtime
}  // namespace qwc
