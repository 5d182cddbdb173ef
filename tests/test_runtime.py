"""Host runtime (cache manager, scheduler, batch layout) against the reference's own unit tests.

Every test restates a `#[test]` of crates/qwc-runtime/src/{cache,scheduler,layout}.rs with the same
numbers and expected values; the citation names it.  No GPU is involved.
"""

import numpy as np
import pytest

from qwencore_b200.engine import CacheManager, RuntimeError_, Scheduler, build_layout


def rejected(name):
    return pytest.raises(RuntimeError_, match=name)


# ---- cache.rs ------------------------------------------------------------------------------

def test_admission_requires_both_resources(built_library):
    # cache.rs:634-646
    m = CacheManager(2, 1000, 64)
    m.admit(1, 128)
    m.admit(2, 128)
    with rejected("NoStateSlot"):
        m.admit(3, 128)
    assert m.free_blocks() > 900
    m.release(1)
    m.admit(3, 128)


def test_kv_can_be_the_binding_constraint(built_library):
    # cache.rs:648-656
    m = CacheManager(64, 10, 64)
    m.admit(1, 640)
    with rejected("NoKvBlocks"):
        m.admit(2, 64)
    assert m.last_shortage() == (1, 0)
    assert m.states_in_use() == 1


def test_append_allocates_lazily(built_library):
    # cache.rs:692-709
    m = CacheManager(4, 100, 64)
    m.admit(1, 64)
    assert len(m.sequence(1)["blocks"]) == 1
    m.append_token(1)
    assert len(m.sequence(1)["blocks"]) == 2
    assert m.sequence(1)["tokens"] == 65
    before = m.free_blocks()
    for _ in range(60):
        m.append_token(1)
    assert m.free_blocks() == before


def test_append_and_rollback_are_transactional(built_library):
    # cache.rs:711-725
    m = CacheManager(1, 2, 64)
    m.admit(1, 64)
    m.append_token(1)
    assert m.sequence(1)["tokens"] == 65 and len(m.sequence(1)["blocks"]) == 2
    m.rollback_token(1)
    assert m.sequence(1)["tokens"] == 64 and len(m.sequence(1)["blocks"]) == 1
    assert m.free_blocks() == 1


def test_unknown_sequence_is_an_error_not_a_panic(built_library):
    # cache.rs:727-732
    m = CacheManager(1, 2, 64)
    with rejected("UnknownSequence"):
        m.append_token(7)
    with rejected("UnknownSequence"):
        m.rollback_token(7)


def test_zero_block_size_is_rejected_at_construction(built_library):
    # cache.rs:734-738
    with pytest.raises(ValueError, match="KV block size must be positive"):
        CacheManager(1, 1, 0)


def test_release_returns_everything(built_library):
    # cache.rs:740-754
    m = CacheManager(4, 100, 64)
    blocks = m.free_blocks()
    for seq in range(4):
        m.admit(seq, 200)
    for seq in range(4):
        m.release(seq)
    assert m.states_in_use() == 0 and m.free_blocks() == blocks and m.active() == 0


def test_pools_hand_out_ascending_ids_and_reuse_lifo(built_library):
    # cache.rs:79,129,158: free lists are (0..capacity).rev() popped from the back
    m = CacheManager(3, 10, 64)
    m.admit(10, 130)
    m.admit(11, 10)
    assert m.sequence(10) == {"state_slot": 0, "tokens": 130, "blocks": [0, 1, 2]}
    assert m.sequence(11) == {"state_slot": 1, "tokens": 10, "blocks": [3]}
    m.release(10)
    m.admit(12, 64)  # most recently freed slot and page come back first
    assert m.sequence(12)["state_slot"] == 0
    assert m.sequence(12)["blocks"] == [2]


def test_double_admission_is_rejected(built_library):
    m = CacheManager(2, 10, 64)
    m.admit(1, 10)
    with rejected("AlreadyAdmitted"):
        m.admit(1, 10)


def test_cache_operations_are_mirrored_as_table_edits(built_library):
    """Every mutation of (tokens, blocks) per slot is recorded for the device-resident copy."""
    m = CacheManager(2, 10, 16)
    m.admit(5, 17)
    assert m.drain_edits().tolist() == [[0, 0, 0, 0], [0, 1, 1, 0], [0, 0, 17, 1]]
    for _ in range(15):
        m.append_token(5)
    assert m.drain_edits()[-1].tolist() == [0, 0, 32, 1]
    m.append_token(5)  # token 33 opens page index 2
    assert m.drain_edits().tolist() == [[0, 2, 2, 0], [0, 0, 33, 1]]
    m.rollback_token(5)
    assert m.drain_edits().tolist() == [[0, 0, 32, 1]]
    m.release(5)
    assert m.drain_edits().tolist() == [[0, 0, 0, 1]]
    assert m.drain_edits().shape == (0, 4)


# ---- cache.rs, prefix cache (:773-968) -------------------------------------------------------

def prompt(length, start=0):
    return list(range(start, start + length))


def snapshot(m, seq, tokens):
    """A snapshot at the end of prompt `tokens` for sequence `seq` (cache.rs:777-782)."""
    number = m.reserve_snapshot()
    assert number is not None
    m.commit_snapshot(number, seq, tokens)
    return number


def test_prefix_hit_shares_full_pages_and_copies_the_tail(built_library):
    # cache.rs:784-806
    m = CacheManager(4, 100, 64)
    m.enable_prefix_cache(2)
    assert m.admit_prompt(1, prompt(150)) == {"reused": 0, "restore": None}
    snap = snapshot(m, 1, prompt(150))
    owner = m.sequence(1)["blocks"]
    m.release(1)
    admission = m.admit_prompt(2, prompt(200))
    assert admission["reused"] == 150 and admission["restore"]["snapshot"] == snap
    blocks = m.sequence(2)["blocks"]
    # two full pages are shared, the third (tail 150 - 128) is a copy
    assert blocks[:2] == owner[:2]
    assert admission["restore"]["copy_block"] == (owner[2], blocks[2]) and blocks[2] != owner[2]
    assert len(blocks) == 4 and m.prefix_stats()["hits"] == 1
    # the device tables follow: every page of the new sequence and its length were recorded
    edits = m.drain_edits()
    slot = m.sequence(2)["state_slot"]
    mine = [e for e in edits.tolist() if e[0] == slot]
    assert [e[2] for e in mine if e[3] == 0][-4:] == blocks and [slot, 0, 200, 1] in mine


def test_aligned_prefix_needs_no_copy(built_library):
    # cache.rs:808-818
    m = CacheManager(4, 100, 64)
    m.enable_prefix_cache(1)
    m.admit_prompt(1, prompt(128))
    snapshot(m, 1, prompt(128))
    m.release(1)
    admission = m.admit_prompt(2, prompt(130))
    assert admission["reused"] == 128 and admission["restore"]["copy_block"] is None


def test_identical_prompt_does_not_hit(built_library):
    # cache.rs:820-830: at least one prompt token has to be run
    m = CacheManager(4, 100, 64)
    m.enable_prefix_cache(1)
    m.admit_prompt(1, prompt(100))
    snapshot(m, 1, prompt(100))
    m.release(1)
    assert m.admit_prompt(2, prompt(100))["reused"] == 0


def test_different_prefix_misses(built_library):
    # cache.rs:832-842
    m = CacheManager(4, 100, 64)
    m.enable_prefix_cache(1)
    m.admit_prompt(1, prompt(100))
    snapshot(m, 1, prompt(100))
    m.release(1)
    other = prompt(150)
    other[10] = 999_999
    assert m.admit_prompt(2, other)["reused"] == 0


def test_shared_pages_return_to_the_pool_only_after_every_owner(built_library):
    # cache.rs:844-864
    m = CacheManager(4, 20, 64)
    m.enable_prefix_cache(1)
    total = m.free_blocks()
    m.admit_prompt(1, prompt(150))
    snapshot(m, 1, prompt(150))
    m.release(1)
    assert m.free_blocks() == total - 3  # the entry holds three pages after the owner leaves
    m.admit_prompt(2, prompt(200))
    m.finish_restore(0)
    m.release(2)
    assert m.free_blocks() == total - 3
    m.admit(3, 20 * 64)                  # pool pressure evicts the entry and returns its pages
    assert m.prefix_entries() == 0 and m.prefix_stats()["evictions"] == 1
    m.release(3)
    assert m.free_blocks() == total


def test_page_pressure_skips_entry_held_by_live_sequence(built_library):
    # cache.rs:870-888
    m = CacheManager(4, 10, 64)
    m.enable_prefix_cache(2)
    m.admit_prompt(1, prompt(150))
    snapshot(m, 1, prompt(150))
    idle = prompt(150, 1000)
    m.admit_prompt(2, idle)
    snapshot(m, 2, idle)
    m.release(2)
    assert m.free_blocks() == 4
    m.admit(3, 6 * 64)
    assert m.prefix_stats()["evictions"] == 1 and m.prefix_entries() == 1
    m.release(3)
    assert m.admit_prompt(4, prompt(200))["reused"] == 150


def test_page_pressure_fails_without_evicting_live_entries(built_library):
    # cache.rs:890-899
    m = CacheManager(4, 4, 64)
    m.enable_prefix_cache(1)
    m.admit_prompt(1, prompt(150))
    snapshot(m, 1, prompt(150))
    with rejected("NoKvBlocks"):
        m.admit(2, 2 * 64)
    assert m.prefix_entries() == 1 and m.prefix_stats()["evictions"] == 0


def test_snapshot_pressure_keeps_entry_of_running_sequence(built_library):
    # cache.rs:901-917
    m = CacheManager(4, 100, 64)
    m.enable_prefix_cache(2)
    m.admit_prompt(1, prompt(150))
    snapshot(m, 1, prompt(150))
    idle = prompt(150, 1000)
    m.admit_prompt(2, idle)
    snapshot(m, 2, idle)
    m.release(2)
    fresh = prompt(100, 5000)            # no slots: the idle entry goes, even though it is newer
    m.admit_prompt(3, fresh)
    snapshot(m, 3, fresh)
    assert m.admit_prompt(4, prompt(200, 1000))["reused"] == 0
    assert m.admit_prompt(5, prompt(200))["reused"] == 150


def test_snapshot_pressure_evicts_superseded_entry_first(built_library):
    # cache.rs:919-944
    m = CacheManager(4, 100, 64)
    m.enable_prefix_cache(2)
    m.admit_prompt(1, prompt(100))       # turn N and turn N + 1 of one dialog: N lies inside N + 1
    snapshot(m, 1, prompt(100))
    m.release(1)
    admission = m.admit_prompt(2, prompt(200))
    m.finish_restore(admission["restore"]["snapshot"])
    snapshot(m, 2, prompt(180))
    m.release(2)
    branch = prompt(100) + [999_999]     # N was touched last - by age N + 1 would have gone
    admission = m.admit_prompt(3, branch)
    assert admission["reused"] == 100
    m.finish_restore(admission["restore"]["snapshot"])
    m.release(3)
    other = prompt(100, 5000)
    m.admit_prompt(4, other)
    snapshot(m, 4, other)
    m.release(4)
    assert m.admit_prompt(5, prompt(250))["reused"] == 180


def test_pinned_entry_survives_until_restored(built_library):
    # cache.rs:946-959
    m = CacheManager(4, 100, 64)
    m.enable_prefix_cache(1)
    m.admit_prompt(1, prompt(100))
    snap = snapshot(m, 1, prompt(100))
    m.release(1)
    m.admit_prompt(2, prompt(120))
    assert m.reserve_snapshot() is None  # the only snapshot slot is pinned
    m.finish_restore(snap)
    assert m.reserve_snapshot() == snap and m.prefix_entries() == 0


def test_disabled_cache_is_plain_admission(built_library):
    # cache.rs:961-966
    m = CacheManager(4, 100, 64)
    assert m.reserve_snapshot() is None
    assert m.admit_prompt(1, prompt(100)) == {"reused": 0, "restore": None}
    with rejected("AlreadyAdmitted"):
        m.admit_prompt(1, prompt(100))


# ---- scheduler.rs ----------------------------------------------------------------------------

def scheduler(states, blocks, max_seqs, tokens):
    return Scheduler(max_seqs, tokens, states, blocks, 64)  # scheduler.rs:673-678


def test_long_prefill_is_split_into_chunks(built_library):
    # scheduler.rs:688-708
    s = scheduler(2, 100, 2, 4)
    s.submit(1, 10, 1)
    for offset, tokens in [(0, 4), (4, 4), (8, 2)]:
        batch = s.next_batch()
        assert batch["prefill"] == [(1, offset, tokens)] and batch["decode"] == []
        s.complete_batch()
    assert s.next_batch()["decode"] == [1]


def test_continuous_batch_mixes_decode_and_prefill(built_library):
    # scheduler.rs:710-729
    s = scheduler(2, 100, 2, 8)
    s.submit(1, 4, 2)
    s.next_batch()
    s.complete_batch()
    s.submit(2, 4, 1)
    batch = s.next_batch()
    assert batch["decode"] == [1] and batch["prefill"] == [(2, 0, 4)]


def test_length_completion_releases_both_resources(built_library):
    # scheduler.rs:731-755
    s = scheduler(1, 2, 1, 64)
    s.submit(1, 64, 2)
    s.next_batch()
    s.complete_batch()
    s.next_batch()
    assert s.complete_batch() == []
    s.next_batch()
    assert s.complete_batch() == [(1, 2, "Length")]
    assert s.active() == 0 and s.cache.states_in_use() == 0 and s.cache.free_blocks() == 2


def test_kv_blocked_head_does_not_hide_smaller_request(built_library):
    # scheduler.rs:757-772
    s = scheduler(3, 4, 3, 256)
    s.submit(1, 128, 2)
    s.next_batch()
    s.complete_batch()
    s.submit(2, 192, 1)
    s.submit(3, 63, 1)
    batch = s.next_batch()
    assert batch["decode"] == [1] and batch["prefill"][0][0] == 3 and s.waiting() == 1


def test_abort_rolls_back_decode_reservation(built_library):
    # scheduler.rs:774-790
    s = scheduler(1, 2, 1, 64)
    s.submit(1, 64, 2)
    s.next_batch()
    s.complete_batch()
    assert s.next_batch()["decode"] == [1]
    assert s.cache.sequence(1)["tokens"] == 65 and s.cache.free_blocks() == 0
    s.abort_batch()
    assert s.cache.sequence(1)["tokens"] == 64 and s.cache.free_blocks() == 1
    assert s.next_batch()["decode"] == [1]


def test_one_in_flight_batch_is_enforced(built_library):
    # scheduler.rs:792-798
    s = scheduler(1, 2, 1, 64)
    s.submit(1, 1, 1)
    s.next_batch()
    with rejected("BatchInFlight"):
        s.next_batch()


def test_invalid_requests_are_rejected_before_queueing(built_library):
    # scheduler.rs:800-814
    s = scheduler(1, 2, 1, 64)
    with rejected("EmptyPrompt"):
        s.submit(1, 0, 1)
    with rejected("ContextTooLong"):
        s.submit(2, 129, 1)
    with rejected("NoOutputTokens"):
        s.submit(4, 1, 0)
    s.submit(3, 1, 1)
    with rejected("Duplicate"):
        s.submit(3, 1, 1)


def test_stopped_sequence_is_released(built_library):
    # scheduler.rs:816-828
    s = scheduler(1, 2, 1, 64)
    s.submit(1, 1, 10)
    s.next_batch()
    s.complete_batch()
    s.next_batch()
    assert s.complete_batch([1]) == [(1, 1, "Stopped")]
    assert s.active() == 0


def test_lifetime_reservation_prevents_decode_deadlock(built_library):
    # scheduler.rs:830-852
    s = scheduler(2, 2, 2, 64)
    s.submit(1, 64, 1)
    s.submit(2, 64, 1)
    prefill = s.next_batch()
    assert len(prefill["prefill"]) == 1 and s.committed_kv_blocks() == 2 and s.waiting() == 1
    s.complete_batch()
    assert s.next_batch()["decode"] == [1]
    s.complete_batch()
    assert s.committed_kv_blocks() == 0
    assert s.next_batch()["prefill"][0][0] == 2


def test_cancellation_releases_admitted_request(built_library):
    # scheduler.rs:854-867
    s = scheduler(1, 2, 1, 64)
    s.submit(1, 64, 10)
    s.next_batch()
    with rejected("SequenceInFlight"):
        s.cancel(1)
    s.complete_batch()
    assert s.cancel(1) is True
    assert s.active() == 0 and s.cache.states_in_use() == 0 and s.cache.free_blocks() == 2
    assert s.cancel(1) is False


def test_queued_request_can_be_cancelled_without_admission(built_library):
    # scheduler.rs:869-877
    s = scheduler(1, 2, 1, 64)
    s.submit(1, 64, 10)
    assert s.cancel(1) is True
    assert s.waiting() == 0 and s.active() == 0 and s.next_batch() is None


def test_complete_batch_validates_stopped_ids(built_library):
    # scheduler.rs:418-426 and :388-396
    s = scheduler(2, 10, 2, 64)
    with rejected("NoBatchInFlight"):
        s.complete_batch()
    with rejected("NoBatchInFlight"):
        s.abort_batch()
    s.submit(1, 4, 5)
    s.next_batch()
    s.complete_batch()
    s.next_batch()
    with rejected("InvalidStopped"):
        s.complete_batch([9])
    with rejected("DuplicateStopped"):
        s.complete_batch([1, 1])
    assert s.remaining_tokens(1) == 5
    s.complete_batch()
    assert s.remaining_tokens(1) == 4 and s.remaining_tokens(2) is None


def test_complete_batch_multi_counts_the_tokens_a_sequence_produced(built_library):
    # scheduler.rs:392-500 (the reference has no test of its own for this; the cases follow its doc comment
    # and its checks at :407-414 and :468-472)
    s = scheduler(2, 10, 2, 64)
    with rejected("NoBatchInFlight"):
        s.complete_batch_multi([], [(1, 2)])
    s.submit(1, 4, 7)
    s.submit(2, 4, 3)
    s.next_batch()
    s.complete_batch()
    assert sorted(s.next_batch()["decode"]) == [1, 2]
    with rejected("Invariant"):
        s.complete_batch_multi([], [(1, 0)])           # a step produces at least one token
    with rejected("InvalidStopped"):
        s.complete_batch_multi([], [(9, 2)])           # not a decode sequence of this batch
    assert s.complete_batch_multi([], [(1, 3)]) == []  # sequence 2 is not named: one token
    assert s.remaining_tokens(1) == 4 and s.remaining_tokens(2) == 2
    s.next_batch()
    # more tokens than the request has left: capped at its length; the first entry of a sequence counts
    done = s.complete_batch_multi([], [(1, 9), (2, 2), (2, 1)])
    assert sorted(done) == [(1, 7, "Length"), (2, 3, "Length")]
    assert s.active() == 0 and s.cache.states_in_use() == 0


def test_decode_rows_take_priority_over_admission(built_library):
    # scheduler.rs:301-323: decode fills the batch first; a full batch admits nobody
    s = scheduler(4, 100, 2, 64)
    for seq in (1, 2, 3):
        s.submit(seq, 4, 8)
    assert [c[0] for c in s.next_batch()["prefill"]] == [1, 2]
    s.complete_batch()
    for _ in range(3):
        batch = s.next_batch()
        assert batch["decode"] == [1, 2] and batch["prefill"] == []
        s.complete_batch()
    assert s.waiting() == 1


# ---- layout.rs ---------------------------------------------------------------------------------

def test_mixed_batch_becomes_csr_metadata(built_library):
    # layout.rs:164-189
    cache = CacheManager(2, 10, 64)
    cache.admit(1, 64)
    cache.append_token(1)
    cache.admit(2, 100)
    layout = build_layout(cache, decode=[1], prefill=[(2, 32, 16)])
    assert layout["num_decode"] == 1
    assert layout["seq_ids"] == [1, 2]
    assert layout["state_slots"] == [0, 1]
    assert layout["position_starts"] == [64, 32]
    assert layout["context_lens"] == [65, 48]
    assert layout["token_offsets"] == [0, 1, 17]
    assert layout["block_table_offsets"] == [0, 2, 3]
    assert layout["block_ids"] == [0, 1, 2]


def test_duplicate_or_missing_sequence_is_rejected(built_library):
    # layout.rs:191-222
    cache = CacheManager(1, 2, 64)
    cache.admit(1, 1)
    cache.append_token(1)
    with rejected("DuplicateSequence") as error:
        build_layout(cache, decode=[1], prefill=[(1, 0, 1)])
    assert error.value.offender == 1
    with rejected("MissingSequence") as error:
        build_layout(cache, decode=[7])
    assert error.value.offender == 7


def test_invalid_prefill_range_is_rejected(built_library):
    # layout.rs:224-239
    cache = CacheManager(1, 2, 64)
    cache.admit(1, 10)
    with rejected("InvalidPrefillRange"):
        build_layout(cache, prefill=[(1, 8, 4)])


# ---- the scheduler's side of the prefix cache (reference tests, crates/qwc-runtime/src/scheduler.rs:877-985) ----

def drain(s):
    """Runs what is queued to the end; the batches it took."""
    batches = []
    while (batch := s.next_batch()) is not None:
        s.complete_batch()
        batches.append(batch)
    return batches


def test_next_turn_continues_from_the_previous_prompt(built_library):
    s = scheduler(2, 100, 2, 512)
    s.enable_prefix_cache(4)
    s.submit_prompt(1, range(150), 2, 150)
    first = drain(s)
    # the prompt ended in the very first step: so did the snapshot
    assert len(first[0]["saves"]) == 1 and first[0]["restores"] == []
    assert s.cache.prefix_entries() == 1

    s.submit_prompt(2, range(200), 1, 200)
    batch = s.next_batch()
    assert batch["prefill"] == [(2, 150, 50)]
    assert len(batch["restores"]) == 1
    assert batch["restores"][0]["snapshot"] == first[0]["saves"][0]["snapshot"]
    assert batch["restores"][0]["copy_block"] is not None
    s.complete_batch()
    assert s.cache.prefix_stats()["reused_tokens"] == 150


def test_aborted_step_keeps_the_restore_and_frees_the_save(built_library):
    s = scheduler(2, 100, 2, 512)
    s.enable_prefix_cache(1)
    s.submit_prompt(1, range(100), 1, 100)
    drain(s)

    s.submit_prompt(2, range(130), 1, 130)
    batch = s.next_batch()
    assert len(batch["restores"]) == 1
    assert batch["saves"] == []  # the only slot belongs to a pinned entry: nowhere to capture
    s.abort_batch()

    retry = s.next_batch()
    assert retry["restores"] == batch["restores"]
    assert retry["prefill"] == batch["prefill"]


def test_cancelling_before_restore_unpins_the_entry(built_library):
    s = scheduler(2, 100, 2, 512)
    s.enable_prefix_cache(1)
    s.submit_prompt(1, range(100), 1, 100)
    drain(s)
    s.submit_prompt(2, range(130), 1, 130)
    assert s.next_batch() is not None
    s.abort_batch()
    assert s.cancel(2)
    # the entry can be evicted again: a new snapshot takes its slot
    s.submit_prompt(3, [t + 7 for t in range(64)], 1, 64)
    assert len(s.next_batch()["saves"]) == 1


def test_prefill_is_cut_at_the_history_boundary(built_library):
    """150 prompt tokens of which the last 6 open the answer: the snapshot lands at 144 and the next
    turn continues from exactly there."""
    s = scheduler(2, 100, 2, 512)
    s.enable_prefix_cache(2)
    s.submit_prompt(1, range(150), 1, 144)
    first = s.next_batch()
    assert first["prefill"][0][2] == 144
    assert len(first["saves"]) == 1
    s.complete_batch()
    tail = s.next_batch()
    assert tail["prefill"] == [(1, 144, 6)]
    assert tail["saves"] == []
    s.complete_batch()
    drain(s)

    following = list(range(144)) + list(range(1000, 1100))
    s.submit_prompt(2, following, 1, 238)
    batch = s.next_batch()
    assert batch["prefill"][0][1] == 144
    assert len(batch["restores"]) == 1


def test_aborted_save_returns_its_snapshot_slot(built_library):
    """abort_batch cancels the step's captures: with one slot, the retry can reserve it again."""
    s = scheduler(2, 100, 2, 512)
    s.enable_prefix_cache(1)
    s.submit_prompt(1, range(100), 1, 100)
    first = s.next_batch()
    assert len(first["saves"]) == 1
    s.abort_batch()
    assert s.cache.prefix_entries() == 0
    retry = s.next_batch()
    assert retry["saves"] == first["saves"]
    s.complete_batch()
    assert s.cache.prefix_entries() == 1


def test_submit_prompt_checks_its_lengths(built_library):
    s = scheduler(2, 100, 2, 512)
    with pytest.raises(ValueError):
        s.submit_prompt(1, range(10), 1, 11)
    s.submit_prompt(1, range(10), 1, 10)
    with pytest.raises(RuntimeError_) as error:
        s.submit_prompt(1, range(10), 1, 10)
    assert error.value.name == "Duplicate"
    # without a prefix cache a prompt is plain admission: no cut, no ops
    batch = s.next_batch()
    assert batch["prefill"] == [(1, 0, 10)] and batch["saves"] == [] and batch["restores"] == []


def test_host_layout_agrees_with_the_oracle_statement(built_library):
    """The C++ BatchLayout and the oracle's restatement of the same file give identical arrays."""
    from oracle import oracle

    page = 16
    cache = CacheManager(8, 400, page)
    rng = np.random.default_rng(3)
    ids = [11, 12, 13, 14, 15]
    for seq in ids:
        cache.admit(seq, int(rng.integers(1, 300)))
        cache.append_token(seq)
    order = [13, 11, 15, 12]
    layout = build_layout(cache, decode=order)
    capacity, max_blocks = 8, 32
    seq_tokens = np.zeros(capacity, np.uint32)
    seq_blocks = np.zeros((capacity, max_blocks), np.uint32)
    counts = np.zeros(capacity, np.uint32)
    for seq in ids:
        info = cache.sequence(seq)
        seq_tokens[info["state_slot"]] = info["tokens"]
        counts[info["state_slot"]] = len(info["blocks"])
        seq_blocks[info["state_slot"], :len(info["blocks"])] = info["blocks"]
    want = oracle.layout_decode(layout["state_slots"], seq_tokens, seq_blocks, counts, max_blocks, page)
    assert want["status"] == 0
    assert want["positions"].tolist() == layout["position_starts"]
    assert want["context_lengths"].tolist() == layout["context_lens"]
    assert want["block_table_offsets"].tolist() == layout["block_table_offsets"]
    assert want["block_ids"].tolist() == layout["block_ids"]


def test_a_drain_carries_one_edit_per_table_word(built_library):
    """The device applies a drain with one thread per edit and no order among them, so the host
    keeps only the last edit of a word: a slot that is released and admitted again within one drain
    (the state pool hands the newest free slot out first) sends one token count, not two."""
    m = CacheManager(2, 8, 16)
    m.admit(1, 20)
    m.drain_edits()
    m.release(1)
    m.admit(2, 40)  # takes the slot that was just released
    edits = m.drain_edits().tolist()
    words = [(slot, kind, index if kind == 0 else 0) for slot, index, _, kind in edits]
    assert len(words) == len(set(words))
    assert [0, 0, 40, 1] in edits and [0, 0, 0, 1] not in edits
    m.append_token(2)
    m.rollback_token(2)
    assert m.drain_edits().tolist() == [[0, 0, 40, 1]]
