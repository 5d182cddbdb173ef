"""Randomised walks over the host runtime (scheduler + cache manager + prefix cache), checked after every
operation against invariants the device side depends on:

* the drained table edits, replayed onto a shadow copy of the device tables, reproduce the token count
  and the page list of every admitted sequence (the protocol `page_table_apply_kernel` consumes: one
  thread per edit and no order among them, so a drain must not name a table word twice);
* no page is lost or handed out twice: free pages plus pages referenced by sequences and cached
  prefixes are the pool; a page shared by several owners is shared through a cached prefix only;
* the state pool follows the sequences; reservations never exceed the pool; every request ends
  (lifetime reservation: no decode deadlock) and gives everything back.

Seeded numpy walks, not a fuzzer: the same walks every run."""

import numpy as np
import pytest

from qwencore_b200.engine import RuntimeError_, Scheduler, Worker

PAGE = 16


class Shadow:
    """The device copy of (tokens, page list) per state slot, as the edit protocol maintains it."""

    def __init__(self, slots, max_pages):
        self.tokens = np.zeros(slots, dtype=np.int64)
        self.pages = np.full((slots, max_pages), -1, dtype=np.int64)

    def apply(self, edits):
        words = set()
        for slot, index, value, kind in edits.tolist():
            word = (slot, 0 if kind else 1, index if kind == 0 else 0)
            assert word not in words, f"a drain names table word {word} twice"
            words.add(word)
            if kind == 0:
                self.pages[slot, index] = value
            elif kind == 1:
                self.tokens[slot] = value
            else:
                assert kind == 2
                self.tokens[slot] += value


class Walk:
    def __init__(self, seed, states, pages, max_seqs, budget, snapshots):
        self.rng = np.random.default_rng(seed)
        self.states, self.pool = states, pages
        self.scheduler = Scheduler(max_seqs, budget, states, pages, PAGE)
        if snapshots:
            self.scheduler.enable_prefix_cache(snapshots)
        self.cache = self.scheduler.cache
        self.shadow = Shadow(states, pages)
        self.live = {}      # id -> [prompt length, max_new_tokens, generated]
        self.finished = {}  # id -> (generated, reason)
        self.next_id = 1
        self.histories = [list(self.rng.integers(0, 50, int(n))) for n in self.rng.integers(20, 120, 4)]

    # ---- operations ----
    def submit(self):
        rng = self.rng
        max_new = int(rng.integers(1, 12))
        seq = self.next_id
        self.next_id += 1
        if rng.random() < 0.6:  # a turn of one of a few dialogs: shared history, then something new
            history = self.histories[int(rng.integers(len(self.histories)))]
            keep = int(rng.integers(max(1, len(history) // 2), len(history) + 1))
            prompt = history[:keep] + list(rng.integers(50, 100, int(rng.integers(1, 30))))
            snapshot_at = int(rng.integers(0, len(prompt) + 1)) if rng.random() < 0.3 else keep
            try:
                self.scheduler.submit_prompt(seq, prompt, max_new, min(snapshot_at, len(prompt)))
            except RuntimeError_:
                return
            length = len(prompt)
        else:
            length = int(rng.integers(1, 200))
            try:
                self.scheduler.submit(seq, length, max_new)
            except RuntimeError_:
                return
        self.live[seq] = [length, max_new, 0]

    def step(self, abort=False):
        batch = self.scheduler.next_batch()
        if batch is None:
            return False
        for seq in batch["decode"]:
            assert seq in self.live
        if abort:
            self.scheduler.abort_batch()
            return True
        stopped = [seq for seq in batch["decode"] if self.rng.random() < 0.08]
        for seq in batch["decode"]:
            self.live[seq][2] += 1
        for seq, generated, reason in self.scheduler.complete_batch(stopped):
            length, max_new, counted = self.live.pop(seq)
            assert generated == counted and 1 <= generated <= max_new
            assert reason == ("Stopped" if seq in stopped else "Length")
            if reason == "Length":
                assert generated == max_new
            self.finished[seq] = (generated, reason)
        for seq in stopped:
            assert seq in self.finished
        return True

    def cancel(self):
        if not self.live:
            return
        seq = int(self.rng.choice(list(self.live)))
        assert self.scheduler.cancel(seq)
        del self.live[seq]
        assert self.scheduler.remaining_tokens(seq) is None

    # ---- invariants ----
    def check(self):
        self.shadow.apply(self.cache.drain_edits())
        admitted, slots, owners = 0, set(), {}
        for seq, (length, max_new, generated) in self.live.items():
            info = self.cache.sequence(seq)
            if info is None:
                continue  # still waiting
            admitted += 1
            slot = info["state_slot"]
            assert slot < self.states and slot not in slots, "two sequences in one state slot"
            slots.add(slot)
            assert info["tokens"] <= length + generated
            assert len(info["blocks"]) >= -(-info["tokens"] // PAGE)
            # the device tables say the same
            assert self.shadow.tokens[slot] == info["tokens"], (seq, slot)
            assert self.shadow.pages[slot, :len(info["blocks"])].tolist() == info["blocks"], (seq, slot)
            for page in info["blocks"]:
                assert 0 <= page < self.pool
                owners.setdefault(page, []).append(seq)
            remaining = self.scheduler.remaining_tokens(seq)
            assert remaining == max_new - generated
        assert self.cache.states_in_use() == admitted == self.scheduler.active()
        assert self.scheduler.waiting() == len(self.live) - admitted
        shared = [page for page, who in owners.items() if len(who) > 1]
        if self.cache.prefix_entries() == 0 and self.cache.prefix_stats()["hits"] == 0:
            assert not shared, "a page in two sequences without a cached prefix"
        # no page both free and owned: owned pages and free pages fit the pool, and without cached
        # prefixes they are exactly the pool
        assert len(owners) + self.cache.free_blocks() <= self.pool
        if self.cache.prefix_entries() == 0:
            assert len(owners) + self.cache.free_blocks() == self.pool
        assert self.scheduler.committed_kv_blocks() <= self.pool
        reserved = sum(-(-(length + max_new) // PAGE) for seq, (length, max_new, _) in self.live.items()
                       if self.cache.sequence(seq) is not None)
        assert self.scheduler.committed_kv_blocks() == reserved

    def run(self, operations):
        for _ in range(operations):
            draw = self.rng.random()
            if draw < 0.35:
                self.submit()
            elif draw < 0.85:
                self.step()
            elif draw < 0.93:
                self.step(abort=True)
            else:
                self.cancel()
            self.check()
        # drain: everything that is left ends without new arrivals
        for _ in range(10_000):
            if not self.live:
                break
            assert self.step(), "requests left but nothing to run: deadlock"
            self.check()
        assert not self.live
        assert self.cache.states_in_use() == 0 and self.scheduler.committed_kv_blocks() == 0
        # cached prefixes may still hold pages; without them the pool is whole again
        if self.cache.prefix_entries() == 0:
            assert self.cache.free_blocks() == self.pool


@pytest.mark.parametrize("seed", range(6))
def test_random_walk_without_prefix_cache(built_library, seed):
    Walk(seed, states=6, pages=64, max_seqs=4, budget=96, snapshots=0).run(400)


@pytest.mark.parametrize("seed", range(6))
def test_random_walk_with_prefix_cache(built_library, seed):
    walk = Walk(100 + seed, states=6, pages=96, max_seqs=4, budget=96, snapshots=3)
    walk.run(500)
    stats = walk.cache.prefix_stats()
    assert stats["lookups"] > 0 and stats["hits"] > 0 and stats["evictions"] > 0  # the walk reaches all of it


def test_random_walk_under_page_pressure(built_library):
    """A pool so small that admission usually waits for pages: nothing deadlocks, nothing leaks."""
    for seed in range(4):
        Walk(200 + seed, states=8, pages=24, max_seqs=8, budget=64, snapshots=2).run(400)


@pytest.mark.parametrize("seed", range(4))
def test_random_traffic_through_the_worker(built_library, seed):
    """Requests, stop tokens, sinks that stop and clients that leave, at random: every request that is not
    abandoned ends with exactly one Done whose count is what was emitted, and both pools are whole again."""
    rng = np.random.default_rng(300 + seed)
    scheduler = Scheduler(4, 96, 6, 96, PAGE)
    scheduler.enable_prefix_cache(3)
    eos = 7
    events, stop_at, abandoned = {}, {}, set()

    def execute(step):
        return [eos if rng.random() < 0.05 else int(rng.integers(8, 1000)) for _ in step["seq_ids"]]

    def sink(seq, kind, value, reason):
        events.setdefault(seq, []).append((kind, value, reason))
        if kind == "token":
            assert value != eos or ignore[seq]
            return sum(1 for k, _, _ in events[seq] if k == "token") >= stop_at.get(seq, 1 << 30)
        return False

    worker = Worker(scheduler, execute, sink, eos_ids=[eos])
    budgets, ignore = {}, {}
    history = list(rng.integers(0, 50, 90))
    next_id = 1
    for _ in range(300):
        draw = rng.random()
        if draw < 0.3:
            keep = int(rng.integers(20, 91))
            prompt = history[:keep] + list(rng.integers(50, 100, int(rng.integers(1, 20))))
            budgets[next_id], ignore[next_id] = int(rng.integers(1, 10)), bool(rng.random() < 0.3)
            if rng.random() < 0.2:
                stop_at[next_id] = int(rng.integers(1, 6))
            worker.submit(next_id, prompt, budgets[next_id], history_tokens=keep, ignore_eos=ignore[next_id])
            next_id += 1
        elif draw < 0.36 and next_id > 1:
            seq = int(rng.integers(1, next_id))
            abandoned.add(seq)
            worker.abandon(seq)
        status, _ = worker.iterate()
        assert status == 0
    for _ in range(2000):
        status, progressed = worker.iterate()
        assert status == 0
        if not progressed and worker.jobs() == 0:
            break
    assert worker.jobs() == 0 and worker.aborted_steps() == 0 and worker.raised is None
    ended = 0
    for seq in range(1, next_id):
        mine = events.get(seq, [])
        done = [(value, reason) for kind, value, reason in mine if kind == "done"]
        tokens = [value for kind, value, _ in mine if kind == "token"]
        assert not [e for e in mine if e[0] == "error"]
        if not done:
            assert seq in abandoned, f"request {seq} never ended"
            continue
        ended += 1
        assert len(done) == 1 and mine[-1][0] == "done"
        count, reason = done[0]
        assert count == len(tokens) <= budgets[seq]
        if reason == 0:  # Length
            assert count == budgets[seq]
        else:  # stopped by its sink at the token it named, or by an end-of-sequence token it does not ignore
            assert count == stop_at.get(seq) or not ignore[seq]
    assert ended > 20
    assert scheduler.active() == 0 and scheduler.waiting() == 0 and scheduler.cache.states_in_use() == 0
    assert scheduler.committed_kv_blocks() == 0
