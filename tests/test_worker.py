"""The serving worker loop at token level (crates/qwc-engine/src/bin/serve.rs:777-1074) against a host
stand-in for the executor: what each step is fed, the stop rules, rollback and fail-all on an executor
error (the failure is made on the host: the stand-in returns an error code), refused requests,
abandoned jobs, the threaded loop, and the prefix-cache ops a step carries."""

import threading

from qwencore_b200.engine import Scheduler, Worker


class Recorder:
    """Collects events; `stop_after[seq] = n` stops a sequence at its n-th token (a stop string or a
    client that hung up, in the reference)."""

    def __init__(self, stop_after=None):
        self.events = []
        self.stop_after = stop_after or {}

    def __call__(self, seq_id, kind, value, reason):
        self.events.append((seq_id, kind, value, reason))
        if kind == "token":
            return len(self.tokens(seq_id)) >= self.stop_after.get(seq_id, 1 << 30)
        return False

    def tokens(self, seq_id):
        return [value for seq, kind, value, _ in self.events if seq == seq_id and kind == "token"]

    def of(self, seq_id, kind):
        return [(value, reason) for seq, k, value, reason in self.events if seq == seq_id and k == kind]


class Executor:
    """Samples `1000 * id + position of the last row`, so a test can tell which token went where."""

    def __init__(self, fail_at_step=None, code=700, sample=None):
        self.steps = []
        self.fail_at_step = fail_at_step
        self.code = code
        self.sample = sample

    def __call__(self, step):
        self.steps.append(step)
        if self.fail_at_step is not None and len(self.steps) == self.fail_at_step:
            return self.code
        if self.sample is not None:
            return self.sample(step)
        return [1000 * seq + context for seq, context in zip(step["seq_ids"], step["context_lens"])]


def drain(worker, limit=200):
    for _ in range(limit):
        status, progressed = worker.iterate()
        if status != 0 or (not progressed and worker.jobs() == 0):
            return status
    raise AssertionError("the worker did not come to rest")


def test_each_step_is_fed_prompt_slices_and_the_previous_samples(built_library):
    scheduler = Scheduler(2, 64, 2, 100, 16)
    executor, sink = Executor(), Recorder()
    worker = Worker(scheduler, executor, sink)
    worker.submit(1, range(100, 120), 3)
    worker.submit(2, range(200, 270), 2)
    assert drain(worker) == 0
    first, second, third, fourth = executor.steps
    # 64 tokens per step: all of prompt 1, the first 44 tokens of prompt 2
    assert first["num_decode"] == 0 and first["seq_ids"] == [1, 2]
    assert first["tokens"] == [list(range(100, 120)), list(range(200, 244))]
    # sequence 1 decodes the token its prefill sampled; prompt 2 goes on where it stopped
    assert second["num_decode"] == 1 and second["seq_ids"] == [1, 2]
    assert second["tokens"] == [[1000 + 20], list(range(244, 270))]
    assert second["position_starts"] == [20, 44]
    # (the scheduler rotates its decode order: compare per sequence)
    assert dict(zip(third["seq_ids"], third["tokens"])) == {1: [1000 + 21], 2: [2000 + 70]}
    assert dict(zip(fourth["seq_ids"], fourth["tokens"])) == {1: [1000 + 22], 2: [2000 + 71]}
    # a decode row emits the token it was fed; the last sample of a sequence is never emitted
    assert sink.tokens(1) == [1020, 1021, 1022] and sink.of(1, "done") == [(3, 0)]
    assert sink.tokens(2) == [2070, 2071] and sink.of(2, "done") == [(2, 0)]
    assert worker.steps() == 4 and worker.aborted_steps() == 0
    assert scheduler.active() == 0 and scheduler.cache.free_blocks() == 100
    # the step carried the page-table edits of its plan: the first one admits both sequences
    assert any(kind == 1 for _, _, _, kind in first["edits"])


def test_end_of_sequence_token_stops_without_being_emitted(built_library):
    scheduler = Scheduler(2, 64, 2, 100, 16)
    # the third sample of every sequence is the end-of-sequence token
    executor = Executor(sample=lambda step: [7 if context == 12 else 50 + context for context in step["context_lens"]])
    sink = Recorder()
    worker = Worker(scheduler, executor, sink, eos_ids=[7, 9])
    worker.submit(1, range(10), 8)
    worker.submit(2, range(10), 8, ignore_eos=True)
    assert drain(worker) == 0
    # prefill samples 60, then 61, then 7: sequence 1 ends when it is FED the 7 (one more step ran)
    assert sink.tokens(1) == [60, 61] and sink.of(1, "done") == [(2, 1)]
    # the same tokens with ignore_eos: the 7 is an ordinary token and the budget ends the request
    assert sink.tokens(2) == [60, 61, 7, 63, 64, 65, 66, 67] and sink.of(2, "done") == [(8, 0)]


def test_the_sink_stops_a_sequence_after_the_token_it_took(built_library):
    scheduler = Scheduler(2, 64, 2, 100, 16)
    sink = Recorder(stop_after={1: 2})
    worker = Worker(scheduler, Executor(), sink)
    worker.submit(1, range(10), 8)
    assert drain(worker) == 0
    assert sink.tokens(1) == [1010, 1011] and sink.of(1, "done") == [(2, 1)]
    assert scheduler.cache.states_in_use() == 0 and scheduler.cache.free_blocks() == 100


def test_executor_failure_rolls_the_step_back_and_fails_every_job(built_library):
    scheduler = Scheduler(2, 64, 2, 100, 16)
    executor, sink = Executor(fail_at_step=3, code=700), Recorder()
    worker = Worker(scheduler, executor, sink)
    worker.submit(1, range(10), 8)
    worker.submit(2, range(10), 8)
    assert worker.iterate() == (0, True) and worker.iterate() == (0, True)
    remaining = scheduler.remaining_tokens(1)
    blocks = scheduler.cache.free_blocks()
    status, progressed = worker.iterate()
    assert (status, progressed) == (700, False)
    # the plan was rolled back: nothing of the failed step is committed, no batch is left in flight
    assert worker.aborted_steps() == 1 and worker.steps() == 2
    assert scheduler.remaining_tokens(1) == remaining and scheduler.cache.free_blocks() == blocks
    assert scheduler.next_batch() is not None
    scheduler.abort_batch()
    # every job heard of it, and the worker stays failed: a later request is answered at once
    assert sink.of(1, "error") == [(700, 0)] and sink.of(2, "error") == [(700, 0)]
    assert worker.jobs() == 0
    worker.submit(3, range(5), 2)
    assert worker.iterate() == (700, False)
    assert sink.of(3, "error") == [(700, 0)]
    assert len(executor.steps) == 3


def test_an_executor_that_returns_too_few_tokens_fails_the_step(built_library):
    scheduler = Scheduler(2, 64, 2, 100, 16)
    sink = Recorder()
    worker = Worker(scheduler, Executor(sample=lambda step: [1]), sink)
    worker.submit(1, range(10), 2)
    worker.submit(2, range(10), 2)
    assert worker.iterate() == (0x5102, False)
    assert worker.aborted_steps() == 1 and sink.of(2, "error") == [(0x5102, 0)]


def test_an_exception_in_the_executor_is_a_failed_step_not_a_crash(built_library):
    scheduler = Scheduler(2, 64, 2, 100, 16)

    def broken(step):
        raise KeyError("no such tensor")

    sink = Recorder()
    worker = Worker(scheduler, broken, sink)
    worker.submit(1, range(10), 2)
    assert worker.iterate() == (0x5200, False)
    assert isinstance(worker.raised, KeyError)
    assert sink.of(1, "error") == [(0x5200, 0)]


def test_a_refused_request_is_answered_at_once_and_never_becomes_a_job(built_library):
    scheduler = Scheduler(2, 64, 2, 100, 16)
    sink = Recorder()
    worker = Worker(scheduler, Executor(), sink)
    worker.submit(1, range(10), 2)
    worker.submit(1, range(10), 2)  # Duplicate
    worker.submit(2, [], 2)  # EmptyPrompt
    worker.submit(3, range(10), 0)  # NoOutputTokens
    worker.submit(4, range(5000), 2)  # ContextTooLong: 100 pages of 16 tokens
    assert drain(worker) == 0
    assert sink.of(1, "error") == [(0x5000 + 1, 0)] and sink.of(1, "done") == [(2, 0)]
    assert sink.of(2, "error") == [(0x5000 + 2, 0)]
    assert sink.of(3, "error") == [(0x5000 + 3, 0)]
    assert sink.of(4, "error") == [(0x5000 + 5, 0)]


def test_an_abandoned_job_is_cancelled_between_steps(built_library):
    scheduler = Scheduler(2, 64, 2, 100, 16)
    executor, sink = Executor(), Recorder()
    worker = Worker(scheduler, executor, sink)
    worker.submit(1, range(10), 50)
    worker.submit(2, range(10), 3)
    assert worker.iterate() == (0, True) and worker.iterate() == (0, True)
    worker.abandon(1)
    worker.abandon(99)  # unknown: nothing to do
    assert worker.iterate() == (0, True)
    # the step that was planned still ran with both; then sequence 1 left and gave everything back
    assert sorted(executor.steps[-1]["seq_ids"]) == [1, 2]
    assert worker.jobs() == 1 and scheduler.active() == 1
    assert drain(worker) == 0
    assert all(step["seq_ids"] == [2] for step in executor.steps[3:])
    assert sink.of(1, "done") == [] and sink.of(1, "error") == [] and sink.of(2, "done") == [(3, 0)]
    assert scheduler.cache.states_in_use() == 0 and scheduler.cache.free_blocks() == 100


def test_a_waiting_job_can_be_abandoned_before_admission(built_library):
    scheduler = Scheduler(1, 64, 1, 100, 16)  # one sequence at a time
    sink = Recorder()
    worker = Worker(scheduler, Executor(), sink)
    worker.submit(1, range(10), 4)
    worker.submit(2, range(10), 4)
    assert worker.iterate() == (0, True)
    assert scheduler.waiting() == 1
    worker.abandon(2)
    assert drain(worker) == 0
    assert sink.of(2, "done") == [] and sink.tokens(2) == [] and sink.of(1, "done") == [(4, 0)]
    assert scheduler.waiting() == 0


def test_the_loop_serves_requests_queued_from_another_thread(built_library):
    scheduler = Scheduler(4, 128, 4, 400, 16)
    sink = Recorder()
    worker = Worker(scheduler, Executor(), sink)
    result = []
    loop = threading.Thread(target=lambda: result.append(worker.run()))
    loop.start()
    try:
        for seq in range(1, 13):
            worker.submit(seq, range(seq, seq + 30), 5)
    finally:
        worker.shutdown()
        loop.join(timeout=30)
    assert not loop.is_alive() and result == [0]
    for seq in range(1, 13):
        assert sink.of(seq, "done") == [(5, 0)]
        assert sink.tokens(seq) == [1000 * seq + 30 + i for i in range(5)]
    assert scheduler.active() == 0 and scheduler.cache.free_blocks() == 400


def test_several_threads_can_queue_and_abandon_while_the_loop_runs(built_library):
    scheduler = Scheduler(8, 256, 8, 800, 16)
    sink = Recorder()
    worker = Worker(scheduler, Executor(), sink)
    result = []
    loop = threading.Thread(target=lambda: result.append(worker.run()))
    loop.start()

    def client(first):
        for seq in range(first, first + 25):
            worker.submit(seq, range(seq % 7, seq % 7 + 20 + seq % 13), 1 + seq % 6)
            if seq % 5 == 0:
                worker.abandon(seq)

    clients = [threading.Thread(target=client, args=(1 + 100 * i,)) for i in range(4)]
    try:
        for thread in clients:
            thread.start()
        for thread in clients:
            thread.join(timeout=30)
    finally:
        worker.shutdown()
        loop.join(timeout=60)
    assert not loop.is_alive() and result == [0]
    for first in (1, 101, 201, 301):
        for seq in range(first, first + 25):
            done, tokens = sink.of(seq, "done"), sink.tokens(seq)
            assert sink.of(seq, "error") == []
            if seq % 5 == 0 and not done:
                continue  # left before it finished: no terminal event, by design
            assert done == [(1 + seq % 6, 0)] and len(tokens) == 1 + seq % 6
    assert scheduler.active() == 0 and scheduler.waiting() == 0 and scheduler.cache.free_blocks() == 800


def test_the_next_turn_carries_the_restore_of_the_previous_prompt(built_library):
    scheduler = Scheduler(2, 512, 2, 100, 64)
    scheduler.enable_prefix_cache(4)
    executor, sink = Executor(), Recorder()
    worker = Worker(scheduler, executor, sink)
    worker.submit(1, range(150), 2, history_tokens=150)
    assert drain(worker) == 0
    assert len(executor.steps[0]["saves"]) == 1 and executor.steps[0]["restores"] == []
    saved = executor.steps[0]["saves"][0]
    assert saved[0] == 1

    before = len(executor.steps)
    worker.submit(2, range(200), 1, history_tokens=200)
    assert drain(worker) == 0
    turn = executor.steps[before]
    # 150 tokens are already computed: the step is fed the other 50 and restores the snapshot first
    assert turn["tokens"] == [list(range(150, 200))] and turn["position_starts"] == [150]
    assert [(seq, snapshot) for seq, _, snapshot in turn["restores"]] == [(2, saved[2])]
    assert scheduler.cache.prefix_stats()["reused_tokens"] == 150


def test_worker_needs_its_callbacks(built_library):
    from qwencore_b200.engine import lib

    assert not lib.qwc_worker_new(None, None, None, None, None, None, 0)
