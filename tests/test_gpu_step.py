"""The whole decode step (device packing, 3:1 DeltaNet / full-attention layers, MLP, FP8 head,
greedy argmax, CUDA graph) against the CPU oracle on a reduced-depth replica of the synthetic
model: same widths as the 27B shape, four layers, a small vocabulary."""

import numpy as np
import pytest

from oracle import oracle
from qwencore_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engine_module(cuda, built_library):
    from qwencore_b200 import abi, engine

    before = abi.get_shape()
    yield engine
    abi.configure(*before)
    assert abi.lib.qwc_device_status() == 0


def small_config(engine_module, **overrides):
    values = dict(num_layers=4, vocab=8192, max_batch=4, max_context=512, kv_pool_blocks=160, state_slots=6,
                  seed=7, use_graph=1, write_logits=1)
    values.update(overrides)
    return engine_module.default_config(**values)


def install(engine, cache, rng, contexts):
    """Admits one sequence per context through the host cache manager and mirrors it on the device."""
    ids = []
    for i, context in enumerate(contexts):
        seq = 100 + i
        cache.admit(seq, int(context))
        ids.append(seq)
    engine.apply_edits(cache.drain_edits())
    return ids


def host_layout(cache, ids, page, capacity, max_blocks):
    seq_tokens = np.zeros(capacity, np.uint32)
    seq_blocks = np.zeros((capacity, max_blocks), np.uint32)
    counts = np.zeros(capacity, np.uint32)
    slots = []
    for seq in ids:
        info = cache.sequence(seq)
        slot = info["state_slot"]
        slots.append(slot)
        seq_tokens[slot] = info["tokens"]
        counts[slot] = len(info["blocks"])
        seq_blocks[slot, :len(info["blocks"])] = info["blocks"]
    return oracle.layout_decode(np.array(slots, np.uint32), seq_tokens, seq_blocks, counts, max_blocks, page)


def test_decode_step_matches_oracle_for_two_steps(cuda, engine_module):
    from step_oracle import HostModel, decode_step

    config = small_config(engine_module)
    engine = engine_module.Engine(config)
    try:
        page, capacity = config.kv_page_size, config.state_slots
        cache = engine_module.CacheManager(capacity, config.kv_pool_blocks, page)
        rng = np.random.default_rng(0)
        ids = install(engine, cache, rng, [37, 300, 129, 16])
        model = HostModel(engine)
        order = [ids[2], ids[0], ids[3], ids[1]]  # batch order differs from slot order
        tokens = np.array([5, 8191, 77, 4000], dtype=np.uint32)
        for step in range(2):  # step 0 runs eagerly, step 1 replays the captured graph
            for seq in order:
                cache.append_token(seq)
            edits = cache.drain_edits()
            layout = host_layout(cache, order, page, capacity, model.max_blocks)
            assert layout["status"] == 0
            sampled = engine.decode(layout["state_slots"], tokens, edits)
            want_logits, want_tokens, want_normed = decode_step(model, layout, tokens)
            got_logits = engine.read("logits", 0, np.float32).reshape(config.max_batch, config.vocab)[:4]

            # integer path: bit-exact
            assert np.array_equal(engine.read("context_lengths", 0, np.uint32)[:4], layout["context_lengths"])
            tables = engine.read("block_tables", 0, np.uint32).reshape(config.max_batch, model.max_blocks)[:4]
            assert np.array_equal(tables, layout["block_tables"])

            # Every kernel meets its own 1e-2 * RMS bound (test_gpu_kernels.py); through ~30 chained
            # kernels with bf16 activations between them single-ulp differences compound, so the
            # end-to-end logits are held to an RMS error of 2e-2 and a worst element of 1e-1 (of RMS).
            rms = np.sqrt(np.mean(want_logits.astype(np.float64) ** 2))
            err = np.max(np.abs(got_logits - want_logits))
            rms_err = np.sqrt(np.mean((got_logits - want_logits).astype(np.float64) ** 2))
            assert np.isfinite(got_logits).all()
            assert rms_err <= 2e-2 * rms, f"step {step}: logits rms err {rms_err} vs rms {rms}"
            assert err <= 1e-1 * rms, f"step {step}: logits err {err} vs rms {rms}"
            # greedy argmax: exact on the GPU logits, equal to the oracle's wherever the top-2 gap is clear
            assert np.array_equal(sampled, oracle.argmax(got_logits, config.vocab, 4))
            ordered = np.sort(want_logits, axis=1)
            clear = (ordered[:, -1] - ordered[:, -2]) > 4 * err
            assert np.array_equal(sampled[clear], want_tokens[clear])
            assert clear.sum() >= 2, "test inputs must exercise the argmax comparison"
            tokens = want_tokens.copy()
            if step == 0:
                # The first DeltaNet layer sees identical inputs up to one projection, whose bf16
                # outputs sit one grid step from the oracle's in a few elements per ten thousand.
                # Such a step in a large element of v (0.5 at magnitude 64) moves that element's
                # whole state row by several int8 codes, so: nearly every code within one step, the
                # rest confined to a handful of rows, and the stored values equal by RMS.
                used = sorted(set(layout["state_slots"].tolist()))
                got = engine.read("state", 0, np.int8).reshape(model.layers[0]["state"].shape)
                diff = np.abs(got.astype(np.int32) - model.layers[0]["state"].astype(np.int32))[used]
                assert np.mean(diff > 0) < 0.01 and np.mean(diff > 1) < 2e-4
                assert (diff.max(axis=-1) > 1).sum() <= 8, "more than a handful of state rows moved"
                scales = engine.read("state_scales", 0, np.float32).reshape(model.layers[0]["state_scales"].shape)
                got_values = got[used].astype(np.float32) * scales[used][..., None]
                want_values = (model.layers[0]["state"][used].astype(np.float32) *
                               model.layers[0]["state_scales"][used][..., None])
                value_rms = np.sqrt(np.mean(want_values.astype(np.float64) ** 2))
                assert np.sqrt(np.mean((got_values - want_values).astype(np.float64) ** 2)) <= 1e-2 * value_rms

        # recurrent state and KV pages after two steps
        for index, layer in enumerate(model.layers):
            if layer["full"]:
                for name in ("k_cache", "v_cache"):
                    got = engine.read(name, index).reshape(layer[name].shape)
                    steps = np.abs(got.astype(np.int32) - layer[name].astype(np.int32))
                    # only 2 steps x 4 rows x 4 heads x 256 bytes were written (0.3 % of the pool); this
                    # layer's inputs carry three layers of bf16-level differences, so a written code
                    # may sit one e4m3 step away, never more than two
                    assert np.mean(steps > 0) < 2e-3, name
                    got_values = synth.e4m3_decode(got).astype(np.float64)
                    want_values = synth.e4m3_decode(layer[name]).astype(np.float64)
                    written = steps > 0
                    if written.any():  # where they differ, they differ by about one e4m3 step
                        relative = np.abs(got_values - want_values)[written] / np.maximum(
                            np.abs(want_values[written]), 2.0 ** -6)
                        assert np.median(relative) <= 0.15, name
            else:
                got = engine.read("state", index, np.int8).reshape(layer["state"].shape)
                diff = np.abs(got.astype(np.int32) - layer["state"].astype(np.int32))
                used = sorted(set(layout["state_slots"].tolist()))
                # Later layers and steps inherit bf16-level input differences, and rows whose values
                # decayed to ~1e-13 have meaningless codes: compare the stored values.
                got_scales = engine.read("state_scales", index, np.float32).reshape(layer["state_scales"].shape)
                got_values = got[used].astype(np.float32) * got_scales[used][..., None]
                want_values = layer["state"][used].astype(np.float32) * layer["state_scales"][used][..., None]
                value_rms = np.sqrt(np.mean(want_values.astype(np.float64) ** 2))
                assert np.sqrt(np.mean((got_values - want_values).astype(np.float64) ** 2)) <= 2e-2 * value_rms
                assert np.mean(diff[used] > 1) < 0.10
                untouched = [s for s in range(capacity) if s not in used]
                assert not diff[untouched].any()
                conv = engine.read("conv_state", index, np.float32).reshape(layer["conv_state"].shape)
                conv_rms = np.sqrt(np.mean(layer["conv_state"].astype(np.float64) ** 2))
                assert np.sqrt(np.mean((conv - layer["conv_state"]).astype(np.float64) ** 2)) <= 2e-2 * conv_rms
    finally:
        engine.close()


def test_graph_replay_and_eager_step_agree(cuda, engine_module):
    """The captured step and the eager step produce the same tokens (executor.rs:965-993)."""
    results = []
    for use_graph in (0, 1):
        engine = engine_module.Engine(small_config(engine_module, use_graph=use_graph, num_layers=4))
        try:
            cache = engine_module.CacheManager(6, 160, 16)
            ids = install(engine, cache, None, [50, 200, 90])
            tokens = np.array([1, 2, 3], dtype=np.uint32)
            produced = []
            for _ in range(4):
                for seq in ids:
                    cache.append_token(seq)
                slots = [cache.sequence(seq)["state_slot"] for seq in ids]
                tokens = engine.decode(slots, tokens, cache.drain_edits())
                produced.append(tokens.copy())
            results.append(np.stack(produced))
        finally:
            engine.close()
    assert np.array_equal(results[0], results[1])


def test_worker_loop_drives_scheduler_and_engine(cuda, engine_module):
    """serve.rs worker iteration: plan, decode, complete; lengths end requests and free both pools."""
    engine = engine_module.Engine(small_config(engine_module, num_layers=4, max_batch=3, state_slots=3))
    try:
        scheduler = engine_module.Scheduler(3, 64, 3, 160, 16)
        for seq, (prompt, new) in enumerate([(20, 3), (33, 5), (16, 2), (8, 4)], start=1):
            scheduler.submit(seq, prompt, new)
        finished, decoded_rows = [], 0
        for _ in range(40):
            rows, done = engine.worker_step(scheduler)
            decoded_rows += rows
            finished += done
            if scheduler.active() == 0 and scheduler.waiting() == 0:
                break
        assert sorted(finished) == [(1, 3, "Length"), (2, 5, "Length"), (3, 2, "Length"), (4, 4, "Length")]
        assert decoded_rows == 3 + 5 + 2 + 4
        assert scheduler.cache.states_in_use() == 0 and scheduler.cache.free_blocks() == 160
        # the device copy of the token counts followed every release
        engine.apply_edits(scheduler.cache.drain_edits())
        assert not engine.read("seq_tokens", 0, np.uint32).any()
    finally:
        engine.close()


def test_token_level_worker_runs_on_the_engine(cuda, engine_module):
    """The worker loop with the engine as its executor (qwc_engine_execute_step): requests queued with
    their prompts, tokens through the event callback, both pools back at the end."""
    config = small_config(engine_module, num_layers=4, max_batch=3, state_slots=3)
    engine = engine_module.Engine(config)
    try:
        scheduler = engine_module.Scheduler(3, 64, 3, 160, 16)
        events = []
        worker = engine_module.Worker(scheduler, engine, lambda *event: events.append(event) and False)
        budgets = {1: 3, 2: 5, 3: 2, 4: 4}
        for seq, prompt in [(1, 20), (2, 33), (3, 16), (4, 8)]:
            worker.submit(seq, range(prompt), budgets[seq])
        for _ in range(60):
            status, progressed = worker.iterate()
            assert status == 0
            if not progressed and worker.jobs() == 0:
                break
        for seq, budget in budgets.items():
            tokens = [value for s, kind, value, _ in events if s == seq and kind == "token"]
            assert len(tokens) == budget and all(token < config.vocab for token in tokens)
            # the first token a sequence emits is the one its (accounted, not computed) prefill sampled
            assert tokens[0] == (seq * 7919 + 1000) % config.vocab
            assert [(value, reason) for s, kind, value, reason in events if s == seq and kind == "done"] == [(budget, 0)]
        assert worker.aborted_steps() == 0
        assert scheduler.cache.states_in_use() == 0 and scheduler.cache.free_blocks() == 160
    finally:
        engine.close()


def test_copy_kv_block_copies_one_page_in_every_attention_layer(cuda, engine_module):
    """Executor::copy_kv_block (executor.rs:825-835): page `to` becomes page `from` in the K and V pools
    of every full-attention layer; nothing else moves; a page outside the pool is refused."""
    from qwencore_b200 import abi

    config = small_config(engine_module, num_layers=8)
    engine = engine_module.Engine(config)
    try:
        attention_layers = [i for i in range(config.num_layers) if (i + 1) % config.full_attention_interval == 0]
        assert attention_layers
        shape = (config.kv_pool_blocks, -1)
        before = {(name, i): engine.read(name, i, np.uint8).reshape(shape).copy()
                  for i in attention_layers for name in ("k_cache", "v_cache")}
        engine.copy_kv_block(5, 131)
        engine.copy_kv_block(7, 7)  # (reading a tensor waits for the engine's stream)
        for (name, i), old in before.items():
            new = engine.read(name, i, np.uint8).reshape(shape)
            assert not np.array_equal(old[5], old[131])  # the seeded pools differ page by page
            want = old.copy()
            want[131] = old[5]
            assert np.array_equal(new, want), (name, i)
        for pages in ((config.kv_pool_blocks, 0), (0, config.kv_pool_blocks)):
            with pytest.raises(abi.QwcError) as error:
                engine.copy_kv_block(*pages)
            assert error.value.code == abi.CUDA_ERROR_INVALID_VALUE
    finally:
        engine.close()


def test_memory_ceiling_refuses_before_the_driver_is_asked(cuda, engine_module):
    """The VRAM ceiling (crates/qwc-cuda/src/memory.rs:31-88, tests/memory_limit.rs): an engine whose
    buffers do not fit its budget is refused with cudaErrorMemoryAllocation and leaves nothing behind;
    with room it reports what it took.  The refusal is host arithmetic: nothing is driven out of memory."""
    import torch

    from qwencore_b200 import abi

    def refused():
        with pytest.raises(abi.QwcError) as error:
            engine_module.Engine(small_config(engine_module, num_layers=4, memory_limit=64 << 20))
        assert error.value.code == 2
        torch.cuda.synchronize()
        return torch.cuda.mem_get_info()[0]

    free_after_first = refused()  # (the first one may also load the library's kernels onto the device)
    for _ in range(3):
        free_now = refused()
    # what a refused engine had taken (up to its 64 MiB) came back every time
    assert free_now >= free_after_first - (4 << 20)

    config = small_config(engine_module, num_layers=4, memory_limit=8 << 30)
    engine = engine_module.Engine(config)
    try:
        usage = engine.memory_usage()
        assert 64 << 20 < usage["used"] <= usage["limit"] <= 8 << 30
        # the host-side memory plan names what the engine took: weights and the two pools, the rest
        # (activations, workspaces, tables) is what a Budget calls workspace
        geometry = engine_module.CacheGeometry.for_config(config)
        planned = (engine_module.weight_bytes(config) + config.state_slots * geometry.state_bytes_per_slot
                   + config.kv_pool_blocks * geometry.kv_bytes_per_block())
        assert planned <= usage["used"] < planned + (512 << 20), (planned, usage["used"])
    finally:
        engine.close()
    unlimited = engine_module.Engine(small_config(engine_module, num_layers=4))
    try:
        assert unlimited.memory_usage() == {"used": usage["used"], "limit": 0}
    finally:
        unlimited.close()


def test_table_edits_are_bounded_on_the_host(cuda, engine_module):
    """Slots, table indices and page ids reach the device tables only through edits, and the engine bounds
    them before anything is copied: a page beyond the pool never gets into a block table."""
    from qwencore_b200 import abi

    config = small_config(engine_module, num_layers=4)  # 6 slots, 160 pages, 32 table entries per slot
    engine = engine_module.Engine(config)
    try:
        cache = engine_module.CacheManager(6, 160, 16)
        install(engine, cache, None, [50, 90])
        tokens_before = engine.read("seq_tokens", 0, np.uint32)
        blocks_before = engine.read("seq_blocks", 0, np.uint32)
        good = [1, 3, 17, 0]
        for bad in ([0, 0, 160, 0], [6, 0, 1, 1], [0, 32, 1, 0], [0, 0, 1, 3], [6, 0, 1, 2]):
            for edits in ([bad], [good, bad]):  # nothing of a drain with a bad edit is applied
                with pytest.raises(abi.QwcError) as error:
                    engine.apply_edits(np.array(edits, dtype=np.uint32))
                assert error.value.code == abi.CUDA_ERROR_INVALID_VALUE
                with pytest.raises(abi.QwcError) as error:
                    engine.decode([0, 1], [3, 4], np.array(edits, dtype=np.uint32))
                assert error.value.code == abi.CUDA_ERROR_INVALID_VALUE
        assert np.array_equal(engine.read("seq_tokens", 0, np.uint32), tokens_before)
        assert np.array_equal(engine.read("seq_blocks", 0, np.uint32), blocks_before)
        engine.apply_edits(np.array([good], dtype=np.uint32))
        assert engine.read("seq_blocks", 0, np.uint32).reshape(6, 32)[1, 3] == 17
    finally:
        engine.close()


def test_decode_reports_packing_errors(cuda, engine_module):
    from qwencore_b200 import abi

    engine = engine_module.Engine(small_config(engine_module, num_layers=4))
    try:
        with pytest.raises(abi.QwcError) as error:  # slot 2 holds no sequence
            engine.decode([2], [1])
        assert error.value.code == 0x1000 + 1
        with pytest.raises(abi.QwcError) as error:
            engine.decode([0, 1, 2, 3, 4], [1] * 5)
        assert error.value.code == abi.CUDA_ERROR_INVALID_VALUE
    finally:
        engine.close()


def test_step_returns_the_device_status_word_and_the_worker_rolls_back(cuda, engine_module):
    """A bounded wait that gave up leaves a code in the sticky status word and kernels skip their
    stores: the step must say so instead of returning tokens (injected on the host: the word is
    set as a failed wait would set it, nothing on the device faults or hangs)."""
    from qwencore_b200 import abi

    engine = engine_module.Engine(small_config(engine_module, num_layers=4, max_batch=3, state_slots=3))
    try:
        scheduler = engine_module.Scheduler(3, 64, 3, 160, 16)
        scheduler.submit(1, 20, 8)
        scheduler.submit(2, 33, 8)
        rows = 0
        while rows == 0:
            rows, _ = engine.worker_step(scheduler)
        assert rows == 2
        remaining = scheduler.remaining_tokens(1)
        assert abi.lib.qwc_device_status_set(0x103) == 0
        try:
            with pytest.raises(abi.QwcError) as error:
                engine.worker_step(scheduler)
            assert error.value.code == 0x4000 + 0x103
        finally:
            assert abi.lib.qwc_device_status_reset() == 0
        # the batch was rolled back: nothing was committed, the next step decodes the same rows
        assert scheduler.remaining_tokens(1) == remaining
        rows, _ = engine.worker_step(scheduler)
        assert rows == 2 and scheduler.remaining_tokens(1) == remaining - 1
        assert abi.lib.qwc_device_status() == 0
    finally:
        engine.close()


def test_phase_timeline_covers_every_phase(cuda, engine_module):
    """Timeline marks (crates/qwc-cuda/src/timeline.rs:17-77): one entry per phase label."""
    from qwencore_b200 import abi

    engine = engine_module.Engine(small_config(engine_module, num_layers=4))
    try:
        cache = engine_module.CacheManager(6, 160, 16)
        ids = install(engine, cache, None, [40, 41])
        for seq in ids:
            cache.append_token(seq)
        engine.decode([0, 1], [3, 4], cache.drain_edits())
        phases = dict((label, (ms, launches)) for label, ms, launches in engine.profile_step(2))
        for label in ("pack", "embed", "norm", "gemm.la_in", "delta.prepare", "delta.scan", "delta.norm",
                      "gemm.la_out", "gemm.attn_qkv", "attn.prepare", "attn.decode", "gemm.attn_out",
                      "gemm.mlp_gate_up", "gemm.mlp_down", "lm_head"):  # sampling is part of the head
            assert label in phases, label
        assert phases["gemm.mlp_down"][1] == 4 and phases["delta.scan"][1] == 3 and phases["attn.decode"][1] == 1
        traffic = engine.traffic(2, 83)
        assert traffic.gemv_launches_per_step == 4 * 2 + 3 * 2 + 2
        assert traffic.kv_bytes == 83 * 2 * 4 * 256
        # graph-timed subsets of the step: the projections, one phase, everything, nothing
        ms, launched = engine.time_phases(2, "gemm.", replays=3)
        assert launched == traffic.gemv_launches_per_step and ms > 0
        ms_scan, launched = engine.time_phases(2, "delta.scan", replays=3)
        assert launched == 3 and 0 < ms_scan < ms * 10
        ms_all, launched = engine.time_phases(2, "", replays=3)
        assert launched == sum(count for _, count in phases.values()) and ms_all >= ms
        with pytest.raises(abi.QwcError):
            engine.time_phases(2, "no.such.phase")
        assert abi.lib.qwc_device_status() == 0
    finally:
        engine.close()
