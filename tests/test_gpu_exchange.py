"""Latency mode's fused exchange, as far as one GPU can show it.

In latency mode every rank computes its rows of a projection and stores the K-split partial sums
into every rank's exchange block as tagged 8-byte words; the consumers sum them after a bounded wait
(include/qwc_exchange.h).  The reference gathers the same rows with ncclAllGather
(crates/qwc-engine/src/executor.rs, tensor-parallel decode); the arithmetic per element is the
unsplit projection's, so the checks are against the one-GPU K-split kernels (bit for bit where the
slices are the same) and against the CPU oracle.

Ranks are played one after another on the one device: producers never wait, so "rank r" is one launch
with its own weight rows whose "peer blocks" are further local buffers, and the consumers run after
all of them.  (Kernels that wait on one another never run here as separate launches; the real
two-process case is tests/test_gpu_split.py.)  A consumer's bounded wait is shown on a row that
nobody writes."""

import ctypes
import time

import numpy as np
import pytest

from oracle import oracle
from qwencore_b200 import synth
from test_gpu_kernels import assert_rms_close, bf16_out, dev, host

pytestmark = pytest.mark.gpu

STATUS_PEER_WAIT = 0x106


@pytest.fixture(scope="module")
def ops(cuda, built_library):
    from qwencore_b200 import abi, ops as module

    yield module
    assert abi.lib.qwc_device_status() == 0, "a bounded device wait gave up during the tests"


class Ranks:
    """`count` exchange blocks on the one device and the epoch word they share."""

    def __init__(self, torch, abi, ops, count, row_bytes):
        self.torch, self.abi, self.ops, self.count = torch, abi, ops, count
        self.blocks = [torch.zeros(row_bytes, dtype=torch.uint8, device="cuda") for _ in range(count)]
        self.epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.steps = 0

    def advance(self):
        self.abi.check(self.abi.lib.qwc_exchange_advance(self.epoch.data_ptr(), self.ops._stream()), "advance")
        self.steps += 1

    def row(self, rank, instance, width, offset=0):
        row = self.abi.ExchangeRow()
        for r, block in enumerate(self.blocks):
            row.blocks[r] = block.data_ptr()
        row.ranks, row.rank, row.epoch = self.count, rank, self.epoch.data_ptr()
        row.instance, row.offset, row.width = instance, offset, width
        return row

    def tag(self, instance):
        return (self.steps << 10) | instance

    def words(self, rank, slices, width):
        raw = host(self.blocks[rank]).view(np.uint32).reshape(-1, 2)[: slices * width]
        return raw[:, 0].copy().view(np.float32).reshape(slices, width), raw[:, 1].reshape(slices, width)


def rank_linear(torch, ops, packed, scales, global_scale, rank, local, in_features):
    rows = slice(rank * local, (rank + 1) * local)
    swizzled = synth.swizzle_block_scales(scales[rows], local, in_features)
    return ops.Linear(dev(torch, np.ascontiguousarray(packed[rows])), dev(torch, swizzled), global_scale, local,
                      in_features)


def staged_row(torch, ops, x_bits, features):
    staged = ops.new_staged(1, features)
    ops.stage_activations(dev(torch, x_bits), staged, 1, features)
    return staged


def test_every_rank_receives_every_slice_and_the_norm_sums_them(cuda, ops):
    """Four ranks x 512 rows of a 2048 x 1024 projection.  The whole matrix as a one-GPU K split has the
    same four K slices, so the exchanged words must be its partial sums bit for bit, in every rank's
    block, and the residual norm on them the one-GPU split norm bit for bit."""
    from qwencore_b200 import abi

    torch = cuda
    lib, stream = abi.lib, ops._stream()
    ranks, out_features, in_features, instance = 4, 2048, 1024, 7
    local = out_features // ranks
    packed, scales, swizzled = synth.nvfp4_matrix(21, "exchange.hidden", out_features, in_features)
    x = synth.normal_bf16(21, "exchange.x", (1, in_features))
    staged_x = staged_row(torch, ops, x, in_features)
    global_scale = 6.0

    whole = ops.Linear(dev(torch, packed), dev(torch, swizzled), global_scale, out_features, in_features)
    slices = ops.split_count(whole)
    assert slices == lib.qwc_nvfp4_exchange_slices(local, in_features, 0), "the case needs equal K slices"
    sums = torch.zeros((slices, 1, out_features), dtype=torch.float32, device="cuda")
    ops.w4a16_split(whole, staged_x, sums, 1)

    group = Ranks(torch, abi, ops, ranks, lib.qwc_exchange_row_bytes(out_features))
    group.advance()
    for rank in range(ranks):
        linear = rank_linear(torch, ops, packed, scales, global_scale, rank, local, in_features)
        row = group.row(rank, instance, out_features)
        abi.check(lib.qwc_nvfp4_w4a16_exchange(linear.packed.data_ptr(), linear.scales.data_ptr(),
                                               staged_x.data_ptr(), ctypes.byref(row), local, in_features, stream),
                  "qwc_nvfp4_w4a16_exchange")
    torch.cuda.synchronize()
    want = host(sums).reshape(slices, out_features)
    for rank in range(ranks):
        values, tags = group.words(rank, slices, out_features)
        assert np.all(tags == group.tag(instance)), f"rank {rank}: every word carries this step's tag"
        assert np.array_equal(values.view(np.uint32), want.view(np.uint32)), f"rank {rank}: partial sums"

    # the residual norm on the exchanged row == the one-GPU norm on the split sums
    residual = synth.normal_bf16(21, "exchange.res", (1, out_features), std=20.0)
    weight = synth.normal_bf16(21, "exchange.w", (out_features,), std=0.02)
    results = []
    for exchanged in (False, True):
        res_dev = dev(torch, residual)
        rows, normed = bf16_out(torch, 1, out_features), bf16_out(torch, 1, out_features)
        staged = ops.new_staged(1, out_features)
        if exchanged:
            row = group.row(2, instance, out_features)  # any rank's block holds the same words
            abi.check(lib.qwc_rmsnorm_bf16_exchanged(ctypes.byref(row), slices, global_scale, rows.data_ptr(),
                                                     res_dev.data_ptr(), dev(torch, weight).data_ptr(),
                                                     normed.data_ptr(), staged.data_ptr(), out_features, 1e-6, stream),
                      "qwc_rmsnorm_bf16_exchanged")
        else:
            ops.rmsnorm_split_staged(sums, slices, global_scale, rows, res_dev, dev(torch, weight), normed, staged, 1,
                                     out_features)
        torch.cuda.synchronize()
        results.append((host(rows), host(res_dev), host(normed), host(staged)))
    for got, want_part, what in zip(results[1], results[0], ("projection rows", "residual", "normed", "staged")):
        assert np.array_equal(got, want_part), what

    # ... and the plain sum to bf16 rows (what the attention prepare step reads)
    summed = bf16_out(torch, 1, out_features)
    row = group.row(0, instance, out_features)
    abi.check(lib.qwc_nvfp4_sum_exchanged(ctypes.byref(row), slices, global_scale, summed.data_ptr(), stream),
              "qwc_nvfp4_sum_exchanged")
    torch.cuda.synchronize()
    assert np.array_equal(host(summed), results[0][0])
    want_rows = oracle.gemv_w4a16(packed, scales, global_scale, x, out_features, in_features, 1)
    assert_rms_close(synth.bf16_value(host(summed)), want_rows, "exchanged projection against the oracle")


def test_swiglu_pair_exchanged_and_combined(cuda, ops):
    """Two ranks x 512 outputs of a 1024-wide SwiGLU pair: [gate | up] slices in every block, combined
    by the consumer into the staged operand of the down projection."""
    from qwencore_b200 import abi

    torch = cuda
    lib, stream = abi.lib, ops._stream()
    ranks, intermediate, hidden, instance = 2, 1024, 1024, 3
    local = intermediate // ranks
    gate_packed, gate_scales, _ = synth.nvfp4_matrix(22, "exchange.gate", intermediate, hidden)
    up_packed, up_scales, _ = synth.nvfp4_matrix(22, "exchange.up", intermediate, hidden)
    x = synth.normal_bf16(22, "exchange.x", (1, hidden))
    staged_x = staged_row(torch, ops, x, hidden)
    slices = lib.qwc_nvfp4_exchange_slices(local, hidden, 1)
    assert 1 <= slices <= 16
    group = Ranks(torch, abi, ops, ranks, lib.qwc_exchange_row_bytes(2 * intermediate))
    group.advance()
    group.advance()  # tags of the second step
    for rank in range(ranks):
        gate = rank_linear(torch, ops, gate_packed, gate_scales, 5.0, rank, local, hidden)
        up = rank_linear(torch, ops, up_packed, up_scales, 3.0, rank, local, hidden)
        row = group.row(rank, instance, 2 * intermediate)
        abi.check(lib.qwc_nvfp4_swiglu_w4a16_exchange(gate.packed.data_ptr(), gate.scales.data_ptr(),
                                                      up.packed.data_ptr(), up.scales.data_ptr(), staged_x.data_ptr(),
                                                      ctypes.byref(row), local, hidden, stream),
                  "qwc_nvfp4_swiglu_w4a16_exchange")
    torch.cuda.synchronize()
    first, tags = group.words(0, slices, 2 * intermediate)
    second, _ = group.words(1, slices, 2 * intermediate)
    assert np.all(tags == group.tag(instance)) and np.array_equal(first.view(np.uint32), second.view(np.uint32))

    combined = bf16_out(torch, 1, intermediate)
    staged = ops.new_staged(1, intermediate)
    row = group.row(1, instance, 2 * intermediate)
    abi.check(lib.qwc_swiglu_combine_exchanged(ctypes.byref(row), slices, 5.0, 3.0, combined.data_ptr(),
                                               staged.data_ptr(), intermediate, stream), "qwc_swiglu_combine_exchanged")
    torch.cuda.synchronize()
    want = oracle.swiglu_combine(oracle.gemv_w4a16(gate_packed, gate_scales, 5.0, x, intermediate, hidden, 1),
                                 oracle.gemv_w4a16(up_packed, up_scales, 3.0, x, intermediate, hidden, 1))
    got = synth.bf16_value(host(combined))
    assert_rms_close(got, want, "exchanged SwiGLU pair")
    want_staged = np.clip(got, -65504.0, 65504.0).astype(np.float16)
    assert np.array_equal(host(ops.unstage(staged, 1, intermediate)).view(np.uint16), want_staged.view(np.uint16))


def test_vocabulary_head_candidates_from_all_ranks_pick_one_token(cuda, ops):
    """Three ranks x 3000 rows of the vocabulary (ragged last tile pair): the token picked from the
    exchanged candidates is the argmax of the whole table's logits, ties to the smaller index."""
    from qwencore_b200 import abi

    torch = cuda
    lib, stream = abi.lib, ops._stream()
    ranks, local, hidden = 3, 3000, 1024
    vocab = ranks * local
    table, row_scales = oracle.fp8_quantize_rows(synth.normal_bf16(23, "exchange.head", (vocab, hidden), std=0.02), vocab,
                                                 hidden)
    table, row_scales = table.reshape(vocab, hidden).copy(), row_scales.reshape(vocab).copy()
    # two equal best rows on different ranks: the smaller index must win
    table[2 * local + 17] = table[41]
    row_scales[2 * local + 17] = row_scales[41] = 40.0 * float(np.max(row_scales))
    x = synth.normal_bf16(23, "exchange.hx", (1, hidden))
    staged_x = staged_row(torch, ops, x, hidden)
    workspace = ops.new_streamk_workspace()
    group = Ranks(torch, abi, ops, ranks, lib.qwc_exchange_candidate_bytes(ranks))
    group.advance()
    sampled = dev(torch, np.full(ranks, 0xFFFFFFFF, dtype=np.uint32))
    status_out = dev(torch, np.full(1, 7, dtype=np.uint32))
    logits = torch.zeros((ranks, local), dtype=torch.float32, device="cuda")
    for rank in range(ranks):
        rows = slice(rank * local, (rank + 1) * local)
        row = group.row(rank, 300, 4)
        last = rank == ranks - 1  # only then are everybody's candidates in place: the others store theirs and leave
        abi.check(lib.qwc_fp8_lm_head_exchange(dev(torch, np.ascontiguousarray(table[rows])).data_ptr(),
                                               dev(torch, np.ascontiguousarray(row_scales[rows])).data_ptr(),
                                               staged_x.data_ptr(), logits[rank].data_ptr(), ctypes.byref(row),
                                               sampled.data_ptr() + 4 * rank if last else None,
                                               status_out.data_ptr() if last else None, hidden, local,
                                               workspace.data_ptr(), stream), "qwc_fp8_lm_head_exchange")
        torch.cuda.synchronize()
    all_logits = host(logits).reshape(1, vocab)
    want = oracle.argmax(all_logits, vocab, 1)
    got = host(sampled)
    assert got[ranks - 1] == want[0]
    assert want[0] == 41, "the tie is between row 41 and its copy on the last rank"
    assert host(status_out)[0] == 0
    want_logits = oracle.fp8_lm_head(table, row_scales, x, 1, hidden, vocab)
    assert_rms_close(all_logits, want_logits, "head logits of the ranks' rows")
    # every block holds the same candidates
    blocks = [host(block) for block in group.blocks]
    assert all(np.array_equal(blocks[0], other) for other in blocks[1:])


def test_consumer_gives_up_on_words_that_nobody_stores(cuda, ops):
    """The bounded wait: a consumer of a row that no rank writes returns after its iteration limit,
    leaves kStatusPeerWait in the device status word, and later waits return at once."""
    from qwencore_b200 import abi

    torch = cuda
    lib, stream = abi.lib, ops._stream()
    hidden = 1024
    group = Ranks(torch, abi, ops, 2, lib.qwc_exchange_row_bytes(hidden))
    group.advance()
    weight = dev(torch, synth.normal_bf16(24, "exchange.tw", (hidden,), std=0.02))
    normed = bf16_out(torch, 1, hidden)
    row = group.row(0, 11, hidden)
    assert lib.qwc_device_status() == 0
    try:
        durations = []
        for _ in range(2):
            torch.cuda.synchronize()
            start = time.perf_counter()
            abi.check(lib.qwc_rmsnorm_bf16_exchanged(ctypes.byref(row), 4, 1.0, None, None, weight.data_ptr(),
                                                     normed.data_ptr(), None, hidden, 1e-6, stream),
                      "qwc_rmsnorm_bf16_exchanged")
            torch.cuda.synchronize()
            durations.append(time.perf_counter() - start)
            assert lib.qwc_device_status() == STATUS_PEER_WAIT
        assert durations[0] < 5.0, "the wait is bounded"
        assert durations[1] < 0.25 * durations[0] + 0.01, f"a later wait gives up at once: {durations}"
        assert np.isfinite(synth.bf16_value(host(normed))).all()
    finally:
        assert lib.qwc_device_status_reset() == 0


def test_invalid_rows_are_refused(cuda, ops):
    from qwencore_b200 import abi

    torch = cuda
    lib, stream = abi.lib, ops._stream()
    hidden = 1024
    group = Ranks(torch, abi, ops, 2, lib.qwc_exchange_row_bytes(hidden))
    weight = dev(torch, synth.normal_bf16(24, "exchange.tw", (hidden,), std=0.02))
    normed = bf16_out(torch, 1, hidden)

    def norm(row, slices=4):
        return lib.qwc_rmsnorm_bf16_exchanged(ctypes.byref(row), slices, 1.0, None, None, weight.data_ptr(),
                                              normed.data_ptr(), None, hidden, 1e-6, stream)

    bad = group.row(0, 1024, hidden)  # instance beyond the tag
    assert norm(bad) == abi.CUDA_ERROR_INVALID_VALUE
    bad = group.row(2, 1, hidden)  # rank outside the group
    assert norm(bad) == abi.CUDA_ERROR_INVALID_VALUE
    bad = group.row(0, 1, hidden)
    bad.blocks[1] = None
    assert norm(bad) == abi.CUDA_ERROR_INVALID_VALUE
    bad = group.row(0, 1, hidden, offset=8)
    assert norm(bad) == abi.CUDA_ERROR_INVALID_VALUE
    assert norm(group.row(0, 1, hidden), slices=17) == abi.CUDA_ERROR_INVALID_VALUE
    assert norm(group.row(0, 1, 2 * hidden)) == abi.CUDA_ERROR_INVALID_VALUE  # the row is not the norm's width
    assert lib.qwc_exchange_row_bytes(6) == 0 and lib.qwc_exchange_candidate_bytes(9) == 0
    packed, scales, swizzled = synth.nvfp4_matrix(21, "exchange.bad", 256, 1024)
    linear = ops.Linear(dev(torch, packed), dev(torch, swizzled), 1.0, 256, 1024)
    x = staged_row(torch, ops, synth.normal_bf16(21, "exchange.bx", (1, 1024)), 1024)
    row = group.row(0, 1, hidden)  # 2 ranks x 256 rows is not a row of 1024
    assert lib.qwc_nvfp4_w4a16_exchange(linear.packed.data_ptr(), linear.scales.data_ptr(), x.data_ptr(),
                                        ctypes.byref(row), 256, 1024, stream) == abi.CUDA_ERROR_INVALID_VALUE
    assert lib.qwc_device_status() == 0


def test_engine_exchanging_with_itself_matches_the_oracle_and_the_plain_engine(cuda, built_library):
    """The whole latency-mode step with a single rank (its own block is the only peer): eager, captured
    and replayed steps against the CPU oracle, and the same tokens as the one-GPU step."""
    from qwencore_b200 import abi, engine as engine_module
    from step_oracle import HostModel, decode_step
    from test_gpu_step import host_layout

    before = abi.get_shape()
    engines = []
    try:
        sampled_by = {}
        for exchange in (1, 0):
            config = engine_module.default_config(num_layers=4, vocab=8192, max_batch=1, max_context=512,
                                                  kv_pool_blocks=64, state_slots=2, seed=11, use_graph=1,
                                                  write_logits=1, exchange=exchange)
            engine = engine_module.Engine(config)
            engines.append(engine)
            cache = engine_module.CacheManager(2, 64, 16)
            cache.admit(100, 37)
            engine.apply_edits(cache.drain_edits())
            model = HostModel(engine)
            tokens = np.array([1234], dtype=np.uint32)
            sampled_by[exchange] = []
            for step in range(3):
                cache.append_token(100)
                edits = cache.drain_edits()
                layout = host_layout(cache, [100], 16, 2, (config.max_context + 15) // 16)
                sampled = engine.decode(layout["state_slots"], tokens, edits)
                logits = engine.read("logits", 0, np.float32).reshape(1, config.vocab)
                want_logits, want_tokens, _ = decode_step(model, layout, tokens)
                rms = np.sqrt(np.mean(want_logits.astype(np.float64) ** 2))
                rms_error = np.sqrt(np.mean((logits - want_logits).astype(np.float64) ** 2))
                worst = np.max(np.abs(logits - want_logits))
                assert np.isfinite(logits).all()
                assert rms_error <= 2e-2 * rms and worst <= 1e-1 * rms, f"exchange {exchange} step {step}"
                assert sampled[0] == int(np.argmax(logits[0]))
                sampled_by[exchange].append(int(sampled[0]))
                tokens = want_tokens.astype(np.uint32)
            assert abi.lib.qwc_device_status() == 0
        assert sampled_by[1] == sampled_by[0]
    finally:
        for engine in engines:
            engine.close()
        abi.configure(*before)
