"""GPU parity of the equal-share projection kernel on staged activations (qwc_nvfp4_w4a16_staged,
qwc_nvfp4_swiglu_w4a16_staged, qwc_fp8_lm_head_staged) against the CPU oracle, through the C ABI.

These entry points have no counterpart in the reference (its projections are
crates/qwc-cuda/cuda/nvfp4.cu:489-537, :585-643 and cuda/vocab_fp8.cu:255 on bf16 rows); the
arithmetic is the same, so the oracle and the tolerances are those of test_gpu_kernels.py.  The
cases are chosen for what is new here: shares that cut a tile's K range into two, three and more
pieces, shares that hold several whole tiles, ragged last tiles, 1..32 rows, the staged output that
feeds the next projection, sampling without logits, and bit-reproducibility of the split sums."""

import numpy as np
import pytest

from oracle import oracle
from qwencore_b200 import synth
from test_gpu_kernels import LcgRng, assert_rms_close, bf16_out, dev, host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(cuda, built_library):
    from qwencore_b200 import abi, ops as module

    yield module
    assert abi.lib.qwc_device_status() == 0, "a bounded device wait gave up during the tests"


@pytest.fixture(scope="module")
def workspace(cuda, ops):
    return ops.new_streamk_workspace()


def assert_staged_holds(staged_values, bf16_values, what):
    """The staged copy is the bf16 value converted to f16: identical where f16 has the bits (|v| >= 2^-14,
    saturated at 65504), rounded to the f16 subnormal grid (2^-24) below that."""
    want = np.clip(np.asarray(bf16_values, dtype=np.float32), -65504.0, 65504.0).astype(np.float16)
    assert np.array_equal(np.asarray(staged_values).view(np.uint16), want.view(np.uint16)), what


def staged_input(torch, ops, x_bits, batch, features):
    staged = ops.new_staged(batch, features)
    ops.stage_activations(dev(torch, x_bits), staged, batch, features)
    return staged


def run_staged(torch, ops, workspace, packed, swizzled, global_scale, x_bits, out_features, in_features, batch,
               want_staged=True):
    linear = ops.Linear(dev(torch, packed), dev(torch, swizzled), global_scale, out_features, in_features)
    out = bf16_out(torch, batch, out_features)
    staged_out = ops.new_staged(batch, out_features) if want_staged else None
    ops.w4a16_staged(linear, staged_input(torch, ops, x_bits, batch, in_features), out, staged_out, batch, workspace)
    torch.cuda.synchronize()
    return host(out), (host(ops.unstage(staged_out, batch, out_features)) if want_staged else None), linear


def test_stage_activations_layout_and_saturation(cuda, ops):
    torch = cuda
    batch, features = 5, 256
    values = np.random.default_rng(0).standard_normal((batch, features)).astype(np.float32)
    values[0, 0], values[1, 7], values[2, 8] = 1.0e6, -3.0e38, 6.0e-8  # beyond f16, and an f16 subnormal
    bits = synth.bf16_bits(values)
    staged = staged_input(torch, ops, bits, batch, features)
    torch.cuda.synchronize()
    raw = host(staged).reshape(features // 8, 16, 8)
    want = np.clip(synth.bf16_value(bits), -65504.0, 65504.0).astype(np.float16)
    for token in range(batch):
        assert np.array_equal(raw[:, token, :].reshape(-1).view(np.uint16), want[token].view(np.uint16))
    assert not raw[:, batch:, :].any()
    assert np.array_equal(host(ops.unstage(staged, batch, features)).view(np.uint16), want.view(np.uint16))


def test_staged_w4a16_matches_cpu_for_all_supported_batches(cuda, ops, workspace):
    """The reference's GEMV test inputs (crates/qwc-cuda/tests/nvfp4.rs:23-111; OUT = 40 is its ragged
    last tile rounded to the 8 rows a staged output is made of), 1..32 rows, plain and fused SwiGLU."""
    torch = cuda
    OUT, IN = 40, 512
    rng = LcgRng(0x4A165090)
    packed = np.array([rng.next_u8() for _ in range(OUT * IN // 2)], dtype=np.uint8).reshape(OUT, IN // 2)
    up_packed = np.array([rng.next_u8() for _ in range(OUT * IN // 2)], dtype=np.uint8).reshape(OUT, IN // 2)
    codes = [0x30, 0x38, 0x3C, 0x40]
    scales = np.array([codes[i % 4] for i in range(OUT * IN // 16)], dtype=np.uint8).reshape(OUT, IN // 16)
    swizzled = synth.swizzle_block_scales(scales, OUT, IN)
    for batch in [1, 2, 3, 4, 7, 8, 9, 16, 17, 31, 32]:
        x = synth.bf16_bits(np.array([rng.next_f32() for _ in range(batch * IN)], dtype=np.float32).reshape(batch, IN))
        want = oracle.gemv_w4a16(packed, scales, 8.0, x, OUT, IN, batch)
        got_bits, got_staged, gate = run_staged(torch, ops, workspace, packed, swizzled, 8.0, x, OUT, IN, batch)
        got = synth.bf16_value(got_bits)
        tolerance = 0.035 + np.abs(want) * 0.012  # tests/nvfp4.rs:68
        assert np.all(np.abs(got - want) <= tolerance), f"batch {batch}"
        # the staged copy holds the same bf16 values, as f16
        assert_staged_holds(got_staged, got, f"staged output, batch {batch}")

        want_up = oracle.gemv_w4a16(up_packed, scales, 4.0, x, OUT, IN, batch)
        want_fused = oracle.swiglu_combine(want, want_up)
        up = ops.Linear(dev(torch, up_packed), dev(torch, swizzled), 4.0, OUT, IN)
        fused = bf16_out(torch, batch, OUT)
        fused_staged = ops.new_staged(batch, OUT)
        ops.swiglu_w4a16_staged(gate, up, staged_input(torch, ops, x, batch, IN), fused, fused_staged, batch, workspace)
        torch.cuda.synchronize()
        got_fused = synth.bf16_value(host(fused))
        tolerance = 0.075 + np.abs(want_fused) * 0.025  # tests/nvfp4.rs:103
        assert np.all(np.abs(got_fused - want_fused) <= tolerance), f"fused batch {batch}"
        assert_staged_holds(host(ops.unstage(fused_staged, batch, OUT)), got_fused, f"fused staged, batch {batch}")


# (out, in, batches, what the shape exercises on 148 SMs)
SHAPES = [
    (34816, 5120, [1, 32]),     # config 0: 136 pairs x 20 stages, shares of 18.4 units: every pair in 2-3 pieces
    (12352, 5120, [5, 16]),     # mixer in-proj: a ragged last pair (64 of 256 rows)
    (5120, 17408, [1, 8, 32]),  # down: 20 pairs x 68 stages, 7-8 pieces per pair
    (5120, 4096, [2, 24]),      # la_out: 2.2 units per share, pieces of one or two stages
    (5120, 6144, [32]),         # attention out
    (1024, 5120, [1, 12]),      # 80 units on 80 CTAs: every share is a single stage
    (256, 256, [3]),            # one unit: one CTA, one whole pair
    (65536, 256, [32]),         # shares of several whole pairs, no piece at all
]


@pytest.mark.parametrize("out_features,in_features,batches", SHAPES)
def test_staged_w4a16_model_shapes_within_rms_bound(cuda, ops, workspace, out_features, in_features, batches):
    torch = cuda
    packed, scales, swizzled = synth.nvfp4_matrix(0, f"w{out_features}x{in_features}", out_features, in_features)
    for batch in batches:
        x = synth.normal_bf16(0, f"x{batch}", (batch, in_features))
        want = oracle.gemv_w4a16(packed, scales, 1.0, x, out_features, in_features, batch)
        got_bits, got_staged, _ = run_staged(torch, ops, workspace, packed, swizzled, 1.0, x, out_features,
                                             in_features, batch)
        got = synth.bf16_value(got_bits)
        assert_rms_close(got, oracle.bf16_round(want), f"staged gemv {out_features}x{in_features} b{batch}")
        assert_staged_holds(got_staged, got, f"staged output {out_features}x{in_features} b{batch}")


def test_staged_w4a16_is_bit_reproducible_and_agrees_with_the_bf16_entry(cuda, ops, workspace):
    """Split sums are taken in K order whoever arrives last: two launches give the same bits.  The
    bf16-row entry point (another kernel, another summation order) agrees within the parity bound."""
    torch = cuda
    out_features, in_features, batch = 5120, 17408, 32
    packed, scales, swizzled = synth.nvfp4_matrix(3, "repro", out_features, in_features)
    x = synth.normal_bf16(3, "repro.x", (batch, in_features))
    first, _, linear = run_staged(torch, ops, workspace, packed, swizzled, 1.0, x, out_features, in_features, batch,
                                  want_staged=False)
    for _ in range(3):
        again, _, _ = run_staged(torch, ops, workspace, packed, swizzled, 1.0, x, out_features, in_features, batch,
                                 want_staged=False)
        assert np.array_equal(first, again)
    legacy = bf16_out(torch, batch, out_features)
    linear.forward_w4a16(dev(torch, x), legacy, batch)
    torch.cuda.synchronize()
    assert_rms_close(synth.bf16_value(first), synth.bf16_value(host(legacy)), "staged vs bf16-row entry")
    assert np.mean(first != host(legacy)) < 0.02


@pytest.mark.parametrize("batch", [1, 6, 13, 32])
def test_staged_swiglu_mlp_shape(cuda, ops, workspace, batch):
    torch = cuda
    out_features, in_features = 17408, 5120
    gate = synth.nvfp4_matrix(1, "gate", out_features, in_features)
    up = synth.nvfp4_matrix(1, "up", out_features, in_features)
    x = synth.normal_bf16(1, f"x{batch}", (batch, in_features))
    want = oracle.swiglu_combine(oracle.gemv_w4a16(gate[0], gate[1], 1.0, x, out_features, in_features, batch),
                                 oracle.gemv_w4a16(up[0], up[1], 2.0, x, out_features, in_features, batch))
    gate_linear = ops.Linear(dev(torch, gate[0]), dev(torch, gate[2]), 1.0, out_features, in_features)
    up_linear = ops.Linear(dev(torch, up[0]), dev(torch, up[2]), 2.0, out_features, in_features)
    staged_out = ops.new_staged(batch, out_features)
    ops.swiglu_w4a16_staged(gate_linear, up_linear, staged_input(torch, ops, x, batch, in_features), None, staged_out,
                            batch, workspace)
    torch.cuda.synchronize()
    got = host(ops.unstage(staged_out, batch, out_features)).astype(np.float32)
    assert_rms_close(got, oracle.bf16_round(want), f"staged swiglu b{batch}")

    # ... and the chain the MLP runs: the staged output is the down projection's input
    down = synth.nvfp4_matrix(1, "down", in_features, out_features)
    down_linear = ops.Linear(dev(torch, down[0]), dev(torch, down[2]), 1.0, in_features, out_features)
    out = bf16_out(torch, batch, in_features)
    ops.w4a16_staged(down_linear, staged_out, out, None, batch, workspace)
    torch.cuda.synchronize()
    hidden_bits = synth.bf16_bits(got)
    want_down = oracle.gemv_w4a16(down[0], down[1], 1.0, hidden_bits, in_features, out_features, batch)
    assert_rms_close(synth.bf16_value(host(out)), oracle.bf16_round(want_down), f"down after staged swiglu b{batch}")


@pytest.mark.parametrize("batch,vocab", [(1, 5000), (8, 5000), (17, 5000), (32, 4096), (5, 12000), (32, 151936)])
def test_staged_lm_head_logits_and_sampling(cuda, ops, workspace, batch, vocab):
    """FP8 head (cuda/vocab_fp8.cu:162-234) with the greedy argmax folded in (cuda/sampling.cu:11-14):
    logits against the oracle, tokens exact on the kernel's own logits, and the same tokens when no
    logits are asked for."""
    torch = cuda
    hidden = 5120 if vocab < 100000 else 1024
    rows = synth.normal_bf16(8, "head", (vocab, hidden), std=0.02)
    weights, scales = oracle.fp8_quantize_rows(rows, vocab, hidden)
    x = synth.normal_bf16(8, f"h{batch}", (batch, hidden))
    want = oracle.fp8_lm_head(weights, scales, x, batch, hidden, vocab)
    staged = staged_input(torch, ops, x, batch, hidden)
    logits = torch.zeros((batch, vocab), dtype=torch.float32, device="cuda")
    tokens = dev(torch, np.full(batch, 0xFFFFFFFF, dtype=np.uint32))
    status = dev(torch, np.full(1, 7, dtype=np.uint32))
    table, row_scales = dev(torch, weights), dev(torch, scales)
    ops.fp8_lm_head_staged(table, row_scales, staged, logits, tokens, status, batch, hidden, vocab, workspace)
    torch.cuda.synchronize()
    got = host(logits)
    assert_rms_close(got, want, f"staged head b{batch} v{vocab}", bf16_grid=False)
    assert np.array_equal(host(tokens), oracle.argmax(got, vocab, batch))
    assert host(status)[0] == 0
    only_tokens = dev(torch, np.full(batch, 0xFFFFFFFF, dtype=np.uint32))
    ops.fp8_lm_head_staged(table, row_scales, staged, None, only_tokens, None, batch, hidden, vocab, workspace)
    torch.cuda.synchronize()
    assert np.array_equal(host(only_tokens), host(tokens))


def test_staged_sampling_ties_go_to_the_lower_index(cuda, ops, workspace):
    """crates/qwc-cuda/tests/sampling.rs:19-27: equal maxima -> the smaller token id, here across
    different tiles and different CTAs of the head."""
    torch = cuda
    vocab, hidden, batch = 40000, 256, 3
    weights = np.zeros((vocab, hidden), dtype=np.uint8)
    one = 0x38  # e4m3 1.0
    for row in (37000, 911, 20500, 912):
        weights[row, 0] = one
    weights[5, 1] = one
    weights[39999, 1] = one
    scales = np.ones(vocab, dtype=np.float32)
    x = np.zeros((batch, hidden), dtype=np.float32)
    x[0, 0] = 2.0   # rows 911, 912, 20500, 37000 tie at 2.0
    x[1, 1] = 3.0   # rows 5 and 39999 tie
    x[2, 0] = -1.0  # every other row is 0 > -1: the first row that is not one of the four
    tokens = dev(torch, np.zeros(batch, dtype=np.uint32))
    ops.fp8_lm_head_staged(dev(torch, weights), dev(torch, scales),
                           staged_input(torch, ops, synth.bf16_bits(x), batch, hidden), None, tokens, None, batch,
                           hidden, vocab, workspace)
    torch.cuda.synchronize()
    assert host(tokens).tolist() == [911, 5, 0]


def test_staged_entries_reject_bad_arguments(cuda, ops, workspace):
    from qwencore_b200 import abi

    torch = cuda
    packed, scales, swizzled = synth.nvfp4_matrix(0, "bad", 256, 256)
    linear = ops.Linear(dev(torch, packed), dev(torch, swizzled), 1.0, 256, 256)
    staged = ops.new_staged(4, 256)
    out = bf16_out(torch, 4, 256)
    p = lambda t: 0 if t is None else t.data_ptr()  # noqa: E731
    stream = torch.cuda.current_stream().cuda_stream

    def call(**changes):
        args = dict(packed=p(linear.packed), scales=p(linear.scales), x=p(staged), out=p(out), staged_out=0, n=256,
                    k=256, batch=4, scale=1.0, workspace=p(workspace))
        args.update(changes)
        return abi.lib.qwc_nvfp4_w4a16_staged(args["packed"], args["scales"], args["x"], args["out"],
                                              args["staged_out"], args["n"], args["k"], args["batch"], args["scale"],
                                              args["workspace"], stream)

    assert call() == 0
    for bad in (dict(packed=0), dict(x=0), dict(out=0), dict(workspace=0), dict(n=252), dict(k=128), dict(batch=0),
                dict(batch=33), dict(scale=0.0), dict(x=p(staged) + 2)):
        assert call(**bad) == abi.CUDA_ERROR_INVALID_VALUE, bad
    assert abi.lib.qwc_staged_activation_bytes(4, 256) == 256 // 8 * 16 * 8 * 2
    assert abi.lib.qwc_staged_activation_bytes(17, 256) == 256 // 8 * 32 * 8 * 2
    assert abi.lib.qwc_staged_activation_bytes(33, 256) == 0
    torch.cuda.synchronize()


# ---------------------------------------------------------------------------------------
# Regular K split with the sum left to the consumer
# ---------------------------------------------------------------------------------------

def run_split(torch, ops, packed, swizzled, x_bits, out_features, in_features, batch):
    linear = ops.Linear(dev(torch, packed), dev(torch, swizzled), 1.0, out_features, in_features)
    slices = ops.split_count(linear)
    sums = torch.zeros((slices, batch, out_features), dtype=torch.float32, device="cuda")
    ops.w4a16_split(linear, staged_input(torch, ops, x_bits, batch, in_features), sums, batch)
    return linear, slices, sums


@pytest.mark.parametrize("out_features,in_features,batch", [(5120, 4096, 32), (5120, 17408, 7), (5120, 6144, 1)])
def test_split_projection_finished_by_the_residual_norm(cuda, ops, out_features, in_features, batch):
    """Mixer output / MLP down: fp32 slices, summed by the residual RMSNorm (cuda/rmsnorm.cu:85-149 on the
    projection's bf16 values, cuda/nvfp4.cu:209-220)."""
    torch = cuda
    packed, scales, swizzled = synth.nvfp4_matrix(5, f"split{in_features}", out_features, in_features)
    x = synth.normal_bf16(5, "split.x", (batch, in_features))
    residual = synth.normal_bf16(5, "split.res", (batch, out_features), std=20.0)
    weight = synth.normal_bf16(5, "split.w", (out_features,), std=0.02)
    global_scale = 4.0
    want_rows = oracle.bf16_from_f32(oracle.gemv_w4a16(packed, scales, global_scale, x, out_features, in_features, batch))
    want_residual = residual.copy()
    want_normed = oracle.rmsnorm_bf16(want_rows, want_residual, weight, batch, out_features)

    linear, slices, sums = run_split(torch, ops, packed, swizzled, x, out_features, in_features, batch)
    assert slices >= 2
    rows = bf16_out(torch, batch, out_features)
    res_dev = dev(torch, residual)
    normed = bf16_out(torch, batch, out_features)
    staged = ops.new_staged(batch, out_features)
    ops.rmsnorm_split_staged(sums, slices, global_scale, rows, res_dev, dev(torch, weight), normed, staged, batch,
                             out_features)
    torch.cuda.synchronize()
    got_rows = synth.bf16_value(host(rows))
    assert_rms_close(got_rows, synth.bf16_value(want_rows), "split projection rows")
    assert_rms_close(synth.bf16_value(host(res_dev)), synth.bf16_value(want_residual), "residual after the split sum")
    assert_rms_close(synth.bf16_value(host(normed)), synth.bf16_value(want_normed), "norm after the split sum")
    assert_staged_holds(host(ops.unstage(staged, batch, out_features)), synth.bf16_value(host(normed)), "staged norm")
    # given its own projection rows the norm is the unsplit kernel bit for bit
    again_res = dev(torch, residual)
    again = bf16_out(torch, batch, out_features)
    ops.rmsnorm_bf16(rows, again_res, dev(torch, weight), again, batch, out_features)
    torch.cuda.synchronize()
    assert np.array_equal(host(again_res), host(res_dev)) and np.array_equal(host(again), host(normed))
    # the slices are bit-reproducible
    _, _, sums_again = run_split(torch, ops, packed, swizzled, x, out_features, in_features, batch)
    torch.cuda.synchronize()
    assert torch.equal(sums, sums_again)


def test_split_slices_summed_to_rows_and_by_the_deltanet_consumers(cuda, ops):
    """The mixer in-projection as a K split: the plain sum to bf16 rows against the oracle, and the
    DeltaNet prepare step and gated RMSNorm reading the slices give the bits they give on those rows."""
    from qwencore_b200 import abi

    torch = cuda
    v_heads, batch, hidden = 32, 9, 5120
    before = abi.get_shape()
    abi.configure(v_heads, 16)
    try:
        channels = 2 * 16 * 128 + v_heads * 128
        z_offset, a_offset = channels, channels + v_heads * 128
        b_offset = a_offset + v_heads
        width = b_offset + v_heads  # 12352
        packed, scales, swizzled = synth.nvfp4_matrix(6, "inproj", width, hidden)
        x = synth.normal_bf16(6, "inproj.x", (batch, hidden), std=0.05)
        linear, slices, sums = run_split(torch, ops, packed, swizzled, x, width, hidden, batch)
        assert slices == 3
        rows = bf16_out(torch, batch, width)
        abi.check(abi.lib.qwc_nvfp4_sum_slices(sums.data_ptr(), slices, 1.0, rows.data_ptr(), batch, width,
                                               torch.cuda.current_stream().cuda_stream), "qwc_nvfp4_sum_slices")
        torch.cuda.synchronize()
        want = oracle.gemv_w4a16(packed, scales, 1.0, x, width, hidden, batch)
        assert_rms_close(synth.bf16_value(host(rows)), oracle.bf16_round(want), "summed in-projection rows")

        capacity = batch + 2
        slots = dev(torch, np.random.default_rng(0).permutation(capacity)[:batch].astype(np.uint32))
        conv_weight = dev(torch, synth.normal_bf16(6, "conv", (channels * 4,), std=0.3))
        a_log = dev(torch, synth.normal_bf16(6, "alog", (v_heads,), std=0.5))
        dt_bias = dev(torch, synth.normal_bf16(6, "dt", (v_heads,), std=0.5))
        conv_init = np.random.default_rng(1).uniform(-1, 1, (capacity, channels, 3)).astype(np.float32)
        out_norm = dev(torch, synth.normal_bf16(6, "onorm", (128,), std=0.05))
        delta_out = dev(torch, np.random.default_rng(2).standard_normal((batch, v_heads, 128)).astype(np.float32))
        stream = torch.cuda.current_stream().cuda_stream
        results = []
        for split in (False, True):
            conv_state = dev(torch, conv_init)
            outs = [torch.zeros(n, dtype=torch.float32, device="cuda")
                    for n in (batch * 2048, batch * 2048, batch * v_heads * 128, batch * v_heads, batch * v_heads,
                              batch * 16)]
            normed = bf16_out(torch, batch, v_heads * 128)
            if split:
                abi.check(abi.lib.qwc_delta_prepare_decode_split(
                    sums.data_ptr(), slices, width, 1.0, a_offset, b_offset, conv_weight.data_ptr(), a_log.data_ptr(),
                    dt_bias.data_ptr(), conv_state.data_ptr(), slots.data_ptr(), *[o.data_ptr() for o in outs],
                    capacity, batch, stream), "qwc_delta_prepare_decode_split")
                abi.check(abi.lib.qwc_delta_gated_rmsnorm_split(
                    delta_out.data_ptr(), sums.data_ptr(), slices, width, 1.0, z_offset, out_norm.data_ptr(),
                    normed.data_ptr(), None, batch, 1e-6, stream), "qwc_delta_gated_rmsnorm_split")
            else:
                ops.delta_prepare_decode(rows, a_offset, b_offset, conv_weight, a_log, dt_bias, conv_state, slots,
                                         *outs, capacity, batch, width)
                ops.delta_gated_rmsnorm(delta_out, rows, z_offset, out_norm, normed, batch, width)
            torch.cuda.synchronize()
            results.append([host(conv_state)] + [host(o) for o in outs] + [host(normed)])
        for on_rows, on_slices in zip(*results):
            assert np.array_equal(on_rows.view(np.uint8), on_slices.view(np.uint8))
    finally:
        abi.configure(*before)


def test_delta_step_form_with_fused_gated_norm_is_the_two_kernels_bit_for_bit(cuda, ops):
    """qwc_delta_decode_int8_step: the recurrent update that fetches slots and state tiles before the
    wait for its predecessor and, with one CTA per head, runs the gated RMSNorm in the same CTA.  It
    must leave the state, the scales and the staged output of qwc_delta_decode_int8 followed by
    qwc_delta_gated_rmsnorm_staged, bit for bit (crates/qwc-cuda/cuda/delta_net.cu:177-256,
    cuda/delta_output.cu:20-64)."""
    from qwencore_b200 import abi

    torch = cuda
    v_heads, batch = 32, 32
    before = abi.get_shape()
    abi.configure(v_heads, 16)
    try:
        assert abi.lib.qwc_delta_decode_fuses_norm(batch) == 1 and abi.lib.qwc_delta_decode_fuses_norm(1) == 0
        case = synth.delta_case(9, batch, v_heads)
        width = v_heads * 128 + 64
        gate_rows = synth.normal_bf16(9, "z", (batch, width))
        out_norm = dev(torch, synth.normal_bf16(9, "onorm", (128,), std=0.05))
        stream = torch.cuda.current_stream().cuda_stream
        inputs = [dev(torch, case[name]) for name in ("slots", "q", "k", "v", "alpha", "beta", "kq")]
        gate_dev = dev(torch, gate_rows)

        state_a, scales_a = dev(torch, case["state"]), dev(torch, case["scales"])
        out_a = torch.zeros((batch, v_heads, 128), dtype=torch.float32, device="cuda")
        ops.delta_decode_slots_packed(state_a, scales_a, *inputs, out_a, case["capacity"], batch)
        staged_a = ops.new_staged(batch, v_heads * 128)
        abi.check(abi.lib.qwc_delta_gated_rmsnorm_staged(out_a.data_ptr(), gate_dev.data_ptr() + 2 * 64,
                                                         out_norm.data_ptr(), None, staged_a.data_ptr(), batch, 1e-6,
                                                         width, stream), "qwc_delta_gated_rmsnorm_staged")

        state_b, scales_b = dev(torch, case["state"]), dev(torch, case["scales"])
        out_b = torch.full((batch, v_heads, 128), 7.0, dtype=torch.float32, device="cuda")
        staged_b = ops.new_staged(batch, v_heads * 128)
        abi.check(abi.lib.qwc_delta_decode_int8_step(
            state_b.data_ptr(), scales_b.data_ptr(), *[t.data_ptr() for t in inputs], out_b.data_ptr(),
            case["capacity"], batch, None, 0, 1.0, gate_dev.data_ptr(), width, 64, out_norm.data_ptr(), 1e-6,
            staged_b.data_ptr(), stream), "qwc_delta_decode_int8_step")
        torch.cuda.synchronize()
        assert torch.equal(state_a, state_b) and torch.equal(scales_a, scales_b)
        assert torch.equal(staged_a.view(torch.int16), staged_b.view(torch.int16))
        assert bool((out_b == 7.0).all()), "the fused form leaves `out` alone"

        # without the fusion (and for a batch whose heads are split over CTAs) it is the plain update
        one = synth.delta_case(10, 1, v_heads)
        one_inputs = [dev(torch, one[name]) for name in ("slots", "q", "k", "v", "alpha", "beta", "kq")]
        results = []
        for step_form in (False, True):
            state, scales = dev(torch, one["state"]), dev(torch, one["scales"])
            out = torch.zeros((1, v_heads, 128), dtype=torch.float32, device="cuda")
            if step_form:
                abi.check(abi.lib.qwc_delta_decode_int8_step(
                    state.data_ptr(), scales.data_ptr(), *[t.data_ptr() for t in one_inputs], out.data_ptr(),
                    one["capacity"], 1, None, 0, 1.0, None, 0, 0, None, 1e-6, None, stream),
                    "qwc_delta_decode_int8_step")
            else:
                ops.delta_decode_slots_packed(state, scales, *one_inputs, out, one["capacity"], 1)
            torch.cuda.synchronize()
            results.append((host(state), host(scales), host(out)))
        for a, b in zip(*results):
            assert np.array_equal(a.view(np.uint8), b.view(np.uint8))
        staged = ops.new_staged(1, v_heads * 128)
        assert abi.lib.qwc_delta_decode_int8_step(
            state.data_ptr(), scales.data_ptr(), *[t.data_ptr() for t in one_inputs], out.data_ptr(), one["capacity"],
            1, None, 0, 1.0, gate_dev.data_ptr(), width, 64, out_norm.data_ptr(), 1e-6, staged.data_ptr(),
            stream) == abi.CUDA_ERROR_INVALID_VALUE
    finally:
        abi.configure(*before)
