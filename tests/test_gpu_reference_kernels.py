"""GPU-side arbiter: the reference's own CUDA kernels (crates/qwc-cuda/cuda/*.cu, recompiled for
sm_100a by oracle/Makefile into oracle/_ref/libqwc_ref_kernels.so) run on the same inputs as this
library, at the shapes the reference supports (48 value heads, page 64, at most 8 projection rows).

Integer and storage results (state codes and scales, conv history, gathered embedding rows, argmax)
must be identical; floating-point outputs must sit within the parity bound of each op.  The test is
skipped where the rebuilt library is absent (it is built only where the reference tree is mounted)."""

import contextlib
import ctypes
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle
from qwencore_b200 import synth

REFERENCE_LIBRARY = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libqwc_ref_kernels.so"


@pytest.fixture(scope="module")
def both(cuda, built_library):
    from qwencore_b200 import abi, ops

    if not REFERENCE_LIBRARY.exists():
        pytest.skip("oracle/_ref/libqwc_ref_kernels.so has not been built")
    reference = ctypes.CDLL(str(REFERENCE_LIBRARY))
    for name, (restype, argtypes) in abi.KERNEL_SYMBOLS.items():
        if hasattr(reference, name):
            function = getattr(reference, name)
            function.restype, function.argtypes = restype, argtypes
    ours = abi.lib

    @contextlib.contextmanager
    def reference_kernels():
        abi.lib = reference
        try:
            yield
        finally:
            abi.lib = ours

    before = abi.get_shape()
    abi.configure(48, 64)  # the constants the reference kernels are compiled with
    yield cuda, ops, reference_kernels
    abi.configure(*before)
    assert ours.qwc_device_status() == 0


def dev(torch, array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def host(tensor):
    return tensor.cpu().numpy()


def bf16_close(got, want, what, bound=1e-2):
    want = want.astype(np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    allowed = bound * rms + 2.0 ** -7 * np.abs(want)
    assert np.isfinite(got).all() and np.all(np.abs(got - want) <= allowed), what


@pytest.mark.gpu
@pytest.mark.parametrize("out_features,in_features", [(1024, 5120), (5120, 4096), (12288, 5120)])
def test_projection_agrees_with_the_reference_kernel(both, out_features, in_features):
    torch, ops, reference_kernels = both
    packed, scales, swizzled = synth.nvfp4_matrix(21, f"ref{out_features}", out_features, in_features)
    linear = ops.Linear(dev(torch, packed), dev(torch, swizzled), 4.0, out_features, in_features)
    for batch in (1, 3, 8):
        x = dev(torch, synth.normal_bf16(21, f"x{batch}", (batch, in_features)))
        mine = torch.zeros((batch, out_features), dtype=torch.uint16, device="cuda")
        theirs = torch.zeros_like(mine)
        linear.forward_w4a16(x, mine, batch)
        with reference_kernels():
            linear.forward_w4a16(x, theirs, batch)
        torch.cuda.synchronize()
        bf16_close(synth.bf16_value(host(mine)), synth.bf16_value(host(theirs)), f"projection batch {batch}")
        # both round the same fp32 dot product to bf16: almost every element is the same code
        assert np.mean(host(mine) != host(theirs)) < 0.02


@pytest.mark.gpu
def test_swiglu_agrees_with_the_reference_kernel(both):
    torch, ops, reference_kernels = both
    N, K = 2048, 5120
    gate = ops.Linear(*(dev(torch, a) for a in synth.nvfp4_matrix(22, "gate", N, K)[::2]), 2.0, N, K)
    up = ops.Linear(*(dev(torch, a) for a in synth.nvfp4_matrix(22, "up", N, K)[::2]), 4.0, N, K)
    for batch in (1, 6):
        x = dev(torch, synth.normal_bf16(22, f"x{batch}", (batch, K), std=0.25))
        mine = torch.zeros((batch, N), dtype=torch.uint16, device="cuda")
        theirs = torch.zeros_like(mine)
        ops.swiglu_w4a16(gate, up, x, mine, batch)
        with reference_kernels():
            ops.swiglu_w4a16(gate, up, x, theirs, batch)
        torch.cuda.synchronize()
        bf16_close(synth.bf16_value(host(mine)), synth.bf16_value(host(theirs)), f"swiglu batch {batch}")


@pytest.mark.gpu
def test_delta_step_agrees_with_the_reference_kernel(both):
    torch, ops, reference_kernels = both
    batch, heads = 5, 48
    case = synth.delta_case(23, batch, heads)
    results = []
    for use_reference in (False, True):
        state, scales = dev(torch, case["state"]), dev(torch, case["scales"])
        out = torch.zeros((batch, heads, 128), dtype=torch.float32, device="cuda")
        arguments = (state, scales, dev(torch, case["slots"]), dev(torch, case["q"]), dev(torch, case["k"]),
                     dev(torch, case["v"]), dev(torch, case["alpha"]), dev(torch, case["beta"]),
                     dev(torch, case["kq"]), out, case["capacity"], batch)
        with (reference_kernels() if use_reference else contextlib.nullcontext()):
            ops.delta_decode_slots_packed(*arguments)
        torch.cuda.synchronize()
        results.append((host(state), host(scales), host(out)))
    (state_a, scales_a, out_a), (state_b, scales_b, out_b) = results
    # the dot products are summed in a different order, so a row's peak may move by an ulp and a code
    # that sat on a rounding boundary by one step; nothing more
    assert np.abs(state_a.astype(np.int32) - state_b.astype(np.int32)).max() <= 1
    assert np.mean(state_a != state_b) < 1e-3
    assert np.allclose(scales_a, scales_b, rtol=1e-5, atol=0)
    rms = np.sqrt(np.mean(out_b.astype(np.float64) ** 2))
    assert np.max(np.abs(out_a - out_b)) <= 1e-3 * rms


@pytest.mark.gpu
def test_glue_kernels_agree_with_the_reference_kernels(both):
    torch, ops, reference_kernels = both
    rng = synth.generator(24, "glue")

    # residual RMSNorm: the residual sum and the normalised row are bf16 roundings of the same values
    batch, hidden = 6, 5120
    x = synth.normal_bf16(24, "x", (batch, hidden))
    residual = synth.normal_bf16(24, "res", (batch, hidden), std=3.0)
    weight = synth.normal_bf16(24, "w", (hidden,), std=0.02)
    outputs = []
    for use_reference in (False, True):
        res = dev(torch, residual)
        out = torch.zeros((batch, hidden), dtype=torch.uint16, device="cuda")
        with (reference_kernels() if use_reference else contextlib.nullcontext()):
            ops.rmsnorm_bf16(dev(torch, x), res, dev(torch, weight), out, batch, hidden)
        torch.cuda.synchronize()
        outputs.append((host(res), host(out)))
    assert np.array_equal(outputs[0][0], outputs[1][0])
    bf16_close(synth.bf16_value(outputs[0][1]), synth.bf16_value(outputs[1][1]), "rmsnorm")
    assert np.mean(outputs[0][1] != outputs[1][1]) < 0.02

    # DeltaNet prepare (48 value heads): conv history bit-exact, gates and normalised q, k close
    batch, capacity, k_heads, v_heads, dim = 4, 6, 16, 48, 128
    channels = 2 * k_heads * dim + v_heads * dim
    z_offset = channels
    a_offset = z_offset + v_heads * dim
    b_offset = a_offset + v_heads
    stride = b_offset + v_heads
    mixed = synth.bf16_bits(rng.standard_normal((batch, stride), dtype=np.float32))
    conv_weight = synth.bf16_bits(rng.standard_normal((channels, 4), dtype=np.float32) * 0.5)
    a_log = synth.bf16_bits(rng.standard_normal(v_heads, dtype=np.float32) * 0.5)
    dt_bias = synth.bf16_bits(rng.standard_normal(v_heads, dtype=np.float32) * 0.5)
    conv_state = rng.standard_normal((capacity, channels, 3), dtype=np.float32)
    slots = rng.permutation(capacity)[:batch].astype(np.uint32)
    values = rng.standard_normal((batch, v_heads, dim), dtype=np.float32)
    norm_weight = synth.bf16_bits(1.0 + 0.1 * rng.standard_normal(dim, dtype=np.float32))
    outputs = []
    for use_reference in (False, True):
        d_mixed, d_state = dev(torch, mixed), dev(torch, conv_state)
        tq = torch.zeros((batch, k_heads, dim), dtype=torch.float32, device="cuda")
        tk = torch.zeros_like(tq)
        tv = torch.zeros((batch, v_heads, dim), dtype=torch.float32, device="cuda")
        ta = torch.zeros((batch, v_heads), dtype=torch.float32, device="cuda")
        tb = torch.zeros_like(ta)
        tkq = torch.zeros((batch, k_heads), dtype=torch.float32, device="cuda")
        normed = torch.zeros((batch, v_heads, dim), dtype=torch.uint16, device="cuda")
        with (reference_kernels() if use_reference else contextlib.nullcontext()):
            ops.delta_prepare_decode(d_mixed, a_offset, b_offset, dev(torch, conv_weight), dev(torch, a_log),
                                     dev(torch, dt_bias), d_state, dev(torch, slots), tq, tk, tv, ta, tb, tkq,
                                     capacity, batch, stride)
            ops.delta_gated_rmsnorm(dev(torch, values), d_mixed, z_offset, dev(torch, norm_weight), normed, batch,
                                    stride)
        torch.cuda.synchronize()
        outputs.append([host(t) for t in (d_state, tv, tq, tk, ta, tb, tkq, normed)])
    ours, theirs = outputs
    assert np.array_equal(ours[0], theirs[0]), "conv history"
    assert np.array_equal(ours[1], theirs[1]), "v after conv and SiLU (bf16-snapped)"
    for index, name in [(2, "q"), (3, "k"), (4, "alpha"), (5, "beta"), (6, "kq")]:
        assert np.allclose(ours[index], theirs[index], rtol=1e-4, atol=1e-7), name
    bf16_close(synth.bf16_value(ours[7]), synth.bf16_value(theirs[7]), "gated rmsnorm")

    # FP8 embedding gather: a copy with a scale, bit-exact; FP8 head and argmax
    vocab, hidden, batch = 4099, 5120, 4
    rows = synth.normal_bf16(24, "head", (vocab, hidden), std=0.02)
    weights, scales = oracle.fp8_quantize_rows(rows, vocab, hidden)
    tokens = np.array([0, 17, vocab - 1, 1234], dtype=np.uint32)
    hidden_rows = synth.normal_bf16(24, "h", (batch, hidden))
    outputs = []
    for use_reference in (False, True):
        gathered = torch.zeros((batch, hidden), dtype=torch.uint16, device="cuda")
        logits = torch.zeros((batch, vocab), dtype=torch.float32, device="cuda")
        parts = 64
        partial_values = torch.zeros(batch * parts, dtype=torch.float32, device="cuda")
        partial_indices = torch.zeros(batch * parts, dtype=torch.int32, device="cuda")
        sampled = torch.zeros(batch, dtype=torch.int32, device="cuda")
        with (reference_kernels() if use_reference else contextlib.nullcontext()):
            ops.fp8_embedding_gather(dev(torch, weights), dev(torch, scales), dev(torch, tokens), gathered, batch,
                                     hidden, vocab)
            ops.fp8_lm_head(dev(torch, weights), dev(torch, scales), dev(torch, hidden_rows), logits, batch, hidden,
                            vocab)
            ops.argmax(logits, partial_values, partial_indices, sampled, vocab, batch, parts)
        torch.cuda.synchronize()
        outputs.append((host(gathered), host(logits), host(sampled)))
    assert np.array_equal(outputs[0][0], outputs[1][0]), "embedding rows"
    rms = np.sqrt(np.mean(outputs[1][1].astype(np.float64) ** 2))
    assert np.max(np.abs(outputs[0][1] - outputs[1][1])) <= 1e-2 * rms, "lm_head logits"
    assert np.array_equal(outputs[0][2], oracle.argmax(outputs[0][1], vocab, batch).astype(np.int32))
    assert np.array_equal(outputs[1][2], oracle.argmax(outputs[1][1], vocab, batch).astype(np.int32))


@pytest.mark.gpu
def test_attention_prepare_agrees_with_the_reference_kernel(both):
    """QK-norm + partial RoPE + e4m3 page write through the reference's own entry point (page 64)."""
    from qwencore_b200 import abi

    torch, ops, reference_kernels = both
    batch, num_blocks, page_size = 3, 7, 64
    rng = synth.generator(25, "attnprep")
    query_gate = synth.bf16_bits(rng.standard_normal((batch, 24 * 512), dtype=np.float32))
    key_proj = synth.bf16_bits(rng.standard_normal((batch, 4 * 256), dtype=np.float32))
    value_proj = synth.bf16_bits(rng.standard_normal((batch, 4 * 256), dtype=np.float32))
    qw = synth.bf16_bits(rng.standard_normal(256, dtype=np.float32) * 0.1)
    kw = synth.bf16_bits(rng.standard_normal(256, dtype=np.float32) * 0.1)
    positions = np.array([0, 5 * page_size + 3, 2 * page_size + page_size - 1], dtype=np.uint32)
    cosine, sine = oracle.rope_rows(positions)
    physical = np.array([6, 2, 4], dtype=np.uint32)
    offsets = (positions % page_size).astype(np.uint32)
    outputs = []
    for use_reference in (False, True):
        key_cache = torch.zeros((num_blocks, 4, page_size, 256), dtype=torch.uint8, device="cuda")
        value_cache = torch.zeros_like(key_cache)
        query = torch.zeros((batch, 24, 256), dtype=torch.uint16, device="cuda")
        tensors = [dev(torch, a) for a in (query_gate, key_proj, value_proj, qw, kw, cosine, sine, physical, offsets)]
        with (reference_kernels() if use_reference else contextlib.nullcontext()):
            abi.check(abi.lib.qwc_prepare_attention_decode_fp8(
                *(t.data_ptr() for t in tensors), query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                batch, 1e-6, torch.cuda.current_stream().cuda_stream), "qwc_prepare_attention_decode_fp8")
        torch.cuda.synchronize()
        outputs.append((host(query), host(key_cache), host(value_cache)))
    (q_a, k_a, v_a), (q_b, k_b, v_b) = outputs
    assert np.array_equal(v_a, v_b), "V pages: a pure bf16 -> e4m3 conversion"
    steps = np.abs(k_a.astype(np.int32) - k_b.astype(np.int32))
    assert steps.max() <= 1 and np.mean(steps > 0) < 0.02, "K pages: at most one e4m3 step on a few codes"
    assert np.array_equal(k_a != 0, k_b != 0) or np.mean((k_a != 0) != (k_b != 0)) < 1e-3
    bf16_close(synth.bf16_value(q_a), synth.bf16_value(q_b), "query")
    assert np.mean(q_a != q_b) < 0.02
