"""The committed oracle vectors (tests/golden/decode_step_vectors.npz, written by
tests/golden/make_fixtures.py): the CPU oracle reproduces them bit for bit, and the CUDA kernels
meet them within the parity bound of each op."""

import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle
from qwencore_b200 import synth

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_fixtures as fixtures  # noqa: E402


@pytest.fixture(scope="module")
def vectors():
    return np.load(GOLDEN / "decode_step_vectors.npz")


@pytest.fixture(scope="module")
def ops(cuda, built_library):
    from qwencore_b200 import ops as module

    return module


def test_oracle_reproduces_the_committed_vectors_bit_for_bit(vectors):
    fresh = fixtures.build()
    assert sorted(fresh) == sorted(vectors.files)
    for name in vectors.files:
        assert fresh[name].dtype == vectors[name].dtype and fresh[name].shape == vectors[name].shape, name
        assert np.array_equal(fresh[name].view(np.uint8), vectors[name].view(np.uint8)), name


def bf16_close(got, want, what):
    want = want.astype(np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    allowed = 1e-2 * rms + 2.0 ** -7 * np.abs(want)  # bound of the parity tests for bf16 outputs
    assert np.isfinite(got).all() and np.all(np.abs(got - want) <= allowed), what


@pytest.mark.gpu
def test_kernels_meet_the_committed_vectors(cuda, ops, vectors):
    torch = cuda

    def dev(array):
        return torch.from_numpy(np.ascontiguousarray(array)).cuda()

    # NVFP4 projection, 1 / 7 / 32 rows
    for batch in fixtures.GEMV_BATCHES:
        packed, scales, swizzled, x = fixtures.gemv_inputs(batch)
        assert np.array_equal(fixtures.digest(packed, scales, x), vectors[f"gemv_b{batch}_inputs_sha256"])
        linear = ops.Linear(dev(packed), dev(swizzled), 2.0, *fixtures.GEMV_SHAPE)
        out = torch.zeros((batch, fixtures.GEMV_SHAPE[0]), dtype=torch.uint16, device="cuda")
        linear.forward_w4a16(dev(x), out, batch)
        torch.cuda.synchronize()
        bf16_close(synth.bf16_value(out.cpu().numpy()), vectors[f"gemv_b{batch}_out"], f"gemv batch {batch}")

    # packed attention: three ragged rows, page 16, per-head scales, output gate, split context
    case = fixtures.attention_inputs()
    rows = len(fixtures.ATTENTION_CONTEXTS)
    out = torch.zeros((rows, 24, 256), dtype=torch.uint16, device="cuda")
    partitions = 4
    workspace = torch.zeros(ops.packed_workspace_bytes(rows, partitions), dtype=torch.uint8, device="cuda")
    ops.gated_packed(dev(case["query"]), dev(case["gate_projection"]), dev(case["key_cache"]),
                     dev(case["value_cache"]), dev(case["block_tables"]), dev(case["contexts"]), case["max_blocks"],
                     out, rows, 0, partitions, workspace, fixtures.ATTENTION_PAGE, dev(case["k_scale"]),
                     dev(case["v_scale"]))
    torch.cuda.synchronize()
    bf16_close(synth.bf16_value(out.cpu().numpy()), vectors["attention_out"], "attention")

    # int8 DeltaNet step: outputs within 1e-2 of the RMS, scales equal to a few ulps, codes within one step
    from qwencore_b200 import abi

    before = abi.get_shape()
    abi.configure(fixtures.DELTA_HEADS, before[1])
    try:
        case = fixtures.delta_inputs()
        state, scales = dev(case["state"]), dev(case["scales"])
        result = torch.zeros((fixtures.DELTA_BATCH, fixtures.DELTA_HEADS, 128), dtype=torch.float32, device="cuda")
        ops.delta_decode_slots_packed(state, scales, dev(case["slots"]), dev(case["q"]), dev(case["k"]),
                                      dev(case["v"]), dev(case["alpha"]), dev(case["beta"]), dev(case["kq"]), result,
                                      case["capacity"], fixtures.DELTA_BATCH)
        torch.cuda.synchronize()
    finally:
        abi.configure(*before)
    want = vectors["delta_out"].astype(np.float64)
    assert np.max(np.abs(result.cpu().numpy() - want)) <= 1e-2 * np.sqrt(np.mean(want ** 2))
    got_scales = scales.cpu().numpy()[case["slots"]]
    assert np.allclose(got_scales, vectors["delta_scales"], rtol=1e-5, atol=0)
    want_state, want_scales = case["state"].copy(), case["scales"].copy()
    oracle.delta_decode_int8(want_state, want_scales, case["slots"], case["q"], case["k"], case["v"], case["alpha"],
                             case["beta"], case["kq"], fixtures.DELTA_BATCH, fixtures.DELTA_HEADS)
    assert np.array_equal(fixtures.digest(want_state), vectors["delta_state_sha256"])
    assert np.abs(state.cpu().numpy().astype(np.int32) - want_state.astype(np.int32)).max() <= 1
    assert abi.lib.qwc_device_status() == 0
