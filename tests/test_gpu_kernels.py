"""GPU parity: every kernel through the C ABI against the CPU oracle on seeded inputs.

Tolerances: floating-point outputs must satisfy max|gpu - oracle| <= 1e-2 * RMS(oracle)
(the bound the north star states); indexing, page tables, slot packing and the int8
requantiser are compared bit for bit.  Where the reference has its own test for a case,
its name and tolerance are cited and also applied.
"""

import numpy as np
import pytest

from oracle import oracle
from qwencore_b200 import synth

pytestmark = pytest.mark.gpu

RMS_BOUND = 1.0e-2


def dev(torch, array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def host(tensor):
    return tensor.detach().cpu().numpy()


def bf16_out(torch, *shape):
    return dev(torch, np.zeros(shape, dtype=np.uint16))


def u32_out(torch, *shape, fill=0):
    return dev(torch, np.full(shape, fill, dtype=np.uint32))


# (comparison, elements that needed the bf16 grid term on top of 1e-2 * RMS, elements compared)
GRID_TERM_USE = []


def assert_rms_close(got, want, what, bound=RMS_BOUND, bf16_grid=True):
    """max|got - want| <= bound * RMS(want).  A bf16 output cannot meet that bound by itself
    beyond 2.6 RMS (its grid step there exceeds 1e-2 RMS), so for bf16 outputs one grid step
    of the expected value (at most 2^-7 relative) is allowed on top."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    allowed = bound * rms + (2.0 ** -7 * np.abs(want) if bf16_grid else 0.0)
    if bf16_grid:  # how many elements the plain bound alone would have failed: printed with the test summary
        GRID_TERM_USE.append((what, int(np.count_nonzero(np.abs(got - want) > bound * rms)), int(got.size)))
    excess = np.abs(got - want) - allowed
    worst = np.unravel_index(np.argmax(excess), excess.shape)
    assert excess[worst] <= 0, (f"{what}: |{got[worst]:.6g} - {want[worst]:.6g}| exceeds {bound} * rms "
                                f"{rms:.4g} at {worst}")


@pytest.fixture(scope="module")
def ops(cuda, built_library):
    from qwencore_b200 import abi, ops as module

    yield module
    assert abi.lib.qwc_device_status() == 0, "a bounded device wait gave up during the tests"


class LcgRng:
    """The generator of the reference's GEMV test (crates/qwc-cuda/tests/nvfp4.rs:7-21)."""

    def __init__(self, seed):
        self.state = seed

    def next_u8(self):
        self.state = (self.state * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        return self.state >> 56

    def next_f32(self):
        return np.float32(np.float32(self.next_u8()) / np.float32(255.0) * np.float32(2.0) - np.float32(1.0))


# ---------------------------------------------------------------------------------------
# NVFP4 W4A16
# ---------------------------------------------------------------------------------------

def run_gemv(torch, ops, packed, scales, swizzled, global_scale, x_bits, out_features, in_features, batch):
    linear = ops.Linear(dev(torch, packed), dev(torch, swizzled), global_scale, out_features, in_features)
    out = bf16_out(torch, batch, out_features)
    linear.forward_w4a16(dev(torch, x_bits), out, batch)
    torch.cuda.synchronize()
    return synth.bf16_value(host(out)), linear


def test_w4a16_matches_cpu_for_all_supported_batches(cuda, ops):
    """crates/qwc-cuda/tests/nvfp4.rs:23-111 (OUT = 37 checks a ragged last tile), extended to 32 rows."""
    torch = cuda
    OUT, IN = 37, 512
    rng = LcgRng(0x4A165090)
    packed = np.array([rng.next_u8() for _ in range(OUT * IN // 2)], dtype=np.uint8).reshape(OUT, IN // 2)
    up_packed = np.array([rng.next_u8() for _ in range(OUT * IN // 2)], dtype=np.uint8).reshape(OUT, IN // 2)
    codes = [0x30, 0x38, 0x3C, 0x40]
    scales = np.array([codes[i % 4] for i in range(OUT * IN // 16)], dtype=np.uint8).reshape(OUT, IN // 16)
    swizzled = synth.swizzle_block_scales(scales, OUT, IN)
    for batch in [1, 2, 3, 4, 7, 8, 9, 16, 17, 31, 32]:
        x = synth.bf16_bits(np.array([rng.next_f32() for _ in range(batch * IN)], dtype=np.float32).reshape(batch, IN))
        want = oracle.gemv_w4a16(packed, scales, 8.0, x, OUT, IN, batch)
        got, gate = run_gemv(torch, ops, packed, scales, swizzled, 8.0, x, OUT, IN, batch)
        tolerance = 0.035 + np.abs(want) * 0.012  # tests/nvfp4.rs:68
        assert np.all(np.abs(got - want) <= tolerance), f"batch {batch}"

        want_up = oracle.gemv_w4a16(up_packed, scales, 4.0, x, OUT, IN, batch)
        want_fused = oracle.swiglu_combine(want, want_up)
        up = ops.Linear(dev(torch, up_packed), dev(torch, swizzled), 4.0, OUT, IN)
        fused = bf16_out(torch, batch, OUT)
        ops.swiglu_w4a16(gate, up, dev(torch, x), fused, batch)
        torch.cuda.synchronize()
        got_fused = synth.bf16_value(host(fused))
        tolerance = 0.075 + np.abs(want_fused) * 0.025  # tests/nvfp4.rs:103
        assert np.all(np.abs(got_fused - want_fused) <= tolerance), f"fused batch {batch}"


@pytest.mark.parametrize("out_features,in_features,batches", [
    (34816, 5120, [1, 32]),      # benchmark config 0 shape (fused gate_up) and the c=32 case
    (12352, 5120, [5, 16]),      # mixer in-proj of the 32-value-head model: 96.5 row blocks
    (5120, 17408, [1, 8, 32]),   # down: narrow output, K split across a cluster
    (5120, 4096, [2, 24]),       # la_out
    (1024, 5120, [1, 12]),       # k / v projections
])
def test_w4a16_model_shapes_up_to_32_rows_oracle_generalisation_beyond_reference_batch_8(cuda, ops, out_features,
                                                                                          in_features, batches):
    torch = cuda
    packed, scales, swizzled = synth.nvfp4_matrix(0, f"w{out_features}x{in_features}", out_features, in_features)
    for batch in batches:
        x = synth.normal_bf16(0, f"x{batch}", (batch, in_features))
        want = oracle.gemv_w4a16(packed, scales, 1.0, x, out_features, in_features, batch)
        got, _ = run_gemv(torch, ops, packed, scales, swizzled, 1.0, x, out_features, in_features, batch)
        assert_rms_close(got, oracle.bf16_round(want), f"gemv {out_features}x{in_features} b{batch}")


def test_prefetch_next_hint_changes_no_result_and_rejects_bad_arguments(cuda, ops):
    """qwc_nvfp4_prefetch_next only moves lines into L2: a hinted launch stores the same bytes."""
    torch = cuda
    from qwencore_b200 import abi
    N, K, batch = 5120, 6144, 32
    packed, scales, swizzled = synth.nvfp4_matrix(3, "hinted", N, K)
    other_p, _, other_sw = synth.nvfp4_matrix(3, "after", 12352, 5120)
    up_p, _, up_sw = synth.nvfp4_matrix(3, "after_up", 12352, 5120)
    x = dev(torch, synth.normal_bf16(3, "x", (batch, K)))
    linear = ops.Linear(dev(torch, packed), dev(torch, swizzled), 1.0, N, K)
    after = ops.Linear(dev(torch, other_p), dev(torch, other_sw), 1.0, 12352, 5120)
    after_up = ops.Linear(dev(torch, up_p), dev(torch, up_sw), 1.0, 12352, 5120)
    plain = bf16_out(torch, batch, N)
    linear.forward_w4a16(x, plain, batch)
    for second in (None, after_up):
        hinted = bf16_out(torch, batch, N)
        ops.prefetch_next(after, second)
        linear.forward_w4a16(x, hinted, batch)
        torch.cuda.synchronize()
        assert np.array_equal(host(hinted), host(plain))
    table = torch.zeros((4096, 5120), dtype=torch.uint8, device="cuda")
    assert abi.lib.qwc_nvfp4_prefetch_next(table.data_ptr(), None, None, None, 4096, 5120, 2) == 0
    hinted = bf16_out(torch, batch, N)
    linear.forward_w4a16(x, hinted, batch)
    torch.cuda.synchronize()
    assert np.array_equal(host(hinted), host(plain))
    invalid = 1  # cudaErrorInvalidValue
    good = (after.packed.data_ptr(), after.scales.data_ptr())
    assert abi.lib.qwc_nvfp4_prefetch_next(None, good[1], None, None, 12352, 5120, 0) == invalid
    assert abi.lib.qwc_nvfp4_prefetch_next(good[0], None, None, None, 12352, 5120, 0) == invalid
    assert abi.lib.qwc_nvfp4_prefetch_next(good[0], good[1], None, None, 12352, 5120, 1) == invalid
    assert abi.lib.qwc_nvfp4_prefetch_next(good[0], good[1], None, None, 12352, 5000, 0) == invalid
    assert abi.lib.qwc_nvfp4_prefetch_next(good[0], good[1], None, None, 0, 5120, 0) == invalid
    assert abi.lib.qwc_nvfp4_prefetch_next(good[0], good[1], None, None, 12352, 5120, 5) == invalid
    assert abi.lib.qwc_nvfp4_prefetch_next(good[0] + 8, good[1], None, None, 12352, 5120, 0) == invalid
    assert abi.lib.qwc_device_status() == 0


@pytest.mark.parametrize("batch", [1, 6, 13, 32])
def test_swiglu_w4a16_mlp_shape(cuda, ops, batch):
    torch = cuda
    N, K = 17408, 5120
    gate_p, gate_s, gate_sw = synth.nvfp4_matrix(1, "gate", N, K)
    up_p, up_s, up_sw = synth.nvfp4_matrix(1, "up", N, K)
    x = synth.normal_bf16(1, f"x{batch}", (batch, K), std=0.25)
    want = oracle.swiglu_combine(oracle.gemv_w4a16(gate_p, gate_s, 2.0, x, N, K, batch),
                                 oracle.gemv_w4a16(up_p, up_s, 4.0, x, N, K, batch))
    gate = ops.Linear(dev(torch, gate_p), dev(torch, gate_sw), 2.0, N, K)
    up = ops.Linear(dev(torch, up_p), dev(torch, up_sw), 4.0, N, K)
    out = bf16_out(torch, batch, N)
    ops.swiglu_w4a16(gate, up, dev(torch, x), out, batch)
    torch.cuda.synchronize()
    assert_rms_close(synth.bf16_value(host(out)), oracle.bf16_round(want), f"swiglu b{batch}")


def test_w4a16_rejects_bad_arguments(cuda, ops):
    from qwencore_b200 import abi

    lib = abi.lib
    buffer = cuda.zeros(4096, dtype=cuda.uint8, device="cuda").data_ptr()
    assert lib.qwc_nvfp4_w4a16(0, buffer, buffer, buffer, 16, 256, 1, 1.0, 0) == abi.CUDA_ERROR_INVALID_VALUE
    assert lib.qwc_nvfp4_w4a16(buffer, buffer, buffer, buffer, 16, 128, 1, 1.0, 0) == abi.CUDA_ERROR_INVALID_VALUE
    assert lib.qwc_nvfp4_w4a16(buffer, buffer, buffer, buffer, 16, 256, 33, 1.0, 0) == abi.CUDA_ERROR_INVALID_VALUE
    assert lib.qwc_nvfp4_w4a16(buffer, buffer, buffer, buffer, 16, 256, 1, 0.0, 0) == abi.CUDA_ERROR_INVALID_VALUE


# ---------------------------------------------------------------------------------------
# Packed paged attention
# ---------------------------------------------------------------------------------------

def run_attention(torch, ops, case, page_size, partitions, batch=None):
    batch = batch or case["contexts"].size
    out = bf16_out(torch, batch, 24, 256)
    workspace = None
    if partitions > 1:
        workspace = torch.zeros(ops.packed_workspace_bytes(batch, partitions), dtype=torch.uint8, device="cuda")
    gate = None if case["gate_projection"] is None else dev(torch, case["gate_projection"])
    ks = None if case["k_scale"] is None else dev(torch, case["k_scale"])
    vs = None if case["v_scale"] is None else dev(torch, case["v_scale"])
    ops.gated_packed(dev(torch, case["query"]), gate, dev(torch, case["key_cache"]), dev(torch, case["value_cache"]),
                     dev(torch, case["block_tables"]), dev(torch, case["contexts"]), case["max_blocks"], out, batch, 0,
                     partitions, workspace, page_size, ks, vs)
    torch.cuda.synchronize()
    return synth.bf16_value(host(out))


def attention_oracle(case, page_size):
    return oracle.paged_attention_fp8(case["query"], case["gate_projection"], case["key_cache"], case["value_cache"],
                                      case["block_tables"], case["contexts"], case["max_blocks"],
                                      batch=case["contexts"].size, page_size=page_size, k_scale=case["k_scale"],
                                      v_scale=case["v_scale"])


def check_attention(got, want, what):
    # reference tolerance (crates/qwc-cuda/tests/paged_attention.rs:115,888) and the RMS bound
    assert np.all(np.abs(got - want) <= 0.004 + 0.004 * np.abs(want) + 2.0 ** -8 * np.abs(want)), what
    assert_rms_close(got, want, what)


@pytest.mark.parametrize("partitions", [1, 3])
def test_packed_attention_short_contexts_reversed_table(cuda, ops, partitions):
    """crates/qwc-cuda/tests/paged_attention.rs:10-131: contexts 23 and 257, page 64, reversed table."""
    case = synth.attention_case(11, [23, 257], page_size=64)
    for b in range(2):
        n = int((case["contexts"][b] + 63) // 64)
        case["block_tables"][b, :n] = case["block_tables"][b, :n][::-1].copy()
    check_attention(run_attention(cuda, ops, case, 64, partitions), attention_oracle(case, 64), "ctx 23/257")


@pytest.mark.parametrize("page_size,partitions", [(64, 1), (64, 5), (16, 1), (16, 8)],
                         ids=["page64_reference_shape", "page64_split_reference_shape",
                              "page16_oracle_generalisation", "page16_split_oracle_generalisation"])
def test_packed_attention_ragged_rows(cuda, ops, page_size, partitions):
    """crates/qwc-cuda/tests/paged_attention.rs:950-973: ragged rows with per-row permuted tables."""
    case = synth.attention_case(12, [1, 63, 64, 65, 3000, 777, 4096], page_size=page_size, with_gate=True)
    check_attention(run_attention(cuda, ops, case, page_size, partitions), attention_oracle(case, page_size),
                    f"ragged page {page_size} P{partitions}")


def test_packed_attention_benchmark_config_page16_scaled_oracle_generalisation_no_reference_test(cuda, ops):
    """Benchmark config 1: 32 sequences, contexts uniform in [128, 2048], page 16, per-head KV scale."""
    contexts = synth.uniform_contexts(0, 32, 128, 2048)
    case = synth.attention_case(0, contexts, page_size=16, with_gate=False, scaled=True)
    want = attention_oracle(case, 16)
    for partitions in (1, 4):
        check_attention(run_attention(cuda, ops, case, 16, partitions), want, f"config 1 P{partitions}")


def test_packed_attention_split_matches_unsplit_and_oversized_workspace(cuda, ops):
    """crates/qwc-cuda/tests/paged_attention.rs:977-1031 and :735-764."""
    torch = cuda
    case = synth.attention_case(13, [2048, 300, 5000], page_size=16, with_gate=True)
    unsplit = run_attention(torch, ops, case, 16, 1)
    split = run_attention(torch, ops, case, 16, 7)
    assert np.max(np.abs(unsplit - split)) <= 0.004 + 0.01 * np.max(np.abs(unsplit))
    # more partitions than 16-token units for the short row: empty partitions must merge cleanly
    many = run_attention(torch, ops, case, 16, 40)
    assert np.max(np.abs(unsplit - many)) <= 0.004 + 0.01 * np.max(np.abs(unsplit))


def test_packed_attention_sharp_softmax(cuda, ops):
    """crates/qwc-cuda/tests/paged_attention.rs:1038-1099: one key dominates the softmax."""
    case = synth.attention_case(14, [900], page_size=16)
    keys = synth.e4m3_decode(case["key_cache"])
    page = case["block_tables"][0, 411 // 16]
    query = synth.bf16_value(case["query"])
    for kv in range(4):
        boost = np.mean(query[0, kv * 6:(kv + 1) * 6], axis=0)
        keys[page, kv, 411 % 16] = np.clip(boost * 40.0, -448, 448)
    case["key_cache"] = synth.e4m3_encode(keys)
    got = run_attention(cuda, ops, case, 16, 2)
    want = attention_oracle(case, 16)
    scale = np.max(np.abs(want))
    assert np.max(np.abs(got - want)) <= 0.006 * scale + 0.004


def test_packed_attention_legacy_entry_uses_configured_page_size(cuda, ops):
    from qwencore_b200 import abi

    torch = cuda
    case = synth.attention_case(15, [70, 129], page_size=64, with_gate=True)
    before = abi.get_shape()
    try:
        abi.configure(before[0], 64)
        out = bf16_out(torch, 2, 24, 256)
        ops.gated_packed_legacy(dev(torch, case["query"]), dev(torch, case["gate_projection"]),
                                dev(torch, case["key_cache"]), dev(torch, case["value_cache"]),
                                dev(torch, case["block_tables"]), dev(torch, case["contexts"]), case["max_blocks"],
                                out, 2, 0, 1, None)
        torch.cuda.synchronize()
        check_attention(synth.bf16_value(host(out)), attention_oracle(case, 64), "legacy entry")
        with pytest.raises(abi.QwcError) as error:  # segment tiles are prefill shapes
            ops.gated_packed_legacy(dev(torch, case["query"]), None, dev(torch, case["key_cache"]),
                                    dev(torch, case["value_cache"]), dev(torch, case["block_tables"]),
                                    dev(torch, case["contexts"]), case["max_blocks"], out, 2, 0, 1, None, tile_size=32)
        assert error.value.code == abi.CUDA_ERROR_NOT_SUPPORTED
        with pytest.raises(abi.QwcError) as error:  # workspace too small (paged_attention.cu:1876-1880)
            ops.gated_packed_legacy(dev(torch, case["query"]), None, dev(torch, case["key_cache"]),
                                    dev(torch, case["value_cache"]), dev(torch, case["block_tables"]),
                                    dev(torch, case["contexts"]), case["max_blocks"], out, 2, 0, 4,
                                    torch.zeros(16, dtype=torch.uint8, device="cuda"))
        assert error.value.code == abi.CUDA_ERROR_INVALID_VALUE
    finally:
        abi.configure(*before)


# ---------------------------------------------------------------------------------------
# Gated DeltaNet int8 step
# ---------------------------------------------------------------------------------------

def run_delta(torch, ops, case, batch, v_heads, beta=None):
    from qwencore_b200 import abi

    before = abi.get_shape()
    abi.configure(v_heads, before[1])
    try:
        state = dev(torch, case["state"])
        scales = dev(torch, case["scales"])
        out = torch.zeros((batch, v_heads, 128), dtype=torch.float32, device="cuda")
        ops.delta_decode_slots_packed(state, scales, dev(torch, case["slots"]), dev(torch, case["q"]),
                                      dev(torch, case["k"]), dev(torch, case["v"]), dev(torch, case["alpha"]),
                                      dev(torch, case["beta"] if beta is None else beta), dev(torch, case["kq"]), out,
                                      case["capacity"], batch)
        torch.cuda.synchronize()
        return host(state), host(scales), host(out)
    finally:
        abi.configure(*before)


@pytest.mark.parametrize("batch,v_heads", [(32, 32), (1, 32), (5, 48)],
                         ids=["b32_h32_oracle_generalisation", "b1_h32_oracle_generalisation", "b5_h48_reference_shape"])
def test_delta_decode_int8_matches_oracle(cuda, ops, batch, v_heads):
    """Benchmark config 2 (32 slots, 32 value heads) and the reference's 48-head shape."""
    case = synth.delta_case(2, batch, v_heads)
    want_state, want_scales = case["state"].copy(), case["scales"].copy()
    want_out = oracle.delta_decode_int8(want_state, want_scales, case["slots"], case["q"], case["k"], case["v"],
                                        case["alpha"], case["beta"], case["kq"], batch, v_heads)
    state, scales, out = run_delta(cuda, ops, case, batch, v_heads)
    # out is read as bf16 downstream (cuda/delta_output.cu:38)
    assert_rms_close(oracle.bf16_round(out), oracle.bf16_round(want_out), "delta out")
    # reference: output within 2e-3 relative (crates/qwc-cuda/tests/delta_net.rs:113-135)
    assert np.max(np.abs(out - want_out)) <= 2e-3 * np.max(np.abs(want_out))
    # state: the fp32 summation order of u differs, so a code may move by one step on a few elements
    diff = np.abs(state.astype(np.int32) - want_state.astype(np.int32))
    assert diff.max() <= 1
    assert np.mean(diff > 0) < 0.02
    assert np.allclose(scales, want_scales, rtol=1e-5, atol=0)
    untouched = sorted(set(range(case["capacity"])) - set(case["slots"].tolist()))
    for slot in untouched:  # crates/qwc-cuda/tests/delta_net.rs:184-245
        assert np.array_equal(state[slot], case["state"][slot])
        assert np.array_equal(scales[slot], case["scales"][slot])


def test_delta_requantiser_is_bit_exact(cuda, ops):
    """beta = 0 makes every fp32 row value alpha * s exactly (tests/delta_net.rs:138-182), so the
    int8 codes and scales must equal the oracle's bit for bit."""
    batch, v_heads = 7, 32
    case = synth.delta_case(4, batch, v_heads, capacity=9)
    beta = np.zeros_like(case["beta"])
    want_state, want_scales = case["state"].copy(), case["scales"].copy()
    want_out = oracle.delta_decode_int8(want_state, want_scales, case["slots"], case["q"], case["k"], case["v"],
                                        case["alpha"], beta, case["kq"], batch, v_heads)
    state, scales, out = run_delta(cuda, ops, case, batch, v_heads, beta=beta)
    assert np.array_equal(state, want_state)
    assert np.array_equal(scales.view(np.uint32), want_scales.view(np.uint32))
    assert np.allclose(out, want_out, rtol=1e-4, atol=1e-6)


def test_delta_zero_rows_store_zero_scale(cuda, ops):
    batch, v_heads = 2, 32
    case = synth.delta_case(5, batch, v_heads, capacity=2)
    case["state"][:] = 0
    case["scales"][:] = 0
    case["v"][:] = 0
    state, scales, out = run_delta(cuda, ops, case, batch, v_heads)
    assert not state.any() and not scales.any() and not out.any()


def test_delta_slot_beyond_the_pool_is_skipped_and_reported(cuda, ops):
    """A row that names a state slot past the pool touches no memory: the kernel skips the row and
    the sticky status word tells the host (nothing faults; the access never happens)."""
    from qwencore_b200 import abi

    batch, v_heads = 3, 32
    case = synth.delta_case(6, batch, v_heads, capacity=4)
    slots = case["slots"].copy()
    bad_row = 1
    slots[bad_row] = 4  # capacity is 4: slots 0..3 exist
    case = dict(case, slots=slots)
    assert abi.lib.qwc_device_status() == 0
    try:
        state, scales, out = run_delta(cuda, ops, case, batch, v_heads)
        assert abi.lib.qwc_device_status() == 0x105
        # the pool is as it was wherever the rows in range did not write, and the bad row wrote nothing
        touched = {int(s) for i, s in enumerate(slots) if i != bad_row}
        for slot in range(case["capacity"]):
            if slot not in touched:
                assert np.array_equal(state[slot], case["state"][slot])
        assert not out[bad_row].any()
    finally:
        assert abi.lib.qwc_device_status_reset() == 0
    assert abi.lib.qwc_device_status() == 0


# ---------------------------------------------------------------------------------------
# Step glue
# ---------------------------------------------------------------------------------------

def test_rmsnorm_bf16_with_and_without_residual(cuda, ops):
    torch = cuda
    batch, hidden = 5, 5120
    x = synth.normal_bf16(6, "x", (batch, hidden))
    res = synth.normal_bf16(6, "res", (batch, hidden), std=3.0)
    w = synth.normal_bf16(6, "w", (hidden,), std=0.02)
    for with_residual in (False, True):
        res_want = res.copy()
        want = oracle.rmsnorm_bf16(x, res_want if with_residual else None, w, batch, hidden)
        res_dev = dev(torch, res)
        out = bf16_out(torch, batch, hidden)
        ops.rmsnorm_bf16(dev(torch, x), res_dev if with_residual else None, dev(torch, w), out, batch, hidden)
        torch.cuda.synchronize()
        if with_residual:  # the residual sum is one bf16 rounding: bit-exact
            assert np.array_equal(host(res_dev), res_want)
        got = synth.bf16_value(host(out))
        want_values = synth.bf16_value(want)
        assert np.max(np.abs(got - want_values)) <= 2.0 ** -7 * np.max(np.abs(want_values))
        assert_rms_close(got, want_values, "rmsnorm")


def test_fp8_embedding_gather_is_bit_exact(cuda, ops):
    torch = cuda
    vocab, cols = 1000, 512
    rows = synth.normal_bf16(7, "emb", (vocab, cols), std=0.02)
    table, scales = oracle.fp8_quantize_rows(rows, vocab, cols)
    tokens = np.array([0, 999, 17, 1000, 4000000000], dtype=np.uint32)  # last two are out of vocabulary
    want = oracle.fp8_embedding_gather(table, scales, tokens, cols, vocab)
    out = bf16_out(torch, tokens.size, cols)
    ops.fp8_embedding_gather(dev(torch, table), dev(torch, scales), dev(torch, tokens), out, tokens.size, cols, vocab)
    torch.cuda.synchronize()
    assert np.array_equal(host(out), want)
    assert not host(out)[3:].any()


# 5003: not a multiple of the row tile nor of the 16-byte store (the mma.sync kernel at every batch size);
# 5000: stores aligned, a ragged last tile (above eight rows the tcgen05 kernel); 12000: a table large
# enough that the tcgen05 kernel takes every batch size.
@pytest.mark.parametrize("batch,vocab", [(1, 5003), (8, 5003), (32, 5003), (8, 5000), (9, 5000), (16, 5000),
                                         (17, 5000), (32, 5000), (32, 4096), (1, 12000), (5, 12000)])
def test_fp8_lm_head_and_argmax(cuda, ops, batch, vocab):
    torch = cuda
    hidden = 5120
    rows = synth.normal_bf16(8, "head", (vocab, hidden), std=0.02)
    weights, scales = oracle.fp8_quantize_rows(rows, vocab, hidden)
    x = synth.normal_bf16(8, f"h{batch}", (batch, hidden))
    want = oracle.fp8_lm_head(weights, scales, x, batch, hidden, vocab)
    logits = torch.zeros((batch, vocab), dtype=torch.float32, device="cuda")
    ops.fp8_lm_head(dev(torch, weights), dev(torch, scales), dev(torch, x), logits, batch, hidden, vocab)
    parts = 64
    pv = torch.zeros(batch * parts, dtype=torch.float32, device="cuda")
    pi = u32_out(torch, batch * parts)
    tokens = u32_out(torch, batch)
    ops.argmax(logits, pv, pi, tokens, vocab, batch, parts)
    torch.cuda.synchronize()
    got = host(logits)
    assert_rms_close(got, want, "lm_head", bf16_grid=False)
    # argmax of the GPU logits is exact; against the oracle logits it agrees wherever the top-2 gap is clear
    assert np.array_equal(host(tokens), oracle.argmax(got, vocab, batch))
    ordered = np.sort(want, axis=1)
    clear = (ordered[:, -1] - ordered[:, -2]) > 4 * np.max(np.abs(got - want))
    assert np.array_equal(host(tokens)[clear], oracle.argmax(want, vocab, batch)[clear])


def test_argmax_ties_go_to_lower_index(cuda, ops):
    """crates/qwc-cuda/tests/sampling.rs:19-27"""
    torch = cuda
    vocab = 151936
    logits = np.full((7, vocab), -2.0, dtype=np.float32)
    logits[0, [150000, 77, 9000]] = 5.0
    logits[1, vocab - 1] = 1.0
    logits[2, :] = 0.25
    # what `value > best || (value == best && index < best_index)` does with the special values
    # (cuda/sampling.cu:11-14): a NaN never wins, -inf is an ordinary smallest value, -0 equals +0
    logits[3, :] = np.nan
    logits[4, :] = -np.inf
    logits[4, 5] = np.nan
    logits[5, :] = -np.inf
    logits[5, [70000, 120001]] = -3.0e38
    logits[6, :] = -1.0
    logits[6, 9] = 0.0
    logits[6, 4] = -0.0
    parts = 256
    pv = torch.zeros(7 * parts, dtype=torch.float32, device="cuda")
    pi = u32_out(torch, 7 * parts)
    tokens = u32_out(torch, 7)
    ops.argmax(dev(torch, logits), pv, pi, tokens, vocab, 7, parts)
    torch.cuda.synchronize()
    assert host(tokens).tolist() == [77, vocab - 1, 0, 0xFFFFFFFF, 0, 70000, 4]


@pytest.mark.parametrize("v_heads", [32, 48], ids=["h32_oracle_generalisation", "h48_reference_shape"])
def test_delta_prepare_and_gated_rmsnorm(cuda, ops, v_heads):
    """crates/qwc-cuda/tests/delta_net.rs:576-716 (CPU conv/gate check) and :716-777."""
    from qwencore_b200 import abi

    torch = cuda
    batch, capacity, k_heads, dim = 4, 6, 16, 128
    channels = 2 * k_heads * dim + v_heads * dim
    z_offset = channels
    a_offset = z_offset + v_heads * dim
    b_offset = a_offset + v_heads
    stride = b_offset + v_heads
    rng = synth.generator(9, f"prepare{v_heads}")
    mixed = synth.bf16_bits(rng.standard_normal((batch, stride), dtype=np.float32))
    conv_weight = synth.bf16_bits(rng.standard_normal((channels, 4), dtype=np.float32) * 0.5)
    a_log = synth.bf16_bits(rng.standard_normal(v_heads, dtype=np.float32) * 0.5)
    dt_bias = synth.bf16_bits(rng.standard_normal(v_heads, dtype=np.float32) * 0.5)
    conv_state = rng.standard_normal((capacity, channels, 3), dtype=np.float32)
    slots = rng.permutation(capacity)[:batch].astype(np.uint32)

    want_state = conv_state.copy()
    base = mixed.ctypes.data
    q, k, v, alpha, beta, kq = oracle.delta_prepare_decode(mixed, base + 2 * a_offset, base + 2 * b_offset, conv_weight,
                                                           a_log, dt_bias, want_state, slots, batch, stride, stride,
                                                           k_heads, v_heads)
    before = abi.get_shape()
    abi.configure(v_heads, before[1])
    try:
        d_mixed = dev(torch, mixed)
        d_state = dev(torch, conv_state)
        tq = torch.zeros((batch, k_heads, dim), dtype=torch.float32, device="cuda")
        tk = torch.zeros_like(tq)
        tv = torch.zeros((batch, v_heads, dim), dtype=torch.float32, device="cuda")
        ta = torch.zeros((batch, v_heads), dtype=torch.float32, device="cuda")
        tb = torch.zeros_like(ta)
        tkq = torch.zeros((batch, k_heads), dtype=torch.float32, device="cuda")
        ops.delta_prepare_decode(d_mixed, a_offset, b_offset, dev(torch, conv_weight), dev(torch, a_log),
                                 dev(torch, dt_bias), d_state, dev(torch, slots), tq, tk, tv, ta, tb, tkq, capacity,
                                 batch, stride)
        values = rng.standard_normal((batch, v_heads, dim), dtype=np.float32)
        weight = synth.bf16_bits(1.0 + 0.1 * rng.standard_normal(dim, dtype=np.float32))
        normed = bf16_out(torch, batch, v_heads, dim)
        ops.delta_gated_rmsnorm(dev(torch, values), d_mixed, z_offset, dev(torch, weight), normed, batch, stride)
        torch.cuda.synchronize()
    finally:
        abi.configure(*before)

    # history shift is a copy: bit-exact; untouched slots stay untouched
    assert np.array_equal(host(d_state), want_state)
    assert np.array_equal(host(tv), v)  # conv + SiLU snapped to bf16: allow no more than one bf16 step
    for got, want, name in [(tq, q, "q"), (tk, k, "k"), (ta, alpha, "alpha"), (tb, beta, "beta"), (tkq, kq, "kq")]:
        assert np.allclose(host(got), want, rtol=2e-3, atol=2e-6), name
    want_norm = oracle.delta_gated_rmsnorm(values, base + 2 * z_offset, weight, batch, v_heads, stride)
    got_norm = synth.bf16_value(host(normed))
    want_norm = synth.bf16_value(want_norm)
    assert np.max(np.abs(got_norm - want_norm)) <= 2.0 ** -6 * np.max(np.abs(want_norm))
    assert_rms_close(got_norm, want_norm, "gated rmsnorm", bound=2e-2)


@pytest.mark.parametrize("page_size,scaled", [(64, False), (16, True)],
                         ids=["page64_reference_shape", "page16_kv_scales_oracle_generalisation"])
def test_prepare_attention_writes_query_and_fp8_pages(cuda, ops, page_size, scaled):
    """crates/qwc-cuda/tests/attention_prepare.rs:9-33"""
    torch = cuda
    batch, num_blocks = 3, 7
    rng = synth.generator(10, f"attnprep{page_size}")
    query_gate = synth.bf16_bits(rng.standard_normal((batch, 24 * 512), dtype=np.float32))
    key_proj = synth.bf16_bits(rng.standard_normal((batch, 4 * 256), dtype=np.float32))
    value_proj = synth.bf16_bits(rng.standard_normal((batch, 4 * 256), dtype=np.float32))
    qw = synth.bf16_bits(rng.standard_normal(256, dtype=np.float32) * 0.1)
    kw = synth.bf16_bits(rng.standard_normal(256, dtype=np.float32) * 0.1)
    positions = np.array([0, 5 * page_size + 3, 2 * page_size + page_size - 1], dtype=np.uint32)
    cosine, sine = oracle.rope_rows(positions)
    physical = np.array([6, 2, 4], dtype=np.uint32)
    offsets = (positions % page_size).astype(np.uint32)
    k_scale = v_scale = None
    if scaled:
        k_scale = np.array([0.02, 0.03, 0.015, 0.025], dtype=np.float32)
        v_scale = np.array([0.01, 0.02, 0.03, 0.04], dtype=np.float32)
    key_cache = np.zeros((num_blocks, 4, page_size, 256), dtype=np.uint8)
    value_cache = np.zeros_like(key_cache)
    want_k, want_v = key_cache.copy(), value_cache.copy()
    want_q = oracle.prepare_attention_decode_fp8(query_gate, key_proj, value_proj, qw, kw, cosine, sine, physical,
                                                 offsets, want_k, want_v, batch, page_size, k_scale=k_scale,
                                                 v_scale=v_scale)
    d_k, d_v = dev(torch, key_cache), dev(torch, value_cache)
    query = bf16_out(torch, batch, 24, 256)
    ops.prepare_attention_decode(dev(torch, query_gate), dev(torch, key_proj), dev(torch, value_proj), dev(torch, qw),
                                 dev(torch, kw), dev(torch, cosine), dev(torch, sine), dev(torch, physical),
                                 dev(torch, offsets), query, d_k, d_v, batch, page_size, 24 * 512, 4 * 256, 4 * 256,
                                 None if k_scale is None else dev(torch, k_scale),
                                 None if v_scale is None else dev(torch, v_scale))
    torch.cuda.synchronize()
    got_q = synth.bf16_value(host(query))
    assert np.max(np.abs(got_q - synth.bf16_value(want_q))) <= 2.0 ** -6 * np.max(np.abs(got_q))
    got_k, got_v = host(d_k), host(d_v)
    # V is a pure bf16 -> e4m3 conversion: bit-exact without scales (with scales the reciprocal may differ by an ulp)
    if not scaled:
        assert np.array_equal(got_v, want_v)
    for got, want in ((got_k, want_k), (got_v, want_v)):
        written = want != 0
        assert np.array_equal(got != 0, written) or np.mean((got != 0) != written) < 1e-3
        steps = np.abs(got.astype(np.int32) - want.astype(np.int32))
        assert steps.max() <= 1 and np.mean(steps > 0) < 0.02  # rsqrt vs 1/sqrt may move a code by one


# ---------------------------------------------------------------------------------------
# Device-side batch packing (bit-exact)
# ---------------------------------------------------------------------------------------

def packing_case(seed, capacity, max_blocks, page_size, live):
    rng = synth.generator(seed, "packing")
    seq_tokens = np.zeros(capacity, dtype=np.uint32)
    seq_blocks = np.zeros((capacity, max_blocks), dtype=np.uint32)
    counts = np.zeros(capacity, dtype=np.uint32)
    pool = rng.permutation(capacity * max_blocks).astype(np.uint32)
    cursor = 0
    slots = rng.permutation(capacity)[:live]
    for slot in slots:
        tokens = int(rng.integers(1, max_blocks * page_size + 1))
        blocks = (tokens + page_size - 1) // page_size
        seq_tokens[slot] = tokens
        counts[slot] = blocks
        seq_blocks[slot, :blocks] = pool[cursor:cursor + blocks]
        cursor += blocks
    return seq_tokens, seq_blocks, counts, slots.astype(np.uint32)


def run_packing(torch, ops, row_slots, slot_active, seq_tokens, seq_blocks, rows, max_blocks, page_size, max_positions):
    capacity = seq_tokens.size
    positions = np.arange(max_positions, dtype=np.uint32)
    cos, sin = oracle.rope_rows(positions)
    rope_table = np.stack([cos, sin], axis=1)  # [position, 2, 64]
    u32 = lambda *shape: u32_out(torch, *shape)
    out = {
        "row_count": u32(1), "state_slots": u32(rows), "positions": u32(rows), "context_lengths": u32(rows),
        "physical_blocks": u32(rows), "block_offsets": u32(rows),
        "block_tables": u32_out(torch, rows, max_blocks, fill=7),
        "block_table_offsets": u32(rows + 1), "block_ids": u32(rows * max_blocks),
        "cosine": bf16_out(torch, rows, 64), "sine": bf16_out(torch, rows, 64), "status": u32(1),
    }
    ops.pack_decode_batch(None if row_slots is None else dev(torch, row_slots),
                          None if slot_active is None else dev(torch, slot_active), dev(torch, seq_tokens),
                          dev(torch, seq_blocks), dev(torch, rope_table), max_positions, out["row_count"],
                          out["state_slots"], out["positions"], out["context_lengths"], out["physical_blocks"],
                          out["block_offsets"], out["block_tables"], out["block_table_offsets"], out["block_ids"],
                          out["cosine"], out["sine"], out["status"], rows, capacity, max_blocks, page_size)
    torch.cuda.synchronize()
    return {k: host(v) for k, v in out.items()}, (cos, sin)


@pytest.mark.parametrize("page_size,capacity,live,max_blocks", [(16, 33, 32, 128), (64, 300, 257, 9), (16, 8, 1, 4)])
def test_pack_decode_batch_matches_host_layout_bit_for_bit(cuda, ops, page_size, capacity, live, max_blocks):
    seq_tokens, seq_blocks, counts, slots = packing_case(20, capacity, max_blocks, page_size, live)
    want = oracle.layout_decode(slots, seq_tokens, seq_blocks, counts, max_blocks, page_size)
    assert want["status"] == 0
    got, (cos, sin) = run_packing(cuda, ops, slots, None, seq_tokens, seq_blocks, live, max_blocks, page_size,
                                  max_blocks * page_size)
    assert got["status"][0] == 0 and got["row_count"][0] == live
    for key in ("state_slots", "positions", "context_lengths", "physical_blocks", "block_offsets", "block_tables",
                "block_table_offsets"):
        assert np.array_equal(got[key], want[key]), key
    total = int(want["block_table_offsets"][-1])
    assert np.array_equal(got["block_ids"][:total], want["block_ids"])
    want_cos, want_sin = oracle.rope_rows(want["positions"])
    assert np.array_equal(got["cosine"], want_cos) and np.array_equal(got["sine"], want_sin)


def test_pack_decode_batch_compacts_active_slots(cuda, ops):
    capacity, max_blocks, page_size = 700, 6, 16
    seq_tokens, seq_blocks, counts, slots = packing_case(21, capacity, max_blocks, page_size, 400)
    active = np.zeros(capacity, dtype=np.uint8)
    chosen = np.sort(slots[:333])
    active[chosen] = 1
    rows = 512  # capacity-level launch shape; the live prefix is reported on the device
    want = oracle.layout_decode(chosen, seq_tokens, seq_blocks, counts, max_blocks, page_size)
    got, _ = run_packing(cuda, ops, None, active, seq_tokens, seq_blocks, rows, max_blocks, page_size,
                         max_blocks * page_size)
    assert got["status"][0] == 0 and got["row_count"][0] == 333
    for key in ("state_slots", "positions", "context_lengths", "physical_blocks", "block_offsets"):
        assert np.array_equal(got[key][:333], want[key]), key
        assert not got[key][333:].any(), key
    assert np.array_equal(got["block_tables"][:333], want["block_tables"])
    assert not got["block_tables"][333:].any()
    assert np.array_equal(got["block_table_offsets"][:334], want["block_table_offsets"])
    assert np.all(got["block_table_offsets"][334:] == want["block_table_offsets"][-1])


def test_pack_decode_batch_reports_errors(cuda, ops):
    capacity, max_blocks, page_size = 10, 4, 16
    seq_tokens, seq_blocks, counts, slots = packing_case(22, capacity, max_blocks, page_size, 6)
    empty = [s for s in range(capacity) if seq_tokens[s] == 0][0]
    duplicate = np.array([slots[0], slots[1], slots[0]], dtype=np.uint32)
    for rows_in, code in [(np.array([slots[0], empty], dtype=np.uint32), 1), (duplicate, 2),
                          (np.array([99], dtype=np.uint32), 1)]:
        got, _ = run_packing(cuda, ops, rows_in, None, seq_tokens, seq_blocks, rows_in.size, max_blocks, page_size, 64)
        assert got["status"][0] == code
    too_long = seq_tokens.copy()
    too_long[slots[0]] = max_blocks * page_size + 1
    got, _ = run_packing(cuda, ops, slots[:1], None, too_long, seq_blocks, 1, max_blocks, page_size, 1000)
    assert got["status"][0] == 4


def test_page_table_apply_edits(cuda, ops):
    from qwencore_b200 import abi

    torch = cuda
    capacity, max_blocks = 5, 4
    seq_tokens = u32_out(torch, capacity)
    seq_blocks = u32_out(torch, capacity, max_blocks)
    edits = np.array([(2, 0, 9, 0), (2, 1, 4, 0), (2, 0, 17, 1), (3, 0, 5, 1), (3, 0, 1, 2), (7, 0, 1, 1)],
                     dtype=np.uint32)  # the last names a slot out of range and is ignored
    ops.page_table_apply(seq_tokens, seq_blocks, dev(torch, edits), len(edits), capacity, max_blocks)
    torch.cuda.synchronize()
    assert host(seq_tokens).tolist() == [0, 0, 17, 6, 0]
    assert host(seq_blocks)[2].tolist() == [9, 4, 0, 0]
    assert abi.lib.qwc_page_table_apply(0, 0, 0, 1, capacity, max_blocks, 0) == abi.CUDA_ERROR_INVALID_VALUE
