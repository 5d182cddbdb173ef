"""Pins the CPU oracle to the reference's own known-answer tests (no GPU).

Every expected value below is a literal the reference asserts in its unit tests; the
citation gives the reference file and line.  An oracle that drifts from these is not an
oracle of this path.
"""

import numpy as np
import pytest

from oracle import oracle
from qwencore_b200 import synth


def test_e2m1_table_matches_reference_spot_values():
    # crates/qwc-cuda/src/nvfp4.rs:698-704
    lib = oracle.lib()
    assert lib.qo_e2m1(0x0) == 0.0
    assert lib.qo_e2m1(0x1) == 0.5
    assert lib.qo_e2m1(0x7) == 6.0
    assert lib.qo_e2m1(0xF) == -6.0
    # crates/qwc-cuda/src/nvfp4.rs:574-576, the whole table
    expected = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    assert [lib.qo_e2m1(i) for i in range(16)] == expected


def test_e4m3_boundaries_match_reference():
    # crates/qwc-cuda/src/nvfp4.rs:706-714
    lib = oracle.lib()
    assert lib.qo_e4m3(0x00) == 0.0
    assert lib.qo_e4m3(0x01) == 2.0 ** -9
    assert lib.qo_e4m3(0x38) == 1.0
    assert lib.qo_e4m3(0x7E) == 448.0
    assert lib.qo_e4m3(0xB8) == -1.0
    assert np.isnan(lib.qo_e4m3(0x7F))
    # scale codes of the GEMV test, crates/qwc-cuda/tests/nvfp4.rs:30-31: 0.5, 1.0, 1.5, 2.0
    assert [lib.qo_e4m3(c) for c in (0x30, 0x38, 0x3C, 0x40)] == [0.5, 1.0, 1.5, 2.0]


def test_e4m3_encode_round_trips_every_code_and_saturates():
    lib = oracle.lib()
    for code in range(256):
        if code & 0x7F == 0x7F:
            continue
        value = lib.qo_e4m3(code)
        if value == 0.0 and code == 0x80:
            assert lib.qo_e4m3_encode(value) == 0x80
            continue
        assert lib.qo_e4m3_encode(value) == code, hex(code)
    assert lib.qo_e4m3_encode(1.0e9) == 0x7E
    assert lib.qo_e4m3_encode(-1.0e9) == 0xFE
    assert lib.qo_e4m3_encode(float("inf")) == 0x7E
    assert lib.qo_e4m3_encode(float("nan")) == 0x7F
    # ties go to the even mantissa: 1.0625 is halfway between 1.0 (0x38) and 1.125 (0x39)
    assert lib.qo_e4m3_encode(1.0625) == 0x38
    assert lib.qo_e4m3_encode(1.1875) == 0x3A
    # halfway between the largest subnormal 7 * 2^-9 and the first normal 2^-6
    assert lib.qo_e4m3_encode(7.5 * 2.0 ** -9) == 0x08


def test_vectorised_encoders_agree_with_the_scalar_one():
    rng = np.random.default_rng(1)
    values = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * 3.0,
        rng.standard_normal(2000).astype(np.float32) * 300.0,
        rng.standard_normal(2000).astype(np.float32) * 0.01,
        np.array([0.0, -0.0, 448.0, 449.0, 1e-9, 2.0 ** -10, 3 * 2.0 ** -10], dtype=np.float32),
    ])
    scalar = oracle.e4m3_encode(values)
    assert np.array_equal(oracle.e4m3_encode_fast(values), scalar)
    assert np.array_equal(synth.e4m3_encode(values), scalar)
    assert np.array_equal(synth.e4m3_decode(np.arange(256, dtype=np.uint8))[:0x7F], oracle.e4m3_table()[:0x7F])


def test_bf16_rounding_matches_reference_rule():
    # crates/qwc-cuda/src/bf16.rs:5-12: RNE on the upper 16 bits, NaN -> 0x7fc0
    lib = oracle.lib()
    assert lib.qo_bf16_from_f32(1.0) == 0x3F80
    assert lib.qo_bf16_from_f32(float("nan")) == 0x7FC0
    one_plus_half_ulp = np.array([0x3F808000], dtype=np.uint32).view(np.float32)[0]
    assert lib.qo_bf16_from_f32(float(one_plus_half_ulp)) == 0x3F80      # tie -> even
    three_halves_ulp = np.array([0x3F818000], dtype=np.uint32).view(np.float32)[0]
    assert lib.qo_bf16_from_f32(float(three_halves_ulp)) == 0x3F82       # tie -> even (up)
    rng = np.random.default_rng(0)
    x = rng.standard_normal(1000).astype(np.float32)
    assert np.array_equal(oracle.bf16_from_f32(x), np.array([lib.qo_bf16_from_f32(float(v)) for v in x], np.uint16))
    assert np.array_equal(synth.bf16_bits(x), oracle.bf16_from_f32(x))


def test_swizzle_matches_reference_probe_points():
    # crates/qwc-cuda/src/nvfp4.rs:716-736
    rows, k = 129, 256
    groups = k // 16
    source = (np.arange(rows * groups) % 256).astype(np.uint8)
    got = oracle.swizzle_block_scales(source, rows, k)
    assert got.size == 256 * groups

    def index(row, group):
        rb, rq, ri = row // 128, row % 128 // 32, row % 32
        gb, gi = group // 4, group % 4
        return ((((rb * (groups // 4) + gb) * 32 + ri) * 4 + rq) * 4) + gi

    for row, group in [(0, 0), (31, 3), (32, 4), (127, 15), (128, 7)]:
        assert got[index(row, group)] == source[row * groups + group]
        assert oracle.lib().qo_block_scale_offset(row, group, k) == index(row, group)
    assert np.array_equal(oracle.unswizzle_block_scales(got, rows, k), source)
    assert np.array_equal(synth.swizzle_block_scales(source, rows, k), got)
    # the device kernel's form of the same index, crates/qwc-cuda/cuda/nvfp4.cu:33-39
    for row, group in [(5, 9), (77, 2), (128 + 45, 13)]:
        tile = (row >> 7) * (groups // 4) + (group >> 2)
        row_bits = ((row & 31) << 4) | (((row >> 5) & 3) << 2)
        assert oracle.lib().qo_block_scale_offset(row, group, k) == (tile << 9) | row_bits | (group & 3)


def test_gemv_oracle_on_a_hand_computed_case():
    # One row, K = 256: nibble 0x2 (1.0) everywhere, scale 0.5 (0x30), global 8 -> each weight 0.0625.
    k = 256
    packed = np.full((1, k // 2), 0x22, dtype=np.uint8)
    scales = np.full((1, k // 16), 0x30, dtype=np.uint8)
    x = synth.bf16_bits(np.ones((1, k), dtype=np.float32))
    out = oracle.gemv_w4a16(packed, scales, 8.0, x, 1, k, 1)
    assert out[0, 0] == 256 * 0.0625
    # low nibble is the even k (crates/qwc-cuda/src/nvfp4.rs:626-627)
    packed[:] = 0x02  # even k -> 1.0, odd k -> 0.0
    x_alt = np.zeros((1, k), dtype=np.float32)
    x_alt[0, 0::2] = 1.0
    out = oracle.gemv_w4a16(packed, scales, 8.0, synth.bf16_bits(x_alt), 1, k, 1)
    assert out[0, 0] == 128 * 0.0625


def test_layout_oracle_reproduces_reference_csr_example():
    # crates/qwc-runtime/src/layout.rs:164-189, decode row of the mixed batch:
    # sequence 1 in slot 0 holds 65 tokens (64 admitted + 1 appended) in pages [0, 1], page size 64.
    seq_tokens = np.array([65, 100], dtype=np.uint32)
    seq_blocks = np.array([[0, 1, 0], [2, 3, 0]], dtype=np.uint32)
    counts = np.array([2, 2], dtype=np.uint32)
    layout = oracle.layout_decode([0], seq_tokens, seq_blocks, counts, max_blocks=3, page_size=64)
    assert layout["status"] == 0
    assert layout["state_slots"].tolist() == [0]
    assert layout["positions"].tolist() == [64]
    assert layout["context_lengths"].tolist() == [65]
    assert layout["block_table_offsets"].tolist() == [0, 2]
    assert layout["block_ids"].tolist() == [0, 1]
    # upload_layout_decode, crates/qwc-engine/src/executor.rs:1968-1975
    assert layout["physical_blocks"].tolist() == [1]
    assert layout["block_offsets"].tolist() == [0]
    assert layout["block_tables"].tolist() == [[0, 1, 0]]


def test_layout_oracle_rejects_duplicate_and_missing_rows():
    # crates/qwc-runtime/src/layout.rs:191-222
    seq_tokens = np.array([2, 0], dtype=np.uint32)
    seq_blocks = np.array([[0, 0], [0, 0]], dtype=np.uint32)
    counts = np.array([1, 0], dtype=np.uint32)
    assert oracle.layout_decode([0, 0], seq_tokens, seq_blocks, counts, 2, 64)["status"] == -2
    assert oracle.layout_decode([1], seq_tokens, seq_blocks, counts, 2, 64)["status"] == -1
    assert oracle.layout_decode([7], seq_tokens, seq_blocks, counts, 2, 64)["status"] == -1
    seq_tokens = np.array([130, 0], dtype=np.uint32)
    assert oracle.layout_decode([0], seq_tokens, seq_blocks, counts, 4, 64)["status"] == -4


def test_int8_grid_matches_reference_host_statement():
    # crates/qwc-cuda/tests/delta_net.rs:1146-1184: per-row scale 2^((row % 7) - 3); expected level is
    # round_ties_even(x / step) with step = peak / 127, compared to 1e-6 * peak.
    rng = np.random.default_rng(0x51ED)
    rows = np.zeros((64, 128), dtype=np.float32)
    for r in range(64):
        rows[r] = oracle.bf16_round((rng.random(128, dtype=np.float32) * 2 - 1) * np.float32(2.0 ** ((r % 7) - 3)))
    codes, scales = oracle.delta_quantize_rows(rows)
    for r in range(64):
        peak = np.max(np.abs(rows[r]))
        step = np.float32(peak * np.float32(1.0 / 127.0))
        assert scales[r] == step
        level = np.clip(np.rint(rows[r] * (np.float32(1.0) / step)), -127, 127)
        recon = codes[r].astype(np.float32) * scales[r]
        assert np.all(np.abs(recon - level * step) <= 1e-6 * max(peak, 1e-6))
        assert np.max(np.abs(recon - rows[r])) <= 0.5 * step * 1.01
    zero_codes, zero_scales = oracle.delta_quantize_rows(np.zeros((1, 128), dtype=np.float32))
    assert not zero_codes.any() and zero_scales[0] == 0.0
    mine_codes, mine_scales = synth.quantize_state_rows(rows)
    assert np.array_equal(mine_codes, codes) and np.array_equal(mine_scales, scales)


def test_delta_oracle_beta_zero_decays_state_exactly():
    # crates/qwc-cuda/tests/delta_net.rs:138-182: beta = 0 -> S <- alpha S and nothing else.
    case = synth.delta_case(3, batch=2, v_heads=32, capacity=3)
    state, scales = case["state"].copy(), case["scales"].copy()
    beta = np.zeros_like(case["beta"])
    oracle.delta_decode_int8(state, scales, case["slots"], case["q"], case["k"], case["v"], case["alpha"], beta,
                             case["kq"], batch=2, v_heads=32)
    for b, slot in enumerate(case["slots"]):
        for h in range(0, 32, 5):
            before = case["state"][slot, h].astype(np.float32) * case["scales"][slot, h][:, None]
            decayed = (np.float32(case["alpha"][b, h]) * before).astype(np.float32)
            want_codes, want_scales = oracle.delta_quantize_rows(decayed)
            assert np.array_equal(state[slot, h], want_codes)
            assert np.array_equal(scales[slot, h], want_scales)
    untouched = [s for s in range(3) if s not in set(case["slots"].tolist())]
    for slot in untouched:  # slots not named stay untouched (tests/delta_net.rs:184-245)
        assert np.array_equal(state[slot], case["state"][slot])


def test_attention_oracle_uniform_scores_average_the_values():
    # All-zero queries give uniform softmax weights: the output is the mean of V over the context.
    case = synth.attention_case(5, [23, 257], page_size=64)
    query = np.zeros_like(case["query"])
    out = oracle.paged_attention_fp8(query, None, case["key_cache"], case["value_cache"], case["block_tables"],
                                     case["contexts"], case["max_blocks"], batch=2, page_size=64)
    values = synth.e4m3_decode(case["value_cache"])
    for b, context in enumerate(case["contexts"]):
        rows = []
        for token in range(int(context)):
            page = case["block_tables"][b, token // 64]
            rows.append(values[page, 0, token % 64])
        want = np.mean(np.stack(rows), axis=0)
        assert np.allclose(out[b, 0], want, atol=2e-5)


def test_argmax_ties_go_to_the_lower_index():
    # crates/qwc-cuda/tests/sampling.rs:19-27 and cuda/sampling.cu:11-14
    logits = np.full((2, 1000), -1.0, dtype=np.float32)
    logits[0, [7, 500]] = 3.0
    logits[1, 999] = 2.0
    assert oracle.argmax(logits, 1000, 2).tolist() == [7, 999]


def test_rmsnorm_oracle_adds_residual_before_statistics():
    # crates/qwc-cuda/src/rmsnorm.rs:117-131: residual <- bf16(in + res), stats on the rounded value
    hidden = 256
    x = synth.normal_bf16(1, "x", (1, hidden))
    res = synth.normal_bf16(1, "r", (1, hidden))
    w = synth.normal_bf16(1, "w", (hidden,), std=0.02)
    res_in = res.copy()
    out = oracle.rmsnorm_bf16(x, res, w, 1, hidden)
    summed = oracle.bf16_round(oracle.bf16_to_f32(x) + oracle.bf16_to_f32(res_in))
    assert np.array_equal(res, oracle.bf16_from_f32(summed))
    inverse = 1.0 / np.sqrt(np.mean(summed.astype(np.float64) ** 2) + 1e-6)
    want = summed[0] * inverse * (1.0 + oracle.bf16_to_f32(w))
    assert np.allclose(oracle.bf16_to_f32(out[0]), want, rtol=1e-2, atol=1e-3)
