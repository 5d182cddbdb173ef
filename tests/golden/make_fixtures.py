"""Writes tests/golden/decode_step_vectors.npz: outputs of the CPU oracle on small seeded cases.

    python tests/golden/make_fixtures.py

The reference's own host code is Rust and cannot run here, so its known-answer tests are restated
value by value in tests/test_oracle_golden.py; this file adds regression vectors for the composite
ops on inputs that the tests regenerate from the same seeds (only expected outputs and a digest of
each input are stored).  The CUDA kernels are compared against the stored outputs by
tests/test_golden_fixtures.py (GPU part); the oracle must reproduce them bit for bit (CPU part)."""

import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import oracle  # noqa: E402
from qwencore_b200 import synth  # noqa: E402

GEMV_SHAPE = (96, 512)          # out_features, in_features
GEMV_BATCHES = (1, 7, 32)
ATTENTION_CONTEXTS = (23, 257, 64)
ATTENTION_PAGE = 16
DELTA_BATCH, DELTA_HEADS = 2, 32


def digest(*arrays) -> np.ndarray:
    h = hashlib.sha256()
    for array in arrays:
        h.update(np.ascontiguousarray(array).tobytes())
    return np.frombuffer(h.digest(), dtype=np.uint8).copy()


def gemv_inputs(batch):
    out_features, in_features = GEMV_SHAPE
    packed, scales, swizzled = synth.nvfp4_matrix(3, "golden", out_features, in_features)
    x = synth.normal_bf16(3, f"golden_x{batch}", (batch, in_features))
    return packed, scales, swizzled, x


def attention_inputs():
    return synth.attention_case(5, list(ATTENTION_CONTEXTS), page_size=ATTENTION_PAGE, with_gate=True, scaled=True)


def delta_inputs():
    return synth.delta_case(7, DELTA_BATCH, DELTA_HEADS)


def build() -> dict:
    vectors = {}
    for batch in GEMV_BATCHES:
        packed, scales, _, x = gemv_inputs(batch)
        vectors[f"gemv_b{batch}_inputs_sha256"] = digest(packed, scales, x)
        vectors[f"gemv_b{batch}_out"] = oracle.gemv_w4a16(packed, scales, 2.0, x, *GEMV_SHAPE, batch)
    case = attention_inputs()
    vectors["attention_inputs_sha256"] = digest(case["query"], case["gate_projection"], case["key_cache"], case["value_cache"],
                                                case["block_tables"], case["contexts"])
    vectors["attention_out"] = oracle.paged_attention_fp8(
        case["query"], case["gate_projection"], case["key_cache"], case["value_cache"], case["block_tables"], case["contexts"],
        case["max_blocks"], batch=len(ATTENTION_CONTEXTS), page_size=ATTENTION_PAGE, k_scale=case["k_scale"],
        v_scale=case["v_scale"])
    case = delta_inputs()
    vectors["delta_inputs_sha256"] = digest(case["state"], case["scales"], case["slots"], case["q"], case["k"],
                                            case["v"], case["alpha"], case["beta"], case["kq"])
    state, scales = case["state"].copy(), case["scales"].copy()
    vectors["delta_out"] = oracle.delta_decode_int8(state, scales, case["slots"], case["q"], case["k"], case["v"],
                                                    case["alpha"], case["beta"], case["kq"], DELTA_BATCH, DELTA_HEADS)
    vectors["delta_state_sha256"] = digest(state)
    vectors["delta_scales"] = scales[case["slots"]]
    return vectors


if __name__ == "__main__":
    target = Path(__file__).resolve().parent / "decode_step_vectors.npz"
    np.savez_compressed(target, **build())
    print(target, target.stat().st_size, "bytes")
