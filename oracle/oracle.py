"""numpy front-end of the CPU oracle (oracle/qwc_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this module;
the shipped package never does.  `build()` compiles the C file on first use.
"""

from __future__ import annotations

import ctypes
import subprocess
from ctypes import c_float, c_int, c_size_t, c_void_p
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent
LIBRARY = ORACLE_DIR / "_build" / "liboracle.so"
REFERENCE_KERNELS = ORACLE_DIR / "_ref" / "libqwc_ref_kernels.so"


def build() -> Path:
    """Compile the checker (and, where the reference tree is mounted, its kernels)."""
    source = ORACLE_DIR / "qwc_oracle.c"
    if not LIBRARY.exists() or LIBRARY.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE_DIR), "_build/liboracle.so"], check=True,
                       capture_output=True)
    return LIBRARY


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.qo_bf16_from_f32.restype = ctypes.c_uint16
        _lib.qo_bf16_from_f32.argtypes = [c_float]
        _lib.qo_bf16_to_f32.restype = c_float
        _lib.qo_bf16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.qo_e2m1.restype = c_float
        _lib.qo_e2m1.argtypes = [ctypes.c_uint8]
        _lib.qo_e4m3.restype = c_float
        _lib.qo_e4m3.argtypes = [ctypes.c_uint8]
        _lib.qo_e4m3_encode.restype = ctypes.c_uint8
        _lib.qo_e4m3_encode.argtypes = [c_float]
        _lib.qo_block_scale_storage_len.restype = c_size_t
        _lib.qo_block_scale_storage_len.argtypes = [c_int, c_int]
        _lib.qo_block_scale_offset.restype = c_size_t
        _lib.qo_block_scale_offset.argtypes = [c_int, c_int, c_int]
        _lib.qo_delta_quantize_row.restype = c_float
        _lib.qo_layout_decode.restype = c_int
        _lib.qo_num_threads.restype = c_int
    return _lib


def _ptr(array):
    if array is None:
        return c_void_p(None)
    assert array.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return array.ctypes.data_as(c_void_p)


# ---- number formats ---------------------------------------------------------------

def bf16_from_f32(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 bits (crates/qwc-cuda/src/bf16.rs:5-12), vectorised."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    out = ((bits + 0x7FFF + lsb) >> 16).astype(np.uint16)
    out[np.isnan(x)] = 0x7FC0
    return out


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    return bf16_to_f32(bf16_from_f32(x))


def e4m3_table() -> np.ndarray:
    return np.array([lib().qo_e4m3(i) for i in range(256)], dtype=np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    flat = np.ascontiguousarray(x, dtype=np.float32).ravel()
    encode = lib().qo_e4m3_encode
    return np.array([encode(float(v)) for v in flat], dtype=np.uint8).reshape(np.shape(x))


def e4m3_encode_fast(x: np.ndarray) -> np.ndarray:
    """Vectorised encoder for large arrays: nearest table value, ties to the even code.

    Checked against the scalar encoder in tests/test_oracle_golden.py.
    """
    table = e4m3_table()
    positive = table[:0x7F].astype(np.float64)  # 0 .. 448, strictly increasing
    x = np.ascontiguousarray(x, dtype=np.float32)
    magnitude = np.minimum(np.abs(x).astype(np.float64), 448.0)
    upper = np.clip(np.searchsorted(positive, magnitude, side="left"), 0, 0x7E)
    lower = np.clip(upper - 1, 0, 0x7E)
    d_up = positive[upper] - magnitude
    d_lo = magnitude - positive[lower]
    pick_lower = (d_lo < d_up) | ((d_lo == d_up) & (lower % 2 == 0))
    code = np.where(pick_lower, lower, upper).astype(np.uint8)
    code[np.isnan(x)] = 0x7F
    return (code | (np.signbit(x).astype(np.uint8) << 7)).astype(np.uint8)


# ---- NVFP4 -------------------------------------------------------------------------

def block_scale_storage_len(rows: int, in_features: int) -> int:
    return int(lib().qo_block_scale_storage_len(rows, in_features))


def swizzle_block_scales(scales: np.ndarray, rows: int, in_features: int) -> np.ndarray:
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    out = np.zeros(block_scale_storage_len(rows, in_features), dtype=np.uint8)
    lib().qo_swizzle_block_scales(_ptr(scales), _ptr(out), c_int(rows), c_int(in_features))
    return out


def unswizzle_block_scales(swizzled: np.ndarray, rows: int, in_features: int) -> np.ndarray:
    out = np.zeros(rows * in_features // 16, dtype=np.uint8)
    lib().qo_unswizzle_block_scales(_ptr(np.ascontiguousarray(swizzled)), _ptr(out), c_int(rows),
                                    c_int(in_features))
    return out


def gemv_w4a16(packed, scales, global_scale, x_bits, out_features, in_features, batch) -> np.ndarray:
    out = np.zeros((batch, out_features), dtype=np.float32)
    lib().qo_gemv_w4a16(_ptr(np.ascontiguousarray(packed, dtype=np.uint8)),
                        _ptr(np.ascontiguousarray(scales, dtype=np.uint8)), c_float(global_scale),
                        _ptr(np.ascontiguousarray(x_bits, dtype=np.uint16)), _ptr(out), c_int(out_features),
                        c_int(in_features), c_int(batch))
    return out


def swiglu_combine(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    up = np.ascontiguousarray(up, dtype=np.float32)
    out = np.zeros_like(gate)
    lib().qo_swiglu_combine(_ptr(gate), _ptr(up), _ptr(out), c_size_t(gate.size))
    return out


# ---- attention ---------------------------------------------------------------------

def paged_attention_fp8(query_bits, gate_projection_bits, key_cache, value_cache, block_tables,
                        context_lengths, max_blocks, batch, q_heads=24, kv_heads=4, head_dim=256,
                        page_size=64, k_scale=None, v_scale=None, softmax_scale=1.0 / 16.0) -> np.ndarray:
    out = np.zeros((batch, q_heads, head_dim), dtype=np.float32)
    gate = None if gate_projection_bits is None else np.ascontiguousarray(gate_projection_bits, dtype=np.uint16)
    ks = None if k_scale is None else np.ascontiguousarray(k_scale, dtype=np.float32)
    vs = None if v_scale is None else np.ascontiguousarray(v_scale, dtype=np.float32)
    lib().qo_paged_attention_fp8(
        _ptr(np.ascontiguousarray(query_bits, dtype=np.uint16)), _ptr(gate),
        _ptr(np.ascontiguousarray(key_cache, dtype=np.uint8)), _ptr(np.ascontiguousarray(value_cache, dtype=np.uint8)),
        _ptr(np.ascontiguousarray(block_tables, dtype=np.uint32)),
        _ptr(np.ascontiguousarray(context_lengths, dtype=np.uint32)), c_int(max_blocks), _ptr(out), c_int(batch),
        c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(page_size), _ptr(ks), _ptr(vs),
        c_float(softmax_scale))
    return out


# ---- DeltaNet ----------------------------------------------------------------------

def delta_quantize_rows(rows: np.ndarray):
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    flat = rows.reshape(-1, rows.shape[-1])
    codes = np.zeros(flat.shape, dtype=np.int8)
    scales = np.zeros(flat.shape[0], dtype=np.float32)
    quantize = lib().qo_delta_quantize_row
    for i in range(flat.shape[0]):
        scales[i] = quantize(_ptr(flat[i]), _ptr(codes[i]), c_int(flat.shape[1]))
    return codes.reshape(rows.shape), scales.reshape(rows.shape[:-1])


def delta_decode_int8(state, state_scales, state_slots, q, k, v, alpha, beta, kq, batch, v_heads, k_heads=16,
                      dv=128, dk=128) -> np.ndarray:
    """Updates `state` / `state_scales` in place and returns out f32[batch, v_heads, dv]."""
    assert state.dtype == np.int8 and state_scales.dtype == np.float32
    out = np.zeros((batch, v_heads, dv), dtype=np.float32)
    slots = None if state_slots is None else np.ascontiguousarray(state_slots, dtype=np.uint32)
    lib().qo_delta_decode_int8(_ptr(state), _ptr(state_scales), _ptr(slots),
                               _ptr(np.ascontiguousarray(q, dtype=np.float32)),
                               _ptr(np.ascontiguousarray(k, dtype=np.float32)),
                               _ptr(np.ascontiguousarray(v, dtype=np.float32)),
                               _ptr(np.ascontiguousarray(alpha, dtype=np.float32)),
                               _ptr(np.ascontiguousarray(beta, dtype=np.float32)),
                               _ptr(np.ascontiguousarray(kq, dtype=np.float32)), _ptr(out), c_int(batch),
                               c_int(v_heads), c_int(k_heads), c_int(dv), c_int(dk))
    return out


# ---- glue --------------------------------------------------------------------------

def rmsnorm_bf16(input_bits, residual_bits, weight_bits, batch, hidden, epsilon=1e-6):
    """Returns output bits; `residual_bits` (or None) is updated in place."""
    out = np.zeros((batch, hidden), dtype=np.uint16)
    lib().qo_rmsnorm_bf16(_ptr(np.ascontiguousarray(input_bits, dtype=np.uint16)), _ptr(residual_bits),
                          _ptr(np.ascontiguousarray(weight_bits, dtype=np.uint16)), _ptr(out), c_int(batch),
                          c_int(hidden), c_float(epsilon))
    return out


def delta_prepare_decode(mixed, a_proj, b_proj, conv_weight, a_log, dt_bias, conv_state, state_slots, batch,
                         mixed_stride, gate_stride, k_heads, v_heads, head_dim=128):
    """`a_proj` / `b_proj` are views into the mixed row (pass offsets via slicing a flat array)."""
    q = np.zeros((batch, k_heads, head_dim), dtype=np.float32)
    k = np.zeros((batch, k_heads, head_dim), dtype=np.float32)
    v = np.zeros((batch, v_heads, head_dim), dtype=np.float32)
    alpha = np.zeros((batch, v_heads), dtype=np.float32)
    beta = np.zeros((batch, v_heads), dtype=np.float32)
    kq = np.zeros((batch, k_heads), dtype=np.float32)
    lib().qo_delta_prepare_decode(
        _ptr(mixed), c_void_p(a_proj), c_void_p(b_proj), _ptr(conv_weight), _ptr(a_log), _ptr(dt_bias),
        _ptr(conv_state), _ptr(np.ascontiguousarray(state_slots, dtype=np.uint32)), _ptr(q), _ptr(k), _ptr(v),
        _ptr(alpha), _ptr(beta), _ptr(kq), c_int(batch), c_int(mixed_stride), c_int(gate_stride), c_int(k_heads),
        c_int(v_heads), c_int(head_dim))
    return q, k, v, alpha, beta, kq


def delta_gated_rmsnorm(values, gate_ptr, weight_bits, batch, heads, gate_stride, head_dim=128, epsilon=1e-6):
    out = np.zeros((batch, heads, head_dim), dtype=np.uint16)
    lib().qo_delta_gated_rmsnorm(_ptr(np.ascontiguousarray(values, dtype=np.float32)), c_void_p(gate_ptr),
                                 _ptr(np.ascontiguousarray(weight_bits, dtype=np.uint16)), _ptr(out), c_int(batch),
                                 c_int(heads), c_int(head_dim), c_float(epsilon), c_int(gate_stride))
    return out


def prepare_attention_decode_fp8(query_gate, key_proj, value_proj, q_norm_w, k_norm_w, cosine, sine, physical_blocks,
                                 block_offsets, key_cache, value_cache, batch, page_size, q_heads=24, kv_heads=4,
                                 head_dim=256, rope_dim=64, epsilon=1e-6, k_scale=None, v_scale=None):
    """Writes the new token's K/V into the caches in place; returns query bits."""
    query = np.zeros((batch, q_heads, head_dim), dtype=np.uint16)
    k_inv = None if k_scale is None else np.ascontiguousarray(1.0 / np.asarray(k_scale, dtype=np.float32),
                                                              dtype=np.float32)
    v_inv = None if v_scale is None else np.ascontiguousarray(1.0 / np.asarray(v_scale, dtype=np.float32),
                                                              dtype=np.float32)
    lib().qo_prepare_attention_decode_fp8(
        _ptr(query_gate), _ptr(key_proj), _ptr(value_proj), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cosine), _ptr(sine),
        _ptr(np.ascontiguousarray(physical_blocks, dtype=np.uint32)),
        _ptr(np.ascontiguousarray(block_offsets, dtype=np.uint32)), _ptr(query), _ptr(key_cache), _ptr(value_cache),
        c_int(batch), c_float(epsilon), c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(rope_dim),
        c_int(page_size), _ptr(k_inv), _ptr(v_inv))
    return query


def fp8_embedding_gather(table, row_scales, token_ids, cols, vocab):
    token_ids = np.ascontiguousarray(token_ids, dtype=np.uint32)
    out = np.zeros((token_ids.size, cols), dtype=np.uint16)
    lib().qo_fp8_embedding_gather(_ptr(table), _ptr(row_scales), _ptr(token_ids), _ptr(out), c_int(token_ids.size),
                                  c_int(cols), c_int(vocab))
    return out


def fp8_lm_head(weights, row_scales, hidden_bits, batch, hidden_size, vocab):
    logits = np.zeros((batch, vocab), dtype=np.float32)
    lib().qo_fp8_lm_head(_ptr(weights), _ptr(row_scales), _ptr(np.ascontiguousarray(hidden_bits, dtype=np.uint16)),
                         _ptr(logits), c_int(batch), c_int(hidden_size), c_int(vocab))
    return logits


def fp8_quantize_rows(input_bits, rows, cols):
    out = np.zeros((rows, cols), dtype=np.uint8)
    scales = np.zeros(rows, dtype=np.float32)
    lib().qo_fp8_quantize_rows(_ptr(np.ascontiguousarray(input_bits, dtype=np.uint16)), _ptr(out), _ptr(scales),
                               c_int(rows), c_int(cols))
    return out, scales


def argmax(logits, vocab, batch):
    out = np.zeros(batch, dtype=np.uint32)
    lib().qo_argmax(_ptr(np.ascontiguousarray(logits, dtype=np.float32)), _ptr(out), c_int(vocab), c_int(batch))
    return out


# ---- layout --------------------------------------------------------------------------

def layout_decode(row_slots, seq_tokens, seq_blocks, seq_block_counts, max_blocks, page_size):
    row_slots = np.ascontiguousarray(row_slots, dtype=np.uint32)
    seq_tokens = np.ascontiguousarray(seq_tokens, dtype=np.uint32)
    seq_blocks = np.ascontiguousarray(seq_blocks, dtype=np.uint32)
    seq_block_counts = np.ascontiguousarray(seq_block_counts, dtype=np.uint32)
    rows = row_slots.size
    capacity = seq_tokens.size
    out = {
        "state_slots": np.zeros(rows, np.uint32),
        "positions": np.zeros(rows, np.uint32),
        "context_lengths": np.zeros(rows, np.uint32),
        "block_table_offsets": np.zeros(rows + 1, np.uint32),
        "block_ids": np.zeros(rows * max_blocks, np.uint32),
        "physical_blocks": np.zeros(rows, np.uint32),
        "block_offsets": np.zeros(rows, np.uint32),
        "block_tables": np.zeros((rows, max_blocks), np.uint32),
    }
    status = lib().qo_layout_decode(_ptr(row_slots), c_int(rows), _ptr(seq_tokens), _ptr(seq_blocks),
                                    _ptr(seq_block_counts), c_int(capacity), c_int(max_blocks), c_int(page_size),
                                    _ptr(out["state_slots"]), _ptr(out["positions"]), _ptr(out["context_lengths"]),
                                    _ptr(out["block_table_offsets"]), _ptr(out["block_ids"]),
                                    _ptr(out["physical_blocks"]), _ptr(out["block_offsets"]),
                                    _ptr(out["block_tables"]))
    out["status"] = int(status)
    if status == 0:
        out["block_ids"] = out["block_ids"][: int(out["block_table_offsets"][-1])].copy()
    return out


def rope_rows(positions, rope_dim=64, theta=1.0e7):
    positions = np.ascontiguousarray(positions, dtype=np.uint32)
    cosine = np.zeros((positions.size, rope_dim), dtype=np.uint16)
    sine = np.zeros((positions.size, rope_dim), dtype=np.uint16)
    lib().qo_rope_rows(_ptr(positions), c_int(positions.size), c_int(rope_dim), c_float(theta), _ptr(cosine),
                       _ptr(sine))
    return cosine, sine


def num_threads() -> int:
    return int(lib().qo_num_threads())


def set_num_threads(threads: int) -> None:
    lib().qo_set_num_threads(c_int(threads))
