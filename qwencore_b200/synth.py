"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

No dataset or checkpoint is involved: every tensor is drawn from a seeded generator.
numpy generators give host arrays for kernel-level parity cases; the `device_*` functions
draw the multi-gigabyte model tensors directly in HBM with a seeded torch generator.
"""

from __future__ import annotations

import hashlib

import numpy as np

# ---- number formats (host) ---------------------------------------------------------


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bits, round to nearest even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    out = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    out[np.isnan(x)] = 0x7FC0
    return out


def bf16_value(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _e4m3_positive_table() -> np.ndarray:
    values = np.zeros(0x7F, dtype=np.float64)
    for code in range(0x7F):
        exponent, mantissa = code >> 3, code & 7
        values[code] = mantissa * 2.0 ** -9 if exponent == 0 else (1 + mantissa / 8.0) * 2.0 ** (exponent - 7)
    return values


_E4M3_POSITIVE = _e4m3_positive_table()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    table = np.concatenate([_E4M3_POSITIVE, [np.nan]])
    magnitude = table[codes & 0x7F]
    return np.where(codes & 0x80, -magnitude, magnitude).astype(np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """Saturating round-to-nearest-even onto the e4m3 grid (finite, max 448)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    magnitude = np.minimum(np.abs(x).astype(np.float64), 448.0)
    upper = np.clip(np.searchsorted(_E4M3_POSITIVE, magnitude, side="left"), 0, 0x7E)
    lower = np.clip(upper - 1, 0, 0x7E)
    d_up = _E4M3_POSITIVE[upper] - magnitude
    d_lo = magnitude - _E4M3_POSITIVE[lower]
    pick_lower = (d_lo < d_up) | ((d_lo == d_up) & (lower % 2 == 0))
    code = np.where(pick_lower, lower, upper).astype(np.uint8)
    code[np.isnan(x)] = 0x7F
    return (code | (np.signbit(x).astype(np.uint8) << 7)).astype(np.uint8)


def generator(seed: int, name: str) -> np.random.Generator:
    """One independent stream per (seed, tensor name)."""
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return np.random.default_rng(int.from_bytes(digest[:8], "little"))


# ---- NVFP4 ---------------------------------------------------------------------------


def block_scale_storage_len(rows: int, in_features: int) -> int:
    return ((rows + 127) // 128 * 128) * ((in_features // 16 + 3) // 4 * 4)


def swizzle_index(rows: int, in_features: int) -> np.ndarray:
    """Destination offset of logical scale (row, group) in the 128x4 block-scale layout."""
    groups = in_features // 16
    group_blocks = (groups + 3) // 4
    row = np.arange(rows, dtype=np.int64)[:, None]
    group = np.arange(groups, dtype=np.int64)[None, :]
    return (((((row // 128) * group_blocks + group // 4) * 32 + row % 32) * 4 + (row % 128) // 32) * 4 +
            group % 4)


def swizzle_block_scales(scales: np.ndarray, rows: int, in_features: int) -> np.ndarray:
    out = np.zeros(block_scale_storage_len(rows, in_features), dtype=np.uint8)
    out[swizzle_index(rows, in_features).ravel()] = np.asarray(scales, dtype=np.uint8).ravel()
    return out


def nvfp4_matrix(seed: int, name: str, out_features: int, in_features: int):
    """Codes uniform over the 16 e2m1 values; one e4m3 scale per 16 = |N(0,1)| * 0.05.

    Returns (packed u8[out, in/2], logical scales u8[out, in/16], swizzled scales u8[...]).
    """
    rng = generator(seed, name)
    packed = rng.integers(0, 256, size=(out_features, in_features // 2), dtype=np.uint8)
    scales = e4m3_encode(np.abs(rng.standard_normal((out_features, in_features // 16), dtype=np.float32)) * 0.05)
    return packed, scales, swizzle_block_scales(scales, out_features, in_features)


def normal_bf16(seed: int, name: str, shape, std: float = 1.0) -> np.ndarray:
    rng = generator(seed, name)
    return bf16_bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))


# ---- paged attention (config: ragged batch over a permuted page pool) -----------------


def attention_case(seed: int, contexts, page_size: int, q_heads: int = 24, kv_heads: int = 4, head_dim: int = 256,
                   with_gate: bool = False, scaled: bool = False, extra_blocks: int = 3):
    """K/V e4m3 from N(0,1) (divided by a per-kv-head scale when `scaled`), Q bf16 N(0,1),
    physical pages randomly permuted in the table."""
    rng = generator(seed, "attention")
    contexts = np.asarray(contexts, dtype=np.uint32)
    batch = contexts.size
    blocks_per_row = (contexts + page_size - 1) // page_size
    max_blocks = int(blocks_per_row.max()) + 1
    num_blocks = int(blocks_per_row.sum()) + extra_blocks
    permutation = rng.permutation(num_blocks).astype(np.uint32)
    tables = np.zeros((batch, max_blocks), dtype=np.uint32)
    cursor = 0
    for b in range(batch):
        n = int(blocks_per_row[b])
        tables[b, :n] = permutation[cursor:cursor + n]
        cursor += n
    k_scale = v_scale = None
    k_values = rng.standard_normal((num_blocks, kv_heads, page_size, head_dim), dtype=np.float32)
    v_values = rng.standard_normal((num_blocks, kv_heads, page_size, head_dim), dtype=np.float32)
    if scaled:
        k_scale = (0.5 + rng.random(kv_heads)).astype(np.float32) / 64.0
        v_scale = (0.5 + rng.random(kv_heads)).astype(np.float32) / 64.0
        k_values = k_values / k_scale[None, :, None, None]
        v_values = v_values / v_scale[None, :, None, None]
    case = {
        "contexts": contexts,
        "block_tables": tables,
        "max_blocks": max_blocks,
        "num_blocks": num_blocks,
        "key_cache": e4m3_encode(k_values),
        "value_cache": e4m3_encode(v_values),
        "query": bf16_bits(rng.standard_normal((batch, q_heads, head_dim), dtype=np.float32)),
        "k_scale": k_scale,
        "v_scale": v_scale,
        "gate_projection": None,
    }
    if with_gate:
        case["gate_projection"] = bf16_bits(rng.standard_normal((batch, q_heads, 2 * head_dim), dtype=np.float32))
    return case


# ---- Gated DeltaNet ---------------------------------------------------------------------


def quantize_state_rows(rows: np.ndarray):
    """int8 codes + per-row fp32 scale: peak/127 grid, round to nearest even."""
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    peak = np.max(np.abs(rows), axis=-1, keepdims=True).astype(np.float32)
    inverse = np.divide(np.float32(127.0), peak, out=np.zeros_like(peak), where=peak > 0)
    codes = np.clip(np.rint(rows * inverse), -127, 127).astype(np.int8)
    scales = (peak[..., 0] * np.float32(1.0 / 127.0)).astype(np.float32)
    return codes, scales


def delta_case(seed: int, batch: int, v_heads: int, capacity: int | None = None, k_heads: int = 16, dim: int = 128):
    """State N(0, 0.1) quantised per row; bf16-representable q/k (L2-normalised, q scaled by
    1/sqrt(dim)), v ~ N(0,1), beta = sigmoid(N(0,1)), alpha = exp(-softplus(N(0,1)))."""
    rng = generator(seed, "delta")
    capacity = capacity or batch + 1
    state = rng.standard_normal((capacity, v_heads, dim, dim), dtype=np.float32) * np.float32(0.1)
    codes, scales = quantize_state_rows(state)
    slots = rng.permutation(capacity)[:batch].astype(np.uint32)

    def unit(x):
        return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + np.float32(1e-6))

    q = unit(bf16_value(bf16_bits(rng.standard_normal((batch, k_heads, dim), dtype=np.float32))))
    k = unit(bf16_value(bf16_bits(rng.standard_normal((batch, k_heads, dim), dtype=np.float32))))
    q = (q * np.float32(1.0 / np.sqrt(dim))).astype(np.float32)
    k = k.astype(np.float32)
    v = bf16_value(bf16_bits(rng.standard_normal((batch, v_heads, dim), dtype=np.float32)))
    beta = (1.0 / (1.0 + np.exp(-rng.standard_normal((batch, v_heads))))).astype(np.float32)
    alpha = np.exp(-np.log1p(np.exp(rng.standard_normal((batch, v_heads))))).astype(np.float32)
    kq = np.sum(q * k, axis=-1).astype(np.float32)
    return {"state": codes, "scales": scales, "slots": slots, "q": q, "k": k, "v": v, "alpha": alpha, "beta": beta,
            "kq": kq, "capacity": capacity}


def log_uniform_contexts(seed: int, batch: int, low: int, high: int) -> np.ndarray:
    rng = generator(seed, "contexts")
    return np.exp(rng.uniform(np.log(low), np.log(high), size=batch)).astype(np.int64).clip(low, high).astype(np.uint32)


def uniform_contexts(seed: int, batch: int, low: int, high: int) -> np.ndarray:
    rng = generator(seed, "contexts")
    return rng.integers(low, high + 1, size=batch).astype(np.uint32)
