"""Checkpoint layouts -> the engine's resident layouts (the layout half of the reference's loader,
crates/qwc-engine/src/weights.rs:374-443, :445-562, :609-659).

A checkpoint hands every NVFP4 projection as packed nibbles `u8[N, K/2]`, logical e4m3 block scales
`u8[N, K/16]` and an fp32 `weight_global_scale`; norms, conv taps and gates as bf16; the vocabulary
tables as bf16 `[vocab, hidden]`.  What the kernels read differs in four ways, and this module does
exactly those four conversions and nothing else (no file parsing: there is no checkpoint here, the
tensors come as numpy arrays under the reference's own names):

* block scales go into the 128 x 4 swizzle of the tensor-core kernels (weights.rs `Linear::from_host`);
* the DeltaNet in-projection is the row-wise concatenation in_proj_qkv | in_proj_z | in_proj_a | in_proj_b,
  legal only when the parts share their global scales (weights.rs:497-560: one scalar per launch);
* this engine also runs q_proj | k_proj | v_proj as one matrix - the same rule applies, and a
  checkpoint whose three scales differ is refused (the reference keeps them apart);
* the vocabulary tables become e4m3 rows with a per-row fp32 scale, chunk by chunk on the device
  (`qwc_fp8_quantize_rows`, weights.rs:609-659), so that the bf16 table never has to be resident.

Every layer tensor the architecture describes must be consumed and none may be left over
(weights.rs:427-432).
"""

from __future__ import annotations

import numpy as np

from . import synth

MIXER_PARTS = ("in_proj_qkv", "in_proj_z", "in_proj_a", "in_proj_b")  # in the order they lie in a row
ATTENTION_PARTS = ("q_proj", "k_proj", "v_proj")
VOCAB_CHUNK_ROWS = 8192  # 84 MB of bf16 staging at hidden 5120, as the reference's loader


class LoadError(ValueError):
    """A checkpoint tensor that is missing, left over, mis-shaped or cannot be fused."""


class QuantLinear:
    """One NVFP4 projection as a checkpoint holds it."""

    def __init__(self, packed: np.ndarray, block_scales: np.ndarray, weight_global_scale: float):
        self.packed = np.ascontiguousarray(packed, dtype=np.uint8)
        self.block_scales = np.ascontiguousarray(block_scales, dtype=np.uint8)
        self.weight_global_scale = float(weight_global_scale)
        if self.packed.ndim != 2 or self.block_scales.shape != (self.packed.shape[0], self.packed.shape[1] // 8):
            raise LoadError(f"packed {self.packed.shape} and block scales {self.block_scales.shape} do not belong together")
        if not self.weight_global_scale > 0.0:
            raise LoadError("weight_global_scale must be positive")

    @property
    def out_features(self) -> int:
        return self.packed.shape[0]

    @property
    def in_features(self) -> int:
        return self.packed.shape[1] * 2


def fuse_rows(parts: dict, order) -> QuantLinear:
    """Row-wise concatenation of projections that read the same input (weights.rs:497-560)."""
    missing = [name for name in order if name not in parts]
    if missing or len(parts) != len(order):
        raise LoadError(f"fused projection needs exactly {list(order)}; got {sorted(parts)}")
    first = parts[order[0]]
    for name in order:
        part = parts[name]
        if part.weight_global_scale != first.weight_global_scale:
            raise LoadError(f"{name}: global scale differs from the other parts of the fused projection")
        if part.in_features != first.in_features:
            raise LoadError(f"{name}: K = {part.in_features} against {first.in_features}")
    return QuantLinear(np.concatenate([parts[name].packed for name in order]),
                       np.concatenate([parts[name].block_scales for name in order]), first.weight_global_scale)


def store_linear(engine, name: str, layer: int, linear: QuantLinear, out_features: int, in_features: int) -> int:
    """Writes one projection into the engine (scales swizzled); returns the resident bytes."""
    if (linear.out_features, linear.in_features) != (out_features, in_features):
        raise LoadError(f"layer {layer} {name}: shape {(linear.out_features, linear.in_features)}, "
                        f"expected {(out_features, in_features)}")
    swizzled = synth.swizzle_block_scales(linear.block_scales, out_features, in_features)
    engine.write(f"{name}.packed", layer, linear.packed)
    engine.write(f"{name}.scales", layer, swizzled)
    engine.set_weight_global_scale(name, layer, linear.weight_global_scale)
    return linear.packed.nbytes + swizzled.nbytes


def layer_shapes(config, layer: int) -> dict:
    """Checkpoint name -> (N, K) of every quantised projection of a layer (crates/qwc-core/src/arch.rs:10-98)."""
    hidden, inter = config.hidden, config.intermediate
    shapes = {"gate_proj": (inter, hidden), "up_proj": (inter, hidden), "down_proj": (hidden, inter)}
    if (layer + 1) % config.full_attention_interval == 0:
        shapes.update({"q_proj": (24 * 2 * 256, hidden), "k_proj": (4 * 256, hidden), "v_proj": (4 * 256, hidden),
                       "o_proj": (hidden, 24 * 256)})
    else:
        heads = config.delta_value_heads
        shapes.update({"in_proj_qkv": (2 * 16 * 128 + heads * 128, hidden), "in_proj_z": (heads * 128, hidden),
                       "in_proj_a": (heads, hidden), "in_proj_b": (heads, hidden), "out_proj": (hidden, heads * 128)})
    return shapes


def plain_names(config, layer: int) -> dict:
    """Checkpoint name -> (engine tensor, element count) of the bf16 tensors of a layer."""
    names = {"input_layernorm.weight": ("input_norm", config.hidden),
             "post_attention_layernorm.weight": ("post_norm", config.hidden)}
    if (layer + 1) % config.full_attention_interval == 0:
        names.update({"self_attn.q_norm.weight": ("q_norm", 256), "self_attn.k_norm.weight": ("k_norm", 256)})
    else:
        heads = config.delta_value_heads
        channels = 2 * 16 * 128 + heads * 128
        names.update({"linear_attn.conv1d.weight": ("conv_weight", channels * 4), "linear_attn.A_log": ("a_log", heads),
                      "linear_attn.dt_bias": ("dt_bias", heads), "linear_attn.norm.weight": ("out_norm", 128)})
    return names


def load_layer(engine, layer: int, projections: dict, plain: dict) -> dict:
    """One layer (weights.rs:374-443): `projections` maps checkpoint names (gate_proj, in_proj_qkv, ...) to
    QuantLinear, `plain` maps checkpoint names to bf16 bit patterns (uint16).  Returns byte counts."""
    config = engine.config
    shapes = layer_shapes(config, layer)
    projections = dict(projections)
    plain = dict(plain)
    stats = {"quantized_bytes": 0, "projections": 0, "plain_bytes": 0}

    def take(name):
        if name not in projections:
            raise LoadError(f"no projection {name} in layer {layer}")
        return projections.pop(name)

    def shaped(name):
        part = take(name)
        if (part.out_features, part.in_features) != shapes[name]:
            raise LoadError(f"layer {layer} {name}: shape {(part.out_features, part.in_features)}, "
                            f"expected {shapes[name]}")
        return part

    def store(engine_name, linear):
        stats["quantized_bytes"] += store_linear(engine, engine_name, layer, linear, linear.out_features,
                                                 linear.in_features)
        stats["projections"] += 1

    store("gate", shaped("gate_proj"))
    store("up", shaped("up_proj"))
    store("down", shaped("down_proj"))
    if (layer + 1) % config.full_attention_interval == 0:
        store("qkv", fuse_rows({name: shaped(name) for name in ATTENTION_PARTS}, ATTENTION_PARTS))
        store("o", shaped("o_proj"))
    else:
        store("in_proj", fuse_rows({name: shaped(name) for name in MIXER_PARTS}, MIXER_PARTS))
        store("la_out", shaped("out_proj"))
    if projections:
        raise LoadError(f"projection {sorted(projections)[0]} of layer {layer} not consumed by the loader")

    for name, (tensor, elements) in plain_names(config, layer).items():
        if name not in plain:
            raise LoadError(f"missing {name} in layer {layer}")
        values = np.ascontiguousarray(plain.pop(name), dtype=np.uint16).reshape(-1)
        if values.size != elements:
            raise LoadError(f"layer {layer} {name}: {values.size} elements, expected {elements}")
        engine.write(tensor, layer, values)
        stats["plain_bytes"] += values.nbytes
    if plain:
        raise LoadError(f"tensor {sorted(plain)[0]} of layer {layer} not consumed by the loader")
    return stats


def load_vocab(engine, name: str, table_bf16: np.ndarray, chunk_rows: int = VOCAB_CHUNK_ROWS) -> int:
    """`[vocab, hidden]` bf16 -> the engine's e4m3 rows and per-row scales ("embed" or "lm_head"), converted
    on the device chunk by chunk through one staging buffer (weights.rs:609-659).  Returns resident bytes."""
    import torch

    from . import abi

    config = engine.config
    table = np.ascontiguousarray(table_bf16, dtype=np.uint16)
    if table.shape != (config.vocab, config.hidden):
        raise LoadError(f"{name}: shape {table.shape}, expected {(config.vocab, config.hidden)}")
    codes, code_bytes = engine.tensor_ptr(name, 0)
    scales, scale_bytes = engine.tensor_ptr(f"{name}_scales", 0)
    if code_bytes != table.size or scale_bytes != 4 * config.vocab:
        raise LoadError(f"{name}: the engine holds {code_bytes} bytes, the table needs {table.size}")
    staging = torch.empty((min(chunk_rows, config.vocab), config.hidden), dtype=torch.int16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for first in range(0, config.vocab, chunk_rows):
        rows = min(chunk_rows, config.vocab - first)
        chunk = table[first:first + rows].view(np.int16)
        if not chunk.flags.writeable:  # a view of a mapped file: torch wants memory it may write to
            chunk = np.array(chunk)
        staging[:rows].copy_(torch.from_numpy(chunk))
        abi.check(abi.lib.qwc_fp8_quantize_rows(staging.data_ptr(), codes, scales, rows, config.hidden, first, stream),
                  "qwc_fp8_quantize_rows")
    torch.cuda.synchronize()
    return code_bytes + scale_bytes


def load_model(engine, layers, final_norm: np.ndarray, embed_bf16: np.ndarray, lm_head_bf16: np.ndarray) -> dict:
    """The whole model: `layers[i] = (projections, plain)` as for load_layer."""
    if len(layers) != engine.config.num_layers:
        raise LoadError(f"{len(layers)} layers, expected {engine.config.num_layers}")
    total = {"quantized_bytes": 0, "projections": 0, "plain_bytes": 0, "vocab_bytes": 0}
    for index, (projections, plain) in enumerate(layers):
        for key, value in load_layer(engine, index, projections, plain).items():
            total[key] += value
    norm = np.ascontiguousarray(final_norm, dtype=np.uint16).reshape(-1)
    if norm.size != engine.config.hidden:
        raise LoadError("final norm: wrong size")
    engine.write("final_norm", 0, norm)
    total["plain_bytes"] += norm.nbytes
    total["vocab_bytes"] += load_vocab(engine, "embed", embed_bf16)
    total["vocab_bytes"] += load_vocab(engine, "lm_head", lm_head_bf16)
    return total
