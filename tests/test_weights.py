"""The layout half of the weight loader (qwencore_b200/weights.py; the reference's
crates/qwc-engine/src/weights.rs:374-562): fusing rules, consumption checks and the scale swizzle, on
CPU against a recording stand-in for the engine."""

import types

import numpy as np
import pytest

from oracle import oracle
from qwencore_b200 import weights


def quant(rng, n, k, scale=1.0):
    return weights.QuantLinear(rng.integers(0, 256, (n, k // 2), dtype=np.uint8),
                               rng.integers(0x20, 0x40, (n, k // 16), dtype=np.uint8), scale)


class Recorder:
    def __init__(self, **config):
        values = dict(hidden=256, intermediate=512, full_attention_interval=4, delta_value_heads=32, num_layers=4,
                      vocab=64)
        values.update(config)
        self.config = types.SimpleNamespace(**values)
        self.written, self.scales = {}, {}

    def write(self, name, layer, values):
        self.written[(name, layer)] = np.array(values, copy=True)

    def set_weight_global_scale(self, name, layer, value):
        self.scales[(name, layer)] = value


def checkpoint_layer(rng, config, layer, scale=1.0):
    projections = {name: quant(rng, n, k, scale) for name, (n, k) in weights.layer_shapes(config, layer).items()}
    plain = {name: rng.integers(0, 65536, count, dtype=np.uint16)
             for name, (_, count) in weights.plain_names(config, layer).items()}
    return projections, plain


def test_mixer_parts_are_concatenated_in_row_order_and_need_one_global_scale():
    # weights.rs:497-560
    rng = np.random.default_rng(0)
    parts = {"in_proj_qkv": quant(rng, 8192, 256, 3.0), "in_proj_z": quant(rng, 4096, 256, 3.0),
             "in_proj_a": quant(rng, 32, 256, 3.0), "in_proj_b": quant(rng, 32, 256, 3.0)}
    fused = weights.fuse_rows(parts, weights.MIXER_PARTS)
    assert (fused.out_features, fused.in_features, fused.weight_global_scale) == (12352, 256, 3.0)
    assert np.array_equal(fused.packed[8192:12288], parts["in_proj_z"].packed)
    assert np.array_equal(fused.block_scales[12320:], parts["in_proj_b"].block_scales)
    parts["in_proj_a"] = quant(rng, 32, 256, 2.0)
    with pytest.raises(weights.LoadError, match="in_proj_a: global scale differs"):
        weights.fuse_rows(parts, weights.MIXER_PARTS)
    del parts["in_proj_a"]
    with pytest.raises(weights.LoadError, match="needs exactly"):
        weights.fuse_rows(parts, weights.MIXER_PARTS)
    parts["in_proj_a"] = quant(rng, 32, 512, 3.0)
    with pytest.raises(weights.LoadError, match="K = 512 against 256"):
        weights.fuse_rows(parts, weights.MIXER_PARTS)


def test_a_layer_is_stored_under_the_engine_names_with_swizzled_scales():
    rng = np.random.default_rng(1)
    engine = Recorder()
    for layer in (0, 3):  # a DeltaNet layer and a full-attention layer
        projections, plain = checkpoint_layer(rng, engine.config, layer, scale=5.0)
        stats = weights.load_layer(engine, layer, projections, plain)
        full = layer == 3
        names = ["gate", "up", "down"] + (["qkv", "o"] if full else ["in_proj", "la_out"])
        assert stats["projections"] == 5 and all(engine.scales[(name, layer)] == 5.0 for name in names)
        gate = projections["gate_proj"]
        assert np.array_equal(engine.written[("gate.packed", layer)], gate.packed)
        assert np.array_equal(engine.written[("gate.scales", layer)],
                              oracle.swizzle_block_scales(gate.block_scales, 512, 256))
        if full:
            rows = np.concatenate([projections[name].packed for name in ("q_proj", "k_proj", "v_proj")])
            assert np.array_equal(engine.written[("qkv.packed", layer)], rows) and rows.shape[0] == 14336
            assert np.array_equal(engine.written[("q_norm", layer)], plain["self_attn.q_norm.weight"])
        else:
            rows = np.concatenate([projections[name].block_scales for name in weights.MIXER_PARTS])
            assert np.array_equal(engine.written[("in_proj.scales", layer)],
                                  oracle.swizzle_block_scales(rows, 12352, 256))
            assert np.array_equal(engine.written[("conv_weight", layer)], plain["linear_attn.conv1d.weight"])
        assert stats["plain_bytes"] == sum(v.nbytes for v in plain.values())


def test_every_tensor_must_be_consumed_and_none_left_over():
    # weights.rs:427-432 and the `take` / `projection` closures
    rng = np.random.default_rng(2)
    engine = Recorder()
    projections, plain = checkpoint_layer(rng, engine.config, 0)
    with pytest.raises(weights.LoadError, match="not consumed"):
        weights.load_layer(engine, 0, dict(projections, q_proj=quant(rng, 16, 256)), plain)
    with pytest.raises(weights.LoadError, match="not consumed"):
        weights.load_layer(engine, 0, projections, dict(plain, extra=np.zeros(4, np.uint16)))
    missing = dict(projections)
    del missing["out_proj"]
    with pytest.raises(weights.LoadError, match="no projection out_proj"):
        weights.load_layer(engine, 0, missing, plain)
    short = dict(plain)
    del short["linear_attn.A_log"]
    with pytest.raises(weights.LoadError, match="missing linear_attn.A_log"):
        weights.load_layer(engine, 0, projections, short)
    wrong = dict(projections, down_proj=quant(rng, 256, 256))
    with pytest.raises(weights.LoadError, match="down_proj: shape"):
        weights.load_layer(engine, 0, wrong, plain)
    with pytest.raises(weights.LoadError, match="do not belong together"):
        weights.QuantLinear(np.zeros((4, 32), np.uint8), np.zeros((4, 5), np.uint8), 1.0)
    with pytest.raises(weights.LoadError, match="positive"):
        weights.QuantLinear(np.zeros((4, 32), np.uint8), np.zeros((4, 4), np.uint8), 0.0)


def test_attention_projections_with_different_scales_are_refused():
    """q | k | v run as one matrix here (one scalar per launch): a checkpoint whose three global scales differ
    cannot be loaded into this layout and is told so."""
    rng = np.random.default_rng(3)
    engine = Recorder()
    projections, plain = checkpoint_layer(rng, engine.config, 3)
    projections["k_proj"] = quant(rng, 1024, 256, 7.0)
    with pytest.raises(weights.LoadError, match="k_proj: global scale differs"):
        weights.load_layer(engine, 3, projections, plain)
