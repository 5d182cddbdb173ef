"""The file side of the weight loader (qwencore_b200/checkpoint.py; the reference's
crates/qwc-model/src/{safetensors,checkpoint,names}.rs): shards through mmap, the index, the tensor
names, the check against the architecture, and the walk that feeds `weights.load_layer`.  The files are
written by the test itself, at a width small enough for a CPU run."""

import json
import os
import struct
import types

import numpy as np
import pytest

from qwencore_b200 import checkpoint, weights
from test_weights import Recorder, checkpoint_layer


def small_config(**overrides):
    values = dict(hidden=256, intermediate=512, full_attention_interval=4, delta_value_heads=32, num_layers=4,
                  vocab=640)
    values.update(overrides)
    return types.SimpleNamespace(**values)


def model_tensors(config, seed=0):
    rng = np.random.default_rng(seed)
    layers = [checkpoint_layer(rng, config, layer, scale=1.0 + layer) for layer in range(config.num_layers)]
    final_norm = rng.integers(0, 65536, config.hidden, dtype=np.uint16)
    embed = rng.integers(0, 65536, (config.vocab, config.hidden), dtype=np.uint16)
    head = rng.integers(0, 65536, (config.vocab, config.hidden), dtype=np.uint16)
    tensors, dtypes = checkpoint.checkpoint_tensors(config, layers, final_norm, embed, head)
    return layers, tensors, dtypes


def write_raw_shard(path, header, data=b""):
    encoded = header if isinstance(header, bytes) else json.dumps(header).encode()
    with open(path, "wb") as file:
        file.write(struct.pack("<Q", len(encoded)) + encoded + data)


def test_shard_round_trip_hands_out_views_of_the_mapping(tmp_path):
    rng = np.random.default_rng(1)
    tensors = {"a.weight_packed": rng.integers(0, 256, (8, 16), dtype=np.uint8),
               "a.weight_scale": rng.integers(0, 256, (8, 2), dtype=np.uint8),
               "a.weight_global_scale": np.array([3.5], dtype=np.float32),
               "norm": rng.integers(0, 65536, 32, dtype=np.uint16)}
    path = str(tmp_path / "one.safetensors")
    checkpoint.write_shard(path, tensors, {"a.weight_scale": "F8_E4M3"})
    shard = checkpoint.Shard(path)
    assert sorted(shard.names()) == sorted(tensors)
    assert [shard.info(name).dtype for name in tensors] == ["U8", "F8_E4M3", "F32", "BF16"]
    assert shard.info("a.weight_packed").shape == [8, 16] and shard.info("norm").bytes() == 64
    for name, array in tensors.items():
        raw = shard.bytes(name)
        assert raw.tobytes() == array.tobytes()
        assert not raw.flags.owndata and not raw.flags.writeable  # a slice of the file, not a copy
    assert shard.info("nothing") is None and shard.bytes("nothing") is None
    assert shard.data_offset % 8 == 0
    # the pages can be dropped and fault in again
    shard.evict_pages()
    assert shard.bytes("norm").tobytes() == tensors["norm"].tobytes()


def test_malformed_shards_are_refused(tmp_path):
    path = str(tmp_path / "bad.safetensors")
    with open(path, "wb") as file:
        file.write(b"\x01\x02")
    with pytest.raises(checkpoint.CheckpointError, match="shorter than"):
        checkpoint.Shard(path)
    with open(path, "wb") as file:
        file.write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(checkpoint.CheckpointError, match="past the end"):
        checkpoint.Shard(path)
    write_raw_shard(path, b"{not json")
    with pytest.raises(checkpoint.CheckpointError, match="does not parse"):
        checkpoint.Shard(path)
    write_raw_shard(path, [1, 2])
    with pytest.raises(checkpoint.CheckpointError, match="not an object"):
        checkpoint.Shard(path)
    write_raw_shard(path, {"t": {"dtype": "I64", "shape": [1], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(checkpoint.CheckpointError, match="unsupported type I64 for t"):
        checkpoint.Shard(path)
    write_raw_shard(path, {"t": {"dtype": "U8", "shape": [4]}}, b"\0" * 4)
    with pytest.raises(checkpoint.CheckpointError, match="no dtype, shape or data_offsets"):
        checkpoint.Shard(path)
    write_raw_shard(path, {"t": {"dtype": "U8", "shape": [16], "data_offsets": [0, 16]}}, b"\0" * 4)
    with pytest.raises(checkpoint.CheckpointError, match="outside the file"):
        checkpoint.Shard(path)
    write_raw_shard(path, {"t": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 4)
    with pytest.raises(checkpoint.CheckpointError, match="4 bytes for shape"):
        checkpoint.Shard(path)
    # metadata is not a tensor
    write_raw_shard(path, {"__metadata__": {"format": "pt"}, "t": {"dtype": "U8", "shape": [2], "data_offsets": [0, 2]}},
                    b"\x07\x09")
    assert checkpoint.Shard(path).bytes("t").tolist() == [7, 9]


def test_tensor_names_follow_the_checkpoint(tmp_path):
    config = small_config()
    linear = {prefix: (rows, cols) for prefix, _, rows, cols in checkpoint.quant_linears(config, 0)}
    assert linear == {
        "model.language_model.layers.0.mlp.gate_proj": (512, 256),
        "model.language_model.layers.0.mlp.up_proj": (512, 256),
        "model.language_model.layers.0.mlp.down_proj": (256, 512),
        "model.language_model.layers.0.linear_attn.in_proj_qkv": (8192, 256),
        "model.language_model.layers.0.linear_attn.in_proj_z": (4096, 256),
        "model.language_model.layers.0.linear_attn.in_proj_a": (32, 256),
        "model.language_model.layers.0.linear_attn.in_proj_b": (32, 256),
        "model.language_model.layers.0.linear_attn.out_proj": (256, 4096)}
    attention = {prefix: (rows, cols) for prefix, _, rows, cols in checkpoint.quant_linears(config, 3)}
    assert attention["model.language_model.layers.3.self_attn.q_proj"] == (2 * 24 * 256, 256)
    assert attention["model.language_model.layers.3.self_attn.k_proj"] == (4 * 256, 256)
    assert attention["model.language_model.layers.3.self_attn.o_proj"] == (256, 24 * 256)
    assert {name: shape for name, _, shape in checkpoint.plain_tensors(config, 0)} == {
        "model.language_model.layers.0.input_layernorm.weight": [256],
        "model.language_model.layers.0.post_attention_layernorm.weight": [256],
        "model.language_model.layers.0.linear_attn.conv1d.weight": [8192, 1, 4],
        "model.language_model.layers.0.linear_attn.A_log": [32],
        "model.language_model.layers.0.linear_attn.dt_bias": [32],
        "model.language_model.layers.0.linear_attn.norm.weight": [128]}
    assert [name for name, _, _ in checkpoint.plain_tensors(config, 3)][2:] == [
        "model.language_model.layers.3.self_attn.q_norm.weight",
        "model.language_model.layers.3.self_attn.k_norm.weight"]


def test_a_complete_checkpoint_validates_and_counts_what_it_holds(tmp_path):
    config = small_config()
    _, tensors, dtypes = model_tensors(config)
    tensors["model.visual.patch_embed.weight"] = np.zeros((4, 8), dtype=np.uint16)  # nothing a text engine reads
    tensors["mtp.norm.weight"] = np.zeros(config.hidden, dtype=np.uint16)
    checkpoint.write_checkpoint(str(tmp_path), tensors, dtypes, tensors_per_shard=40)
    files = sorted(name for name in os.listdir(tmp_path) if name.endswith(".safetensors"))
    assert len(files) == -(-len(tensors) // 40) and files[0] == f"model-00001-of-{len(files):05d}.safetensors"
    model = checkpoint.Checkpoint.open(str(tmp_path))
    assert model.tensor_count() == len(tensors) and len(model.shards) == len(files)
    problems, stats = model.validate(config)
    assert problems == []
    # three DeltaNet layers of 3 + 5 projections, one attention layer of 3 + 4
    assert stats["quantized_linears"] == 3 * 8 + 7
    assert stats["tensors"] == 4 * stats["quantized_linears"] + (3 * 6 + 4) + 3 + 1
    assert stats["packed_bytes"] == sum(t.nbytes for n, t in tensors.items() if n.endswith("weight_packed"))
    assert stats["scale_bytes"] == stats["packed_bytes"] // 8
    assert stats["embed_bytes"] == stats["lm_head_bytes"] == config.vocab * config.hidden * 2
    assert (stats["unused_tensors"], stats["unused_bytes"], stats["mtp_bytes"]) == (1, 64, 2 * config.hidden)
    assert model.scalar_f32("model.language_model.layers.2.mlp.down_proj.weight_global_scale") == 3.0
    assert model.info("not.there") is None and model.bytes("not.there") is None and model.scalar_f32("not.there") is None


def test_validate_names_every_mismatch(tmp_path):
    config = small_config()
    _, tensors, dtypes = model_tensors(config)
    gate = "model.language_model.layers.1.mlp.gate_proj"
    del tensors["model.language_model.layers.0.linear_attn.A_log"]
    del tensors[f"{gate}.input_global_scale"]
    tensors["model.language_model.layers.3.self_attn.q_norm.weight"] = np.zeros(128, dtype=np.uint16)
    tensors["model.language_model.layers.2.mlp.up_proj.weight_packed"] = np.zeros((512, 64), dtype=np.uint8)
    del dtypes["model.language_model.layers.2.mlp.down_proj.weight_scale"]  # written as plain U8
    tensors[checkpoint.LM_HEAD] = np.zeros((config.vocab, 128), dtype=np.uint16)
    checkpoint.write_checkpoint(str(tmp_path), tensors, dtypes)
    problems, stats = checkpoint.Checkpoint(str(tmp_path)).validate(config)
    assert sorted(problems) == sorted([
        "missing model.language_model.layers.0.linear_attn.A_log",
        f"missing {gate}.input_global_scale",
        "model.language_model.layers.3.self_attn.q_norm.weight: shape [128], expected [256]",
        "model.language_model.layers.2.mlp.up_proj.weight_packed: shape [512, 64], expected [512, 128]",
        "model.language_model.layers.2.mlp.down_proj.weight_scale: type U8, expected F8_E4M3",
        "lm_head.weight: shape [640, 128], expected [640, 256]"])
    assert stats["quantized_linears"] == 31 - 3


def test_an_index_without_a_weight_map_is_refused(tmp_path):
    with open(tmp_path / "model.safetensors.index.json", "w") as file:
        json.dump({"metadata": {}}, file)
    with pytest.raises(checkpoint.CheckpointError, match="no weight_map"):
        checkpoint.Checkpoint(str(tmp_path))
    with open(tmp_path / "model.safetensors.index.json", "w") as file:
        file.write("{")
    with pytest.raises(checkpoint.CheckpointError, match="does not parse"):
        checkpoint.Checkpoint(str(tmp_path))
    with pytest.raises(FileNotFoundError):
        checkpoint.Checkpoint(str(tmp_path / "nowhere"))


def test_the_walk_over_the_layers_feeds_the_loader(tmp_path):
    """Checkpoint.layer hands `weights.load_layer` what it takes: a recording engine ends up with the same
    tensors as when the arrays are passed directly."""
    config = small_config()
    layers, tensors, dtypes = model_tensors(config, seed=4)
    checkpoint.write_checkpoint(str(tmp_path), tensors, dtypes, tensors_per_shard=25)
    model = checkpoint.Checkpoint(str(tmp_path))
    direct, from_files = Recorder(vocab=config.vocab), Recorder(vocab=config.vocab)
    for layer in range(config.num_layers):
        want = weights.load_layer(direct, layer, *layers[layer])
        projections, plain = model.layer(config, layer)
        assert projections["gate_proj"].input_global_scale == 1.0
        assert not projections["gate_proj"].packed.flags.owndata  # still the mapping
        got = weights.load_layer(from_files, layer, projections, plain)
        assert got == want
        model.evict_file_pages()
    assert direct.written.keys() == from_files.written.keys() and direct.scales == from_files.scales
    for key, value in direct.written.items():
        assert np.array_equal(value, from_files.written[key]), key
    assert np.array_equal(model.vocab_table(config, checkpoint.EMBED), tensors[checkpoint.EMBED])
    with pytest.raises(checkpoint.CheckpointError, match="expected BF16"):
        model.vocab_table(small_config(vocab=641), checkpoint.LM_HEAD)


def test_load_refuses_a_checkpoint_that_does_not_validate(tmp_path):
    config = small_config()
    _, tensors, dtypes = model_tensors(config)
    del tensors[checkpoint.FINAL_NORM]
    checkpoint.write_checkpoint(str(tmp_path), tensors, dtypes)
    engine = Recorder(vocab=config.vocab)
    with pytest.raises(checkpoint.CheckpointError, match="missing model.language_model.norm.weight"):
        checkpoint.load(engine, checkpoint.Checkpoint(str(tmp_path)))
    assert engine.written == {}  # nothing was uploaded before the check
