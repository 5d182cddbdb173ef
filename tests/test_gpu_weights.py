"""Weight-loader layouts on the device: the bf16 -> e4m3 row conversion of the vocabulary tables
(qwc_fp8_quantize_rows, crates/qwc-cuda/src/ffi.rs:60-68, cuda/vocab_fp8.cu:70-111) against the CPU
oracle bit for bit, and a whole model handed over in checkpoint layout (qwencore_b200/weights.py;
crates/qwc-engine/src/weights.rs:374-562, :609-659) that must decode exactly as the engine it was read from."""

import numpy as np
import pytest

from oracle import oracle
from qwencore_b200 import synth
from test_gpu_kernels import dev, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols,first_row", [(37, 5120, 0), (5, 5120, 11), (9, 1000, 3), (4, 1003, 0)],
                         ids=["vector", "vector_offset", "vector_narrow", "scalar_odd_width"])
def test_fp8_quantize_rows_is_bit_exact(cuda, built_library, rows, cols, first_row):
    from qwencore_b200 import abi, ops

    torch = cuda
    values = np.random.default_rng(rows).standard_normal((rows, cols)).astype(np.float32) * 0.05
    values[1] = 0.0                      # an empty row: scale 1, codes 0
    values[2, 7] = 300.0                 # one outlier sets the row's scale
    values[3, :8] = [1e-9, -1e-9, 2.0 ** -9, -(2.0 ** -10), 448.0, -448.0, 0.0, -0.0]
    bits = synth.bf16_bits(values)
    want_codes, want_scales = oracle.fp8_quantize_rows(bits, rows, cols)
    total = first_row + rows + 2
    codes = dev(torch, np.full((total, cols), 0xAA, dtype=np.uint8))
    scales = dev(torch, np.full(total, -1.0, dtype=np.float32))
    abi.check(abi.lib.qwc_fp8_quantize_rows(dev(torch, bits).data_ptr(), codes.data_ptr(), scales.data_ptr(), rows, cols,
                                            first_row, ops._stream()), "qwc_fp8_quantize_rows")
    torch.cuda.synchronize()
    got_codes, got_scales = host(codes), host(scales)
    assert np.array_equal(got_scales[first_row:first_row + rows], want_scales.reshape(-1))
    assert np.array_equal(got_codes[first_row:first_row + rows], want_codes.reshape(rows, cols))
    # nothing outside the chunk's rows is touched
    assert (got_codes[:first_row] == 0xAA).all() and (got_codes[first_row + rows:] == 0xAA).all()
    assert (got_scales[:first_row] == -1.0).all() and (got_scales[first_row + rows:] == -1.0).all()
    assert abi.lib.qwc_fp8_quantize_rows(None, codes.data_ptr(), scales.data_ptr(), rows, cols, 0,
                                         ops._stream()) == abi.CUDA_ERROR_INVALID_VALUE
    assert abi.lib.qwc_fp8_quantize_rows(codes.data_ptr(), codes.data_ptr(), scales.data_ptr(), rows, cols, -1,
                                         ops._stream()) == abi.CUDA_ERROR_INVALID_VALUE


def checkpoint_of(engine, rng):
    """An engine's weights taken apart into what a checkpoint holds (logical scales, unfused parts)."""
    from qwencore_b200 import weights

    c = engine.config
    layers = []
    for layer in range(c.num_layers):
        full = (layer + 1) % c.full_attention_interval == 0
        shapes = weights.layer_shapes(c, layer)
        fused = {"qkv": weights.ATTENTION_PARTS, "o": ("o_proj",)} if full else \
                {"in_proj": weights.MIXER_PARTS, "la_out": ("out_proj",)}
        fused.update({"gate": ("gate_proj",), "up": ("up_proj",), "down": ("down_proj",)})
        projections = {}
        for name, parts in fused.items():
            n, k = sum(shapes[p][0] for p in parts), shapes[parts[0]][1]
            packed = engine.read(f"{name}.packed", layer).reshape(n, k // 2)
            scales = oracle.unswizzle_block_scales(engine.read(f"{name}.scales", layer), n, k).reshape(n, k // 16)
            row = 0
            for part in parts:
                rows = shapes[part][0]
                projections[part] = weights.QuantLinear(packed[row:row + rows], scales[row:row + rows], 1.0)
                row += rows
        plain = {name: engine.read(tensor, layer, np.uint16) for name, (tensor, _) in weights.plain_names(c, layer).items()}
        layers.append((projections, plain))
    table = synth.bf16_bits(rng.standard_normal((c.vocab, c.hidden)).astype(np.float32) * 0.02)
    head = synth.bf16_bits(rng.standard_normal((c.vocab, c.hidden)).astype(np.float32) * 0.02)
    return layers, engine.read("final_norm", 0, np.uint16), table, head


def test_model_in_checkpoint_layout_loads_into_the_same_engine(cuda, built_library):
    from qwencore_b200 import abi, engine as E, weights
    from test_gpu_step import host_layout

    before = abi.get_shape()
    engines = []
    try:
        def make(seed):
            config = E.default_config(num_layers=4, vocab=8192, max_batch=2, max_context=256, kv_pool_blocks=48,
                                      state_slots=3, seed=seed, use_graph=1)
            engine = E.Engine(config)
            engines.append(engine)
            return engine

        source, target = make(5), make(6)
        layers, final_norm, table, head = checkpoint_of(source, np.random.default_rng(0))
        # the source takes the same vocabulary tables through the same path
        for engine in (source, target):
            stats = weights.load_model(engine, layers, final_norm, table, head) if engine is target else {
                "vocab_bytes": weights.load_vocab(engine, "embed", table) + weights.load_vocab(engine, "lm_head", head)}
        c = target.config
        assert stats["projections"] == 5 * c.num_layers and stats["vocab_bytes"] == 2 * c.vocab * (c.hidden + 4)
        want_codes, want_scales = oracle.fp8_quantize_rows(head, c.vocab, c.hidden)
        assert np.array_equal(target.read("lm_head"), want_codes.reshape(-1))
        assert np.array_equal(target.read("lm_head_scales", 0, np.float32), want_scales.reshape(-1))
        shapes_k = {"gate": c.hidden, "up": c.hidden, "down": c.intermediate, "qkv": c.hidden, "o": 24 * 256,
                    "in_proj": c.hidden, "la_out": c.delta_value_heads * 128}
        for layer in range(c.num_layers):
            full = (layer + 1) % c.full_attention_interval == 0
            for name in ["gate", "up", "down"] + (["qkv", "o"] if full else ["in_proj", "la_out"]):
                assert np.array_equal(target.read(f"{name}.packed", layer), source.read(f"{name}.packed", layer))
                n = target.read(f"{name}.packed", layer).size * 2 // shapes_k[name]
                # (the storage pads the rows to whole 128-row tiles; the synthetic fill leaves noise there)
                logical = [oracle.unswizzle_block_scales(e.read(f"{name}.scales", layer), n, shapes_k[name])
                           for e in (target, source)]
                assert np.array_equal(logical[0], logical[1]), f"{name} scales, layer {layer}"
                assert target.weight_global_scale(name, layer) == 1.0
        # recurrent state and KV pages are the engines' own (seeded differently): give the target the source's
        for layer in range(c.num_layers):
            full = (layer + 1) % c.full_attention_interval == 0
            for name in (("k_cache", "v_cache", "k_scale", "v_scale") if full else ("state", "state_scales", "conv_state")):
                target.write(name, layer, source.read(name, layer))
        tokens = np.array([11, 4000], dtype=np.uint32)
        sampled = []
        for engine in (source, target):
            cache = E.CacheManager(3, 48, 16)
            for seq, context in ((1, 40), (2, 17)):
                cache.admit(seq, context)
            engine.apply_edits(cache.drain_edits())
            out = []
            step_tokens = tokens.copy()
            for _ in range(3):
                for seq in (1, 2):
                    cache.append_token(seq)
                layout = host_layout(cache, [1, 2], 16, 3, (c.max_context + 15) // 16)
                step_tokens = engine.decode(layout["state_slots"], step_tokens, cache.drain_edits())
                out.append(step_tokens.tolist())
            sampled.append(out)
        assert sampled[0] == sampled[1]
        # a global scale is a launch argument: set on a loaded engine it changes the result of that projection
        target.set_weight_global_scale("down", 0, 2.0)
        assert target.weight_global_scale("down", 0) == 2.0
        with pytest.raises(abi.QwcError):
            target.set_weight_global_scale("qkv", 0, 1.0)  # layer 0 is a DeltaNet layer
        assert abi.lib.qwc_device_status() == 0
    finally:
        for engine in engines:
            engine.close()
        abi.configure(*before)


def test_model_loads_from_safetensors_files(cuda, built_library, tmp_path):
    """The file side (qwencore_b200/checkpoint.py): an engine's tensors written as a sharded safetensors
    checkpoint, validated against the architecture, and loaded into a second engine layer by layer with
    the file pages dropped behind the upload; every resident weight tensor then equals the source's."""
    from qwencore_b200 import abi, checkpoint, engine as E, weights

    before = abi.get_shape()
    engines = []
    try:
        def make(seed):
            config = E.default_config(num_layers=4, vocab=4096, max_batch=2, max_context=256, kv_pool_blocks=48,
                                      state_slots=3, seed=seed, use_graph=1)
            engines.append(E.Engine(config))
            return engines[-1]

        source, target = make(5), make(6)
        c = source.config
        layers, final_norm, table, head = checkpoint_of(source, np.random.default_rng(1))
        tensors, dtypes = checkpoint.checkpoint_tensors(c, layers, final_norm, table, head)
        checkpoint.write_checkpoint(str(tmp_path), tensors, dtypes, tensors_per_shard=48)
        del tensors, layers
        model = checkpoint.Checkpoint.open(str(tmp_path))
        problems, counted = model.validate(c)
        assert problems == [] and counted["quantized_linears"] == 3 * 8 + 7 and counted["unused_tensors"] == 0
        stats = checkpoint.load(target, model)
        assert stats["projections"] == 5 * c.num_layers
        assert stats["quantized_bytes"] >= counted["packed_bytes"] + counted["scale_bytes"]  # (+ swizzle padding)
        assert stats["vocab_bytes"] == 2 * c.vocab * (c.hidden + 4)
        weights.load_vocab(source, "embed", table)
        weights.load_vocab(source, "lm_head", head)
        for name in ("embed", "lm_head"):
            assert np.array_equal(target.read(name), source.read(name))
            assert np.array_equal(target.read(f"{name}_scales", 0, np.float32), source.read(f"{name}_scales", 0, np.float32))
        assert np.array_equal(target.read("final_norm", 0, np.uint16), source.read("final_norm", 0, np.uint16))
        shapes_k = {"gate": c.hidden, "up": c.hidden, "down": c.intermediate, "qkv": c.hidden, "o": 24 * 256,
                    "in_proj": c.hidden, "la_out": c.delta_value_heads * 128}
        for layer in range(c.num_layers):
            full = (layer + 1) % c.full_attention_interval == 0
            for name in ["gate", "up", "down"] + (["qkv", "o"] if full else ["in_proj", "la_out"]):
                packed = target.read(f"{name}.packed", layer)
                assert np.array_equal(packed, source.read(f"{name}.packed", layer)), (name, layer)
                n = packed.size * 2 // shapes_k[name]
                logical = [oracle.unswizzle_block_scales(e.read(f"{name}.scales", layer), n, shapes_k[name])
                           for e in (target, source)]
                assert np.array_equal(logical[0], logical[1]), (name, layer)
            for _, (tensor, _) in weights.plain_names(c, layer).items():
                assert np.array_equal(target.read(tensor, layer, np.uint16), source.read(tensor, layer, np.uint16))
    finally:
        for engine in engines:
            engine.close()
        abi.configure(*before)
