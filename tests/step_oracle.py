"""CPU oracle of the whole decode step, composed from the per-op oracle functions in the
order of crates/qwc-engine/src/executor.rs:997-1112 with every inter-kernel rounding point
(bf16 activations between kernels, e4m3 KV pages, int8 state).  Test infrastructure only."""

import numpy as np

from oracle import oracle
from qwencore_b200 import synth

KEY_HEADS, DIM, Q_HEADS, KV_HEADS, HEAD_DIM = 16, 128, 24, 4, 256


class HostModel:
    """Weights and caches of an engine, copied to the host."""

    def __init__(self, engine):
        c = engine.config
        self.cfg = c
        self.v_heads = c.delta_value_heads
        self.channels = 2 * KEY_HEADS * DIM + self.v_heads * DIM
        self.z_offset = self.channels
        self.a_offset = self.z_offset + self.v_heads * DIM
        self.b_offset = self.a_offset + self.v_heads
        self.mixer_width = self.b_offset + self.v_heads
        self.qkv_width = Q_HEADS * 2 * HEAD_DIM + 2 * KV_HEADS * HEAD_DIM
        self.max_blocks = (c.max_context + c.kv_page_size - 1) // c.kv_page_size
        self.layers = []
        for i in range(c.num_layers):
            full = (i + 1) % c.full_attention_interval == 0
            layer = {"full": full}
            for name in ("input_norm", "post_norm"):
                layer[name] = engine.read(name, i, np.uint16)
            shapes = {"gate": (c.intermediate, c.hidden), "up": (c.intermediate, c.hidden),
                      "down": (c.hidden, c.intermediate)}
            if full:
                shapes.update({"qkv": (self.qkv_width, c.hidden), "o": (c.hidden, Q_HEADS * HEAD_DIM)})
            else:
                shapes.update({"in_proj": (self.mixer_width, c.hidden), "la_out": (c.hidden, self.v_heads * DIM)})
            for name, (n, k) in shapes.items():
                packed = engine.read(f"{name}.packed", i).reshape(n, k // 2)
                scales = oracle.unswizzle_block_scales(engine.read(f"{name}.scales", i), n, k).reshape(n, k // 16)
                layer[name] = (packed, scales, n, k)
            if full:
                for name in ("q_norm", "k_norm"):
                    layer[name] = engine.read(name, i, np.uint16)
                layer["k_scale"] = engine.read("k_scale", i, np.float32)
                layer["v_scale"] = engine.read("v_scale", i, np.float32)
                shape = (c.kv_pool_blocks, KV_HEADS, c.kv_page_size, HEAD_DIM)
                layer["k_cache"] = engine.read("k_cache", i).reshape(shape)
                layer["v_cache"] = engine.read("v_cache", i).reshape(shape)
            else:
                layer["conv_weight"] = engine.read("conv_weight", i, np.uint16)
                layer["a_log"] = engine.read("a_log", i, np.uint16)
                layer["dt_bias"] = engine.read("dt_bias", i, np.uint16)
                layer["out_norm"] = engine.read("out_norm", i, np.uint16)
                layer["state"] = engine.read("state", i, np.int8).reshape(c.state_slots, self.v_heads, DIM, DIM)
                layer["state_scales"] = engine.read("state_scales", i, np.float32).reshape(c.state_slots,
                                                                                          self.v_heads, DIM)
                layer["conv_state"] = engine.read("conv_state", i, np.float32).reshape(c.state_slots,
                                                                                      self.channels, 3)
            self.layers.append(layer)
        self.final_norm = engine.read("final_norm", 0, np.uint16)
        self.embed = engine.read("embed").reshape(c.vocab, c.hidden)
        self.embed_scales = engine.read("embed_scales", 0, np.float32)
        self.lm_head = engine.read("lm_head").reshape(c.vocab, c.hidden)
        self.lm_head_scales = engine.read("lm_head_scales", 0, np.float32)


def project(weight, x_bits, batch):
    packed, scales, n, k = weight
    return oracle.bf16_from_f32(oracle.gemv_w4a16(packed, scales, 1.0, x_bits, n, k, batch))


def decode_step(model: HostModel, layout, tokens):
    """One step on the host copies (updated in place).  `layout` is oracle.layout_decode output.
    Returns (logits f32[batch, vocab], argmax u32[batch])."""
    c = model.cfg
    batch = len(tokens)
    slots = layout["state_slots"]
    cosine, sine = oracle.rope_rows(layout["positions"])
    residual = oracle.fp8_embedding_gather(model.embed, model.embed_scales, tokens, c.hidden, c.vocab)
    normed = oracle.rmsnorm_bf16(residual, None, model.layers[0]["input_norm"], batch, c.hidden)
    for index, layer in enumerate(model.layers):
        if not layer["full"]:
            mixed = project(layer["in_proj"], normed, batch)
            base = mixed.ctypes.data
            q, k, v, alpha, beta, kq = oracle.delta_prepare_decode(
                mixed, base + 2 * model.a_offset, base + 2 * model.b_offset, layer["conv_weight"], layer["a_log"],
                layer["dt_bias"], layer["conv_state"], slots, batch, model.mixer_width, model.mixer_width, KEY_HEADS,
                model.v_heads)
            out = oracle.delta_decode_int8(layer["state"], layer["state_scales"], slots, q, k, v, alpha, beta, kq,
                                           batch, model.v_heads)
            gated = oracle.delta_gated_rmsnorm(out, base + 2 * model.z_offset, layer["out_norm"], batch,
                                               model.v_heads, model.mixer_width)
            mixer_out = project(layer["la_out"], gated.reshape(batch, -1), batch)
        else:
            qkv = project(layer["qkv"], normed, batch)
            q_width = Q_HEADS * 2 * HEAD_DIM
            query_gate = np.ascontiguousarray(qkv[:, :q_width])
            key_proj = np.ascontiguousarray(qkv[:, q_width:q_width + KV_HEADS * HEAD_DIM])
            value_proj = np.ascontiguousarray(qkv[:, q_width + KV_HEADS * HEAD_DIM:])
            query = oracle.prepare_attention_decode_fp8(
                query_gate, key_proj, value_proj, layer["q_norm"], layer["k_norm"], cosine, sine,
                layout["physical_blocks"], layout["block_offsets"], layer["k_cache"], layer["v_cache"], batch,
                c.kv_page_size, k_scale=layer["k_scale"], v_scale=layer["v_scale"])
            attended = oracle.paged_attention_fp8(
                query, query_gate, layer["k_cache"], layer["v_cache"], layout["block_tables"],
                layout["context_lengths"], model.max_blocks, batch, page_size=c.kv_page_size,
                k_scale=layer["k_scale"], v_scale=layer["v_scale"])
            mixer_out = project(layer["o"], oracle.bf16_from_f32(attended).reshape(batch, -1), batch)
        normed = oracle.rmsnorm_bf16(mixer_out, residual, layer["post_norm"], batch, c.hidden)
        gate = oracle.gemv_w4a16(layer["gate"][0], layer["gate"][1], 1.0, normed, c.intermediate, c.hidden, batch)
        up = oracle.gemv_w4a16(layer["up"][0], layer["up"][1], 1.0, normed, c.intermediate, c.hidden, batch)
        hidden = oracle.bf16_from_f32(oracle.swiglu_combine(gate, up))
        mlp_out = project(layer["down"], hidden, batch)
        next_norm = model.layers[index + 1]["input_norm"] if index + 1 < len(model.layers) else model.final_norm
        normed = oracle.rmsnorm_bf16(mlp_out, residual, next_norm, batch, c.hidden)
    logits = oracle.fp8_lm_head(model.lm_head, model.lm_head_scales, normed, batch, c.hidden, c.vocab)
    return logits, oracle.argmax(logits, c.vocab, batch), normed
