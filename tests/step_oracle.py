"""The engine's weights and caches copied to the host, for the CPU oracle of the whole step
(oracle/step.py).  Test infrastructure only."""

import numpy as np

from oracle import oracle
from oracle.step import DIM, HEAD_DIM, KEY_HEADS, KV_HEADS, Q_HEADS, decode_step, model_dimensions, project  # noqa: F401


class HostModel:
    """Weights and caches of an engine, copied to the host."""

    def __init__(self, engine):
        c = engine.config
        model_dimensions(self, c)
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
