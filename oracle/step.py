"""CPU oracle of the whole decode step, composed from the per-op oracle functions in the
order of crates/qwc-engine/src/executor.rs:997-1112 with every inter-kernel rounding point
(bf16 activations between kernels, e4m3 KV pages, int8 state).

Test infrastructure: the parity tests compare the engine with `decode_step`, and the benchmark's
CPU legs time it on a reduced-depth synthetic model (`SyntheticModel`).  Nothing of the product
path imports this module."""

from types import SimpleNamespace

import numpy as np

from . import oracle

KEY_HEADS, DIM, Q_HEADS, KV_HEADS, HEAD_DIM = 16, 128, 24, 4, 256


def model_dimensions(model, cfg) -> None:
    """Derived widths of the hybrid model (crates/qwc-engine/src/weights.rs:50-60)."""
    model.cfg = cfg
    model.v_heads = cfg.delta_value_heads
    model.channels = 2 * KEY_HEADS * DIM + model.v_heads * DIM
    model.z_offset = model.channels
    model.a_offset = model.z_offset + model.v_heads * DIM
    model.b_offset = model.a_offset + model.v_heads
    model.mixer_width = model.b_offset + model.v_heads
    model.qkv_width = Q_HEADS * 2 * HEAD_DIM + 2 * KV_HEADS * HEAD_DIM
    model.max_blocks = (cfg.max_context + cfg.kv_page_size - 1) // cfg.kv_page_size


def project(weight, x_bits, batch):
    packed, scales, n, k = weight
    return oracle.bf16_from_f32(oracle.gemv_w4a16(packed, scales, 1.0, x_bits, n, k, batch))


def decode_step(model, layout, tokens, trace=None, head=True):
    """One step on the host copies (updated in place).  `layout` is oracle.layout_decode output.
    Returns (logits f32[batch, vocab], argmax u32[batch], final normed row bits).  When `trace` is a
    list, every layer appends (mixer output bits, residual bits after the MLP) to it.  With
    `head=False` the vocabulary head and the argmax are left out (logits and tokens are None)."""
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
        if trace is not None:
            trace.append((mixer_out.copy(), residual.copy()))
    if not head:
        return None, None, normed
    logits = oracle.fp8_lm_head(model.lm_head, model.lm_head_scales, normed, batch, c.hidden, c.vocab)
    return logits, oracle.argmax(logits, c.vocab, batch), normed


class SyntheticModel:
    """A host-side model of the benchmark's widths for timing the CPU path: `num_layers` layers in the
    3:1 DeltaNet : full-attention pattern, seeded random tensors.  One set of matrices per layer kind
    is shared by all layers of that kind (scalar CPU time does not depend on the values), the caches
    hold `contexts` tokens per row in consecutive pages."""

    def __init__(self, contexts, num_layers=4, interval=4, hidden=5120, intermediate=17408, vocab=151936,
                 v_heads=32, page=16, head_rows=None, seed=0):
        contexts = np.asarray(contexts, dtype=np.int64)
        rows = contexts.size
        blocks = (contexts + 1 + page - 1) // page
        cfg = SimpleNamespace(num_layers=num_layers, full_attention_interval=interval, hidden=hidden,
                              intermediate=intermediate, vocab=head_rows or vocab, delta_value_heads=v_heads,
                              kv_page_size=page, max_batch=rows, max_context=int(contexts.max()) + page,
                              kv_pool_blocks=int(blocks.sum()), state_slots=rows)
        model_dimensions(self, cfg)
        rng = np.random.default_rng(seed)

        def matrix(n, k):
            packed = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
            scales = rng.integers(0x08, 0x30, size=(n, k // 16), dtype=np.uint8)
            return packed, scales, n, k

        def norm(n, mean=0.0, std=0.02):
            return oracle.bf16_from_f32((mean + std * rng.standard_normal(n)).astype(np.float32))

        mlp = {"gate": matrix(intermediate, hidden), "up": matrix(intermediate, hidden),
               "down": matrix(hidden, intermediate)}
        linear = {"in_proj": matrix(self.mixer_width, hidden), "la_out": matrix(hidden, v_heads * DIM)}
        full = {"qkv": matrix(self.qkv_width, hidden), "o": matrix(hidden, Q_HEADS * HEAD_DIM)}
        cache_shape = (cfg.kv_pool_blocks, KV_HEADS, page, HEAD_DIM)
        self.layers = []
        for i in range(num_layers):
            is_full = (i + 1) % interval == 0
            layer = {"full": is_full, "input_norm": norm(hidden), "post_norm": norm(hidden), **mlp}
            if is_full:
                layer.update(full)
                layer["q_norm"], layer["k_norm"] = norm(HEAD_DIM, 0.0, 0.05), norm(HEAD_DIM, 0.0, 0.05)
                layer["k_scale"] = np.full(KV_HEADS, 1.0 / 64.0, np.float32)
                layer["v_scale"] = np.full(KV_HEADS, 1.0 / 64.0, np.float32)
                codes = rng.integers(0, 0x70, size=cache_shape, dtype=np.uint8)
                layer["k_cache"] = codes | (rng.integers(0, 2, size=cache_shape, dtype=np.uint8) << 7)
                layer["v_cache"] = np.roll(layer["k_cache"], 1, axis=0)
            else:
                layer.update(linear)
                layer["conv_weight"] = norm(self.channels * 4, 0.0, 0.3)
                layer["a_log"], layer["dt_bias"] = norm(v_heads, 0.0, 0.5), norm(v_heads, 0.0, 0.5)
                layer["out_norm"] = norm(DIM, 1.0, 0.05)
                layer["state"] = rng.integers(-127, 128, size=(rows, v_heads, DIM, DIM), dtype=np.int8)
                layer["state_scales"] = rng.uniform(0.0005, 0.003, size=(rows, v_heads, DIM)).astype(np.float32)
                layer["conv_state"] = rng.uniform(-1, 1, size=(rows, self.channels, 3)).astype(np.float32)
            self.layers.append(layer)
        self.final_norm = norm(hidden)
        head_rows = head_rows or vocab
        self.embed = rng.integers(0, 0x70, size=(head_rows, hidden), dtype=np.uint8)
        self.embed_scales = np.full(head_rows, 0.0002, np.float32)
        self.lm_head = self.embed
        self.lm_head_scales = self.embed_scales
        # rows in slot order, consecutive pages; one token appended for the step being timed
        seq_blocks = np.zeros((rows, self.max_blocks), np.uint32)
        first = np.concatenate([[0], np.cumsum(blocks)[:-1]])
        for row in range(rows):
            seq_blocks[row, :blocks[row]] = np.arange(first[row], first[row] + blocks[row], dtype=np.uint32)
        self.layout = oracle.layout_decode(np.arange(rows, dtype=np.uint32), (contexts + 1).astype(np.uint32),
                                           seq_blocks, blocks.astype(np.uint32), self.max_blocks, page)
        assert self.layout["status"] == 0
        self.tokens = rng.integers(0, head_rows, rows).astype(np.uint32)
