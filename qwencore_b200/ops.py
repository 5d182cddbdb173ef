"""Host-side mirror of the reference's per-op wrapper modules, over the C ABI.

Each function has the argument meaning and the error behaviour of its reference wrapper
(crates/qwc-cuda/src/{nvfp4,paged_attention,delta_net,rmsnorm,vocab,sampling}.rs): shapes are
asserted on the host before the call, the launcher's cudaError_t becomes an exception, and
the call is asynchronous on the current CUDA stream.  torch tensors are only device memory
here (`data_ptr()`), exactly what `DeviceBuffer<T>` is on the Rust side.
"""

from __future__ import annotations

import math

import torch

from . import abi

GROUP_SIZE = 16            # crates/qwc-cuda/src/nvfp4.rs:10
MAX_W4A16_BATCH = 32       # the reference stops at 8 (nvfp4.rs:15); north star asks for 32
NUM_ATTN_HEADS = 24
NUM_KV_HEADS = 4
ATTN_HEAD_DIM = 256
GQA_GROUP = 6
ROPE_DIM = 64
LA_NUM_K_HEADS = 16
LA_HEAD_DIM = 128
PACKED_PARTIAL_BYTES = 520  # crates/qwc-cuda/src/paged_attention.rs (max, sum f32 + 256 f16)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(tensor) -> int:
    return 0 if tensor is None else tensor.data_ptr()


def block_scale_storage_len(rows: int, in_features: int) -> int:
    """crates/qwc-cuda/src/nvfp4.rs:475-477"""
    return ((rows + 127) // 128 * 128) * ((in_features // GROUP_SIZE + 3) // 4 * 4)


class Linear:
    """An NVFP4 matrix resident on the device (crates/qwc-cuda/src/nvfp4.rs:84-166).

    `packed` u8[out, in/2] and `swizzled_scales` u8 in the 128x4 block-scale layout are
    device tensors; `weight_global_scale` is the checkpoint's divisor.
    """

    def __init__(self, packed: torch.Tensor, swizzled_scales: torch.Tensor, weight_global_scale: float,
                 out_features: int, in_features: int):
        assert out_features > 0 and in_features > 0 and in_features % 256 == 0
        assert packed.numel() == out_features * in_features // 2 and packed.dtype == torch.uint8
        assert swizzled_scales.numel() == block_scale_storage_len(out_features, in_features)
        assert math.isfinite(weight_global_scale) and weight_global_scale > 0.0
        self.packed = packed
        self.scales = swizzled_scales
        self.weight_global_scale = float(weight_global_scale)
        self.out_features = out_features
        self.in_features = in_features

    def forward_w4a16(self, x: torch.Tensor, out: torch.Tensor, batch: int) -> None:
        assert 1 <= batch <= MAX_W4A16_BATCH
        assert x.numel() >= batch * self.in_features and out.numel() >= batch * self.out_features
        abi.check(abi.lib.qwc_nvfp4_w4a16(_p(self.packed), _p(self.scales), _p(x), _p(out), self.out_features,
                                          self.in_features, batch, self.weight_global_scale, _stream()),
                  "qwc_nvfp4_w4a16")

    def weight_bytes(self) -> int:
        """DRAM traffic of the weights: nibbles + one scale byte per 16 (nvfp4.rs:213-215)."""
        return self.out_features * self.in_features // 2 + self.out_features * self.in_features // GROUP_SIZE


def swiglu_w4a16(gate: Linear, up: Linear, x: torch.Tensor, out: torch.Tensor, batch: int) -> None:
    """crates/qwc-cuda/src/nvfp4.rs:525-554"""
    assert gate.out_features == up.out_features and gate.in_features == up.in_features
    assert 1 <= batch <= MAX_W4A16_BATCH
    abi.check(abi.lib.qwc_nvfp4_swiglu_w4a16(_p(gate.packed), _p(gate.scales), _p(up.packed), _p(up.scales), _p(x),
                                             _p(out), gate.out_features, gate.in_features, batch,
                                             gate.weight_global_scale, up.weight_global_scale, _stream()),
              "qwc_nvfp4_swiglu_w4a16")


# ---- staged activations and the equal-share projection kernel (additive entry points) ----------

def padded_rows(batch: int) -> int:
    return 16 if batch <= 16 else 32


def staged_elements(batch: int, features: int) -> int:
    """f16 elements of a staged activation matrix: [features / 8][16 or 32 rows][8]."""
    return int(abi.lib.qwc_staged_activation_bytes(batch, features)) // 2


def new_staged(batch: int, features: int) -> torch.Tensor:
    return torch.zeros(staged_elements(batch, features), dtype=torch.float16, device="cuda")


def new_streamk_workspace() -> torch.Tensor:
    """Device memory through which split tiles are summed; cleared once, then left to the library."""
    workspace = torch.empty(int(abi.lib.qwc_streamk_workspace_bytes()), dtype=torch.uint8, device="cuda")
    abi.check(abi.lib.qwc_streamk_workspace_init(_p(workspace), _stream()), "qwc_streamk_workspace_init")
    return workspace


def stage_activations(x: torch.Tensor, staged: torch.Tensor, batch: int, features: int) -> None:
    assert x.numel() >= batch * features and staged.numel() >= staged_elements(batch, features)
    abi.check(abi.lib.qwc_stage_activations(_p(x), _p(staged), batch, features, _stream()), "qwc_stage_activations")


def unstage(staged: torch.Tensor, batch: int, features: int) -> torch.Tensor:
    """Staged f16 [features / 8][rows][8] back to rows [batch][features] (tests)."""
    rows = padded_rows(batch)
    return staged[: features * rows].reshape(features // 8, rows, 8).permute(1, 0, 2).reshape(rows, features)[:batch]


def w4a16_staged(linear: Linear, staged_x, out, staged_out, batch: int, workspace) -> None:
    abi.check(abi.lib.qwc_nvfp4_w4a16_staged(_p(linear.packed), _p(linear.scales), _p(staged_x), _p(out),
                                             _p(staged_out), linear.out_features, linear.in_features, batch,
                                             linear.weight_global_scale, _p(workspace), _stream()),
              "qwc_nvfp4_w4a16_staged")


def swiglu_w4a16_staged(gate: Linear, up: Linear, staged_x, out, staged_out, batch: int, workspace) -> None:
    assert gate.out_features == up.out_features and gate.in_features == up.in_features
    abi.check(abi.lib.qwc_nvfp4_swiglu_w4a16_staged(_p(gate.packed), _p(gate.scales), _p(up.packed), _p(up.scales),
                                                    _p(staged_x), _p(out), _p(staged_out), gate.out_features,
                                                    gate.in_features, batch, gate.weight_global_scale,
                                                    up.weight_global_scale, _p(workspace), _stream()),
              "qwc_nvfp4_swiglu_w4a16_staged")


def fp8_lm_head_staged(weights, row_scales, staged_x, logits, sampled, status_out, batch: int, hidden_size: int,
                       vocab: int, workspace) -> None:
    abi.check(abi.lib.qwc_fp8_lm_head_staged(_p(weights), _p(row_scales), _p(staged_x), _p(logits), _p(sampled),
                                             _p(status_out), batch, hidden_size, vocab, _p(workspace), _stream()),
              "qwc_fp8_lm_head_staged")


def split_count(linear: Linear) -> int:
    return int(abi.lib.qwc_nvfp4_split_count(linear.out_features, linear.in_features))


def w4a16_split(linear: Linear, staged_x, partial_sums, batch: int) -> None:
    """fp32 partial rows [split_count][batch][out] of a regular K split; the consumer sums them."""
    assert partial_sums.dtype == torch.float32
    assert partial_sums.numel() >= split_count(linear) * batch * linear.out_features
    abi.check(abi.lib.qwc_nvfp4_w4a16_split(_p(linear.packed), _p(linear.scales), _p(staged_x), _p(partial_sums),
                                            linear.out_features, linear.in_features, batch, _stream()),
              "qwc_nvfp4_w4a16_split")


def rmsnorm_split_staged(partial_sums, splits: int, weight_global_scale: float, projection_out, residual, weight,
                         out, staged_out, batch: int, hidden: int, epsilon: float = 1e-6) -> None:
    abi.check(abi.lib.qwc_rmsnorm_bf16_split_staged(_p(partial_sums), splits, weight_global_scale,
                                                    _p(projection_out), _p(residual), _p(weight), _p(out),
                                                    _p(staged_out), batch, hidden, epsilon, _stream()),
              "qwc_rmsnorm_bf16_split_staged")


def prefetch_next(first: Linear, second: Linear | None = None) -> None:
    """Names the projection that follows the next one launched from this thread (a hint for L2):
    one matrix, or the gate and up matrices of a SwiGLU pair."""
    if second is None:
        abi.check(abi.lib.qwc_nvfp4_prefetch_next(_p(first.packed), _p(first.scales), None, None, first.out_features,
                                                  first.in_features, 0), "qwc_nvfp4_prefetch_next")
    else:
        abi.check(abi.lib.qwc_nvfp4_prefetch_next(_p(first.packed), _p(first.scales), _p(second.packed),
                                                  _p(second.scales), first.out_features, first.in_features, 1),
                  "qwc_nvfp4_prefetch_next")


def packed_workspace_bytes(rows: int, partitions: int) -> int:
    return int(abi.lib.qwc_paged_attention_packed_workspace_bytes(rows, partitions))


def packed_partition_count(rows: int, context: int, sms: int = 148) -> int:
    """Upper bound on the context partitions of a decode row, which sizes the workspace.

    Same role as packed_partition_count (crates/qwc-cuda/src/paged_attention.rs:230-253), with a
    different meaning of the result: the kernel cuts the rows into tasks of equal size on the
    device (from the sum of the contexts it finds), and `partitions` only caps how many tasks one
    row may become.  Spans of at least 128 tokens; at most 4096 partial slots per head.
    """
    assert rows > 0 and context > 0
    want = max(1, (context + 127) // 128)
    most = max(8, 4096 // rows)
    return max(1, min(want, most))


def gated_packed(query, query_gate_projection, key_cache, value_cache, block_tables, context_lengths,
                 max_blocks_per_sequence: int, output, rows: int, row_base: int, partitions: int, workspace,
                 page_size: int, key_scales=None, value_scales=None, gate_stride: int = 0) -> None:
    """crates/qwc-cuda/src/paged_attention.rs:373-421 (PackedShape::Rows)."""
    end = row_base + rows
    assert query.numel() >= end * NUM_ATTN_HEADS * ATTN_HEAD_DIM
    assert output.numel() >= end * NUM_ATTN_HEADS * ATTN_HEAD_DIM
    assert context_lengths.numel() >= end and block_tables.numel() >= end * max_blocks_per_sequence
    workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    abi.check(abi.lib.qwc_paged_attention_packed_fp8_scaled(
        _p(query), _p(query_gate_projection), _p(key_cache), _p(value_cache), _p(block_tables), _p(context_lengths),
        _p(key_scales), _p(value_scales), _p(output), _p(workspace), workspace_bytes, rows, row_base,
        max_blocks_per_sequence, page_size, gate_stride, partitions, 1.0 / math.sqrt(ATTN_HEAD_DIM), _stream()),
        "qwc_paged_attention_packed_fp8_scaled")


def gated_packed_noalloc(query, query_gate_projection, key_cache, value_cache, block_tables, context_lengths,
                         max_blocks_per_sequence: int, output, rows: int, row_base: int, partitions: int,
                         page_size: int, key_scales=None, value_scales=None, gate_stride: int = 0) -> None:
    """Packed attention on the library's built-in scratch, for callers that cannot allocate a workspace.

    rows * partitions must not exceed `qwc_paged_attention_packed_noalloc_max_pairs()`; calls share
    the scratch, so overlapping calls on different streams race.  Make the first call on a device
    outside any stream capture."""
    abi.check(abi.lib.qwc_paged_attention_packed_fp8_noalloc(
        _p(query), _p(query_gate_projection), _p(key_cache), _p(value_cache), _p(block_tables), _p(context_lengths),
        _p(key_scales), _p(value_scales), _p(output), rows, row_base, max_blocks_per_sequence, page_size, gate_stride,
        partitions, 1.0 / math.sqrt(ATTN_HEAD_DIM), _stream()), "qwc_paged_attention_packed_fp8_noalloc")


def gated_packed_legacy(query, query_gate_projection, key_cache, value_cache, block_tables, context_lengths,
                        max_blocks_per_sequence: int, output, rows: int, row_base: int, partitions: int,
                        workspace, tile_size: int = GQA_GROUP) -> None:
    """The reference-signature entry point; page size comes from qwc_configure."""
    workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    abi.check(abi.lib.qwc_paged_attention_packed_fp8(
        _p(query), _p(query_gate_projection), _p(key_cache), _p(value_cache), _p(block_tables), _p(context_lengths),
        _p(output), _p(workspace), workspace_bytes, rows, row_base, max_blocks_per_sequence, tile_size, partitions,
        1.0 / math.sqrt(ATTN_HEAD_DIM), _stream()), "qwc_paged_attention_packed_fp8")


def delta_decode_slots_packed(state, state_scales, state_slots, q, k, v, alpha, beta, kq, out, state_capacity: int,
                              batch: int) -> None:
    """crates/qwc-cuda/src/delta_net.rs:617-650"""
    assert state.dtype == torch.int8 and state_scales.dtype == torch.float32
    abi.check(abi.lib.qwc_delta_decode_int8(_p(state), _p(state_scales), _p(state_slots), _p(q), _p(k), _p(v),
                                            _p(alpha), _p(beta), _p(kq), _p(out), state_capacity, batch, _stream()),
              "qwc_delta_decode_int8")


def delta_prepare_decode(mixed, a_offset: int, b_offset: int, conv_weight, a_log, dt_bias, conv_state, state_slots,
                         query, key, value, alpha, beta, kq, state_capacity: int, batch: int, mixed_stride: int) -> None:
    """crates/qwc-cuda/src/delta_net.rs prepare_decode; a/b are strided views of the mixed row."""
    base = mixed.data_ptr()
    abi.check(abi.lib.qwc_delta_prepare_decode(base, base + 2 * a_offset, base + 2 * b_offset, _p(conv_weight),
                                               _p(a_log), _p(dt_bias), _p(conv_state), _p(state_slots), _p(query),
                                               _p(key), _p(value), _p(alpha), _p(beta), _p(kq), state_capacity, batch,
                                               mixed_stride, mixed_stride, _stream()), "qwc_delta_prepare_decode")


def delta_gated_rmsnorm(values, mixed, z_offset: int, weight, output, batch: int, mixed_stride: int,
                        epsilon: float = 1e-6) -> None:
    abi.check(abi.lib.qwc_delta_gated_rmsnorm(_p(values), mixed.data_ptr() + 2 * z_offset, _p(weight), _p(output),
                                              batch, epsilon, mixed_stride, _stream()), "qwc_delta_gated_rmsnorm")


def prepare_attention_decode(query_gate, key_projection, value_projection, q_norm_weight, k_norm_weight, cosine,
                             sine, physical_blocks, block_offsets, query, key_cache, value_cache, batch: int,
                             page_size: int, query_stride: int, key_stride: int, value_stride: int,
                             key_scales=None, value_scales=None, epsilon: float = 1e-6) -> None:
    abi.check(abi.lib.qwc_prepare_attention_decode_fp8_scaled(
        _p(query_gate), _p(key_projection), _p(value_projection), _p(q_norm_weight), _p(k_norm_weight), _p(cosine),
        _p(sine), _p(physical_blocks), _p(block_offsets), _p(key_scales), _p(value_scales), _p(query), _p(key_cache),
        _p(value_cache), batch, page_size, query_stride, key_stride, value_stride, epsilon, _stream()),
        "qwc_prepare_attention_decode_fp8_scaled")


def rmsnorm_bf16(x, residual, weight, out, batch: int, hidden: int, epsilon: float = 1e-6) -> None:
    """crates/qwc-cuda/src/rmsnorm.rs forward_bf16"""
    abi.check(abi.lib.qwc_rmsnorm_bf16(_p(x), _p(residual), _p(weight), _p(out), batch, hidden, epsilon, _stream()),
              "qwc_rmsnorm_bf16")


def fp8_embedding_gather(table, row_scales, token_ids, out, batch: int, cols: int, vocab: int) -> None:
    abi.check(abi.lib.qwc_fp8_embedding_gather(_p(table), _p(row_scales), _p(token_ids), _p(out), batch, cols, vocab,
                                               _stream()), "qwc_fp8_embedding_gather")


def fp8_lm_head(weights, row_scales, hidden, logits, batch: int, hidden_size: int, vocab: int) -> None:
    abi.check(abi.lib.qwc_fp8_lm_head_batched(_p(weights), _p(row_scales), _p(hidden), _p(logits), batch, hidden_size,
                                              vocab, _stream()), "qwc_fp8_lm_head_batched")


def argmax(logits, partial_values, partial_indices, output, vocab: int, batch: int, parts: int = 256) -> None:
    abi.check(abi.lib.qwc_argmax(_p(logits), _p(partial_values), _p(partial_indices), _p(output), vocab, batch, parts,
                                 _stream()), "qwc_argmax")


def page_table_apply(seq_tokens, seq_blocks, edits, count: int, capacity: int, max_blocks: int) -> None:
    abi.check(abi.lib.qwc_page_table_apply(_p(seq_tokens), _p(seq_blocks), _p(edits), count, capacity, max_blocks,
                                           _stream()), "qwc_page_table_apply")


def pack_decode_batch(row_slots, slot_active, seq_tokens, seq_blocks, rope_table, max_positions: int, row_count,
                      state_slots, positions, context_lengths, physical_blocks, block_offsets, block_tables,
                      block_table_offsets, block_ids, cosine, sine, status, rows: int, capacity: int, max_blocks: int,
                      page_size: int) -> None:
    abi.check(abi.lib.qwc_pack_decode_batch(
        _p(row_slots), _p(slot_active), _p(seq_tokens), _p(seq_blocks), _p(rope_table), max_positions, _p(row_count),
        _p(state_slots), _p(positions), _p(context_lengths), _p(physical_blocks), _p(block_offsets), _p(block_tables),
        _p(block_table_offsets), _p(block_ids), _p(cosine), _p(sine), _p(status), rows, capacity, max_blocks,
        page_size, _stream()), "qwc_pack_decode_batch")
