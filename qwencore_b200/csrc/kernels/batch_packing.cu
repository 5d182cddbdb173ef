// Device-side construction of the ragged decode batch.
//
// The reference builds these arrays on the host every step and uploads them with eight
// blocking copies: BatchLayout::build (crates/qwc-runtime/src/layout.rs:54-152) followed by
// Executor::upload_layout_decode (crates/qwc-engine/src/executor.rs:1939-1990).  Here the
// page table and token counts live on the device, the host only sends the edits a step
// makes (a few words), and two small kernels derive everything the step reads:
//   kernel 1 (one CTA): slot compaction by prefix sum (optional), validation, per-row
//     scalars, exclusive scan of the page counts (the CSR offsets);
//   kernel 2 (one CTA per row): dense block-table row, CSR block ids, RoPE row gather.
// All outputs are integers or table lookups, so they are bit-exact against the host
// statement.

#include "common.cuh"

#include "../../../include/qwc_abi.h"

namespace qwc {
namespace {

constexpr int kThreads = 256;

// Inclusive scan of one value per thread across the CTA; returns the exclusive prefix
// and leaves the CTA total in *total_out (same value for every thread).
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t value, uint32_t* warp_totals, uint32_t* total_out) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    uint32_t inclusive = value;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t other = __shfl_up_sync(0xffffffffu, inclusive, off);
        if (lane >= off) {
            inclusive += other;
        }
    }
    __syncthreads();
    if (lane == 31) {
        warp_totals[warp] = inclusive;
    }
    __syncthreads();
    uint32_t warp_prefix = 0;
    uint32_t total = 0;
    for (int w = 0; w < kThreads / 32; ++w) {
        const uint32_t t = warp_totals[w];
        if (w < warp) {
            warp_prefix += t;
        }
        total += t;
    }
    *total_out = total;
    return warp_prefix + inclusive - value;
}

__global__ void __launch_bounds__(kThreads) page_table_apply_kernel(uint32_t* __restrict__ seq_tokens,
                                                                    uint32_t* __restrict__ seq_blocks,
                                                                    const qwc_table_edit* __restrict__ edits,
                                                                    int count, int capacity, int max_blocks) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) {
        return;
    }
    const qwc_table_edit e = edits[i];
    if (e.slot >= static_cast<uint32_t>(capacity)) {
        return;
    }
    if (e.kind == 0) {
        if (e.index < static_cast<uint32_t>(max_blocks)) {
            seq_blocks[static_cast<size_t>(e.slot) * max_blocks + e.index] = e.value;
        }
    } else if (e.kind == 1) {
        seq_tokens[e.slot] = e.value;
    } else if (e.kind == 2) {
        atomicAdd(&seq_tokens[e.slot], e.value);
    }
}

__global__ void __launch_bounds__(kThreads) pack_rows_kernel(
    const uint32_t* __restrict__ row_slots, const uint8_t* __restrict__ slot_active,
    const uint32_t* __restrict__ seq_tokens, uint32_t* __restrict__ row_count, uint32_t* __restrict__ state_slots,
    uint32_t* __restrict__ positions, uint32_t* __restrict__ context_lengths,
    const uint32_t* __restrict__ seq_blocks, uint32_t* __restrict__ physical_blocks,
    uint32_t* __restrict__ block_offsets, uint32_t* __restrict__ block_table_offsets, uint32_t* __restrict__ status,
    int rows, int capacity, int max_blocks, int page_size, int max_positions) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ uint32_t warp_totals[kThreads / 32];
    __shared__ uint32_t carry;
    __shared__ uint32_t error;
    __shared__ uint32_t live_rows;
    extern __shared__ uint32_t seen[];  // one bit per slot

    if (threadIdx.x == 0) {
        carry = 0;
        error = 0;
        live_rows = static_cast<uint32_t>(rows);
    }
    for (int i = threadIdx.x; i < (capacity + 31) / 32; i += kThreads) {
        seen[i] = 0;
    }
    __syncthreads();

    // Optional compaction: rows are the active slots in ascending order.
    if (row_slots == nullptr) {
        for (int base = 0; base < capacity; base += kThreads) {
            const int slot = base + threadIdx.x;
            const uint32_t flag = (slot < capacity && slot_active[slot] != 0) ? 1u : 0u;
            uint32_t total;
            const uint32_t before = block_exclusive_scan(flag, warp_totals, &total);
            const uint32_t index = carry + before;
            if (flag && index < static_cast<uint32_t>(rows)) {
                state_slots[index] = static_cast<uint32_t>(slot);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                carry += total;
            }
            __syncthreads();
        }
        if (threadIdx.x == 0) {
            live_rows = carry < static_cast<uint32_t>(rows) ? carry : static_cast<uint32_t>(rows);
            carry = 0;
        }
        __syncthreads();
    } else {
        for (int row = threadIdx.x; row < rows; row += kThreads) {
            state_slots[row] = row_slots[row];
        }
        __syncthreads();
    }
    const int live = static_cast<int>(live_rows);
    if (threadIdx.x == 0 && row_count != nullptr) {
        *row_count = live_rows;
    }

    // Per-row scalars and the exclusive scan of page counts.
    if (threadIdx.x == 0) {
        block_table_offsets[0] = 0;
    }
    for (int base = 0; base < rows; base += kThreads) {
        const int row = base + threadIdx.x;
        uint32_t blocks = 0;
        if (row < rows) {
            uint32_t slot = 0, tokens = 0, position = 0, physical = 0, offset = 0;
            if (row < live) {
                slot = state_slots[row];
                if (slot >= static_cast<uint32_t>(capacity) || seq_tokens[slot] == 0) {
                    atomicCAS(&error, 0u, 1u);
                    slot = 0;
                } else {
                    const uint32_t bit = 1u << (slot & 31);
                    if (atomicOr(&seen[slot >> 5], bit) & bit) {
                        atomicCAS(&error, 0u, 2u);
                    }
                    tokens = seq_tokens[slot];
                    position = tokens - 1;
                    blocks = (tokens + page_size - 1) / page_size;
                    if (blocks > static_cast<uint32_t>(max_blocks)) {
                        atomicCAS(&error, 0u, 4u);
                        blocks = 0;
                        tokens = 0;
                        position = 0;
                    } else {
                        if (position >= static_cast<uint32_t>(max_positions)) {
                            atomicCAS(&error, 0u, 8u);
                        }
                        physical = seq_blocks[static_cast<size_t>(slot) * max_blocks + position / page_size];
                        offset = position % page_size;
                    }
                }
            }
            state_slots[row] = slot;
            positions[row] = position;
            context_lengths[row] = tokens;
            physical_blocks[row] = physical;
            block_offsets[row] = offset;
        }
        uint32_t total;
        const uint32_t before = block_exclusive_scan(blocks, warp_totals, &total);
        if (row < rows) {
            block_table_offsets[row + 1] = carry + before + blocks;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            carry += total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        *status = error;
    }
}

__global__ void __launch_bounds__(kThreads) pack_tables_kernel(
    const uint32_t* __restrict__ state_slots, const uint32_t* __restrict__ positions,
    const uint32_t* __restrict__ context_lengths, const uint32_t* __restrict__ seq_blocks,
    const uint32_t* __restrict__ block_table_offsets, const __nv_bfloat16* __restrict__ rope_table,
    uint32_t* __restrict__ block_tables, uint32_t* __restrict__ block_ids, __nv_bfloat16* __restrict__ cosine,
    __nv_bfloat16* __restrict__ sine, int max_blocks, int page_size, int max_positions) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    const uint32_t slot = state_slots[row];
    const uint32_t context = context_lengths[row];
    const uint32_t blocks = (context + page_size - 1) / page_size;
    const uint32_t* source = seq_blocks + static_cast<size_t>(slot) * max_blocks;
    uint32_t* table = block_tables + static_cast<size_t>(row) * max_blocks;
    const uint32_t csr_begin = block_table_offsets[row];
    for (int i = threadIdx.x; i < max_blocks; i += kThreads) {
        const uint32_t id = static_cast<uint32_t>(i) < blocks ? source[i] : 0u;
        table[i] = id;
        if (block_ids != nullptr && static_cast<uint32_t>(i) < blocks) {
            block_ids[csr_begin + i] = id;
        }
    }
    if (threadIdx.x < 2 * kRopeDim && cosine != nullptr) {
        const uint32_t position = positions[row] < static_cast<uint32_t>(max_positions) ? positions[row] : 0u;
        const int which = threadIdx.x / kRopeDim;  // 0 cosine, 1 sine
        const int d = threadIdx.x % kRopeDim;
        const __nv_bfloat16 value = rope_table[(static_cast<size_t>(position) * 2 + which) * kRopeDim + d];
        (which == 0 ? cosine : sine)[static_cast<size_t>(row) * kRopeDim + d] = value;
    }
}

}  // namespace
}  // namespace qwc

using namespace qwc;

extern "C" int qwc_page_table_apply(uint32_t* seq_tokens, uint32_t* seq_blocks, const qwc_table_edit* edits,
                                    int count, int capacity, int max_blocks, qwc_stream stream_handle) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    if (seq_tokens == nullptr || seq_blocks == nullptr || capacity <= 0 || max_blocks <= 0 || count < 0 ||
        (count > 0 && edits == nullptr)) {
        return cudaErrorInvalidValue;
    }
    if (count == 0) {
        return cudaSuccess;
    }
    return qwc::launch_chained(page_table_apply_kernel, dim3((count + kThreads - 1) / kThreads), dim3(kThreads), 0, stream, 
        seq_tokens, seq_blocks, edits, count, capacity, max_blocks);
}

extern "C" int qwc_pack_decode_batch(const uint32_t* row_slots, const uint8_t* slot_active,
                                     const uint32_t* seq_tokens, const uint32_t* seq_blocks, const void* rope_table,
                                     int max_positions, uint32_t* row_count, uint32_t* state_slots,
                                     uint32_t* positions, uint32_t* context_lengths, uint32_t* physical_blocks,
                                     uint32_t* block_offsets, uint32_t* block_tables,
                                     uint32_t* block_table_offsets, uint32_t* block_ids, void* cosine, void* sine,
                                     uint32_t* status, int rows, int capacity, int max_blocks, int page_size,
                                     qwc_stream stream_handle) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    if ((row_slots == nullptr && slot_active == nullptr) || seq_tokens == nullptr || seq_blocks == nullptr ||
        state_slots == nullptr || positions == nullptr || context_lengths == nullptr ||
        physical_blocks == nullptr || block_offsets == nullptr || block_tables == nullptr ||
        block_table_offsets == nullptr || status == nullptr || rows <= 0 || rows > kMaxStepRows || capacity <= 0 ||
        capacity > (1 << 20) || max_blocks <= 0 || (page_size != 16 && page_size != 64) ||
        ((cosine != nullptr || sine != nullptr) && (rope_table == nullptr || cosine == nullptr || sine == nullptr ||
                                                     max_positions <= 0))) {
        return cudaErrorInvalidValue;
    }
    const size_t seen_bytes = static_cast<size_t>((capacity + 31) / 32) * sizeof(uint32_t);
    if (seen_bytes > 40 * 1024) {
        return cudaErrorInvalidValue;
    }
    cudaError_t launched = qwc::launch_chained(pack_rows_kernel, dim3(1), dim3(kThreads), seen_bytes, stream, 
        row_slots, slot_active, seq_tokens, row_count, state_slots, positions, context_lengths, seq_blocks,
        physical_blocks, block_offsets, block_table_offsets, status, rows, capacity, max_blocks, page_size,
        max_positions > 0 ? max_positions : 0x7fffffff);
    if (launched != cudaSuccess) {
        return launched;
    }
    return qwc::launch_chained(pack_tables_kernel, dim3(rows), dim3(kThreads), 0, stream, 
        state_slots, positions, context_lengths, seq_blocks, block_table_offsets,
        static_cast<const __nv_bfloat16*>(rope_table), block_tables, block_ids,
        static_cast<__nv_bfloat16*>(cosine), static_cast<__nv_bfloat16*>(sine), max_blocks, page_size,
        max_positions > 0 ? max_positions : 0x7fffffff);
}
