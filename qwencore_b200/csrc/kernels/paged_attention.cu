// Packed-GQA paged attention over an e4m3 KV cache for ragged decode rows.
//
// Replaces crates/qwc-cuda/cuda/paged_attention.cu:1913-1958 (qwc_paged_attention_packed_fp8)
// for decode rows (tile of six packed query heads per KV head).  Semantics follow the
// reference: Q, K, V and P enter the tensor cores as f16 (e4m3 -> f16 is exact), softmax
// and accumulation in fp32, optional sigmoid output gate, split-context partials merged
// by a second kernel (cuda/paged_attention.cu:1464-1574,1736-1823).
//
// The op reads every K and V byte of the row's context once and nothing else of size,
// so it is HBM-bound.  Layout for sm_100a:
//   * grid (kv head, row, partition); the partition's span is cut on the device from
//     the row's real context, so the launch shape depends only on capacity-level values
//     and the step stays capturable in a CUDA graph;
//   * KV moves in 4 KiB units (16 tokens x 256 B of one kv head: a whole 16-token page,
//     or a quarter of a 64-token page) by bulk-async copies (TMA 1-D) into a 3-stage
//     ring of 8 units (128 tokens, 64 KiB of K+V per stage) guarded by mbarriers -
//     up to 192 KiB in flight per SM and no registers spent on loads;
//   * each unit lands 16 bytes further than a multiple of 4 KiB.  An MMA column tile is
//     "token j of 8 different units", so the eight rows an ldmatrix or a fragment load
//     touches fall in eight different 16-byte bank groups: conflict-free without a
//     swizzled tensor map;
//   * QK^T: the six heads of the group are rows of one m16 tile, e4m3 pairs are widened
//     by the hardware converter straight into B fragments; PV: V is transposed on the
//     fly by ldmatrix.trans on byte pairs and a byte permute; the four warps split the
//     tokens for QK^T and the 256 output dims for PV, exchanging P through 2 KiB of
//     shared memory.
//
// Cache memory must hold finite e4m3 codes in every allocated page (a zero-initialised
// pool, as the reference allocates it): positions past the context are masked by
// zero probabilities, not skipped.

#include "common.cuh"

namespace qwc {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = 4;
constexpr int kUnitTokens = 16;
constexpr int kUnitBytes = kUnitTokens * kHeadDim;  // 4096
constexpr int kUnitPitch = kUnitBytes + 16;         // staggered landing offset
constexpr int kStageUnits = 8;
constexpr int kStages = 3;
constexpr int kStageBytes = kStageUnits * kUnitPitch;    // per K or V
constexpr int kPartialFloats = 2;
constexpr size_t kPartialBytes = 2 * sizeof(float) + kHeadDim * sizeof(__half);  // 520
constexpr float kLog2e = 1.4426950408889634f;

struct Smem {
    uint8_t k[kStages][kStageBytes];
    uint8_t v[kStages][kStageBytes];
    uint2 p[kStageUnits][32];       // P as A fragments: [pv k-step][lane]
    float warp_max[kWarps][8];
    float warp_sum[kWarps][8];
    uint64_t full[kStages];
    int failed;
};

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(address));
}

// low / high 16 bits of a word holding two e4m3 pairs -> two f16x2
__device__ __forceinline__ void cvt_e4m3x4(uint32_t word, uint32_t& lo, uint32_t& hi) {
    asm("{\n"
        ".reg .b16 a, b;\n"
        "mov.b32 {a, b}, %2;\n"
        "cvt.rn.f16x2.e4m3x2 %0, a;\n"
        "cvt.rn.f16x2.e4m3x2 %1, b;\n"
        "}\n"
        : "=r"(lo), "=r"(hi)
        : "r"(word));
}

template <bool kSplit>
__global__ void __launch_bounds__(kThreads, 1) paged_attention_packed_kernel(
    const __nv_bfloat16* __restrict__ query, const __nv_bfloat16* __restrict__ query_gate_projection,
    const uint8_t* __restrict__ key_cache, const uint8_t* __restrict__ value_cache,
    const uint32_t* __restrict__ block_tables, const uint32_t* __restrict__ context_lengths,
    const float* __restrict__ key_scales, const float* __restrict__ value_scales,
    __nv_bfloat16* __restrict__ output, float* __restrict__ partial_stats, __half* __restrict__ partial_out,
    int max_blocks, int row_base, int page_size, int gate_stride, float softmax_scale, int* status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);

    if (status_is_set(status)) {
        return;
    }
    const int kv_head = blockIdx.x;
    const int row = row_base + blockIdx.y;
    const int part = blockIdx.z;
    const int partitions = gridDim.z;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;

    const int context = static_cast<int>(context_lengths[row]);
    const int total_units = (context + kUnitTokens - 1) / kUnitTokens;
    const int units_per_part = (total_units + partitions - 1) / partitions;
    const int unit_begin = part * units_per_part;
    const int unit_end = min(total_units, unit_begin + units_per_part);
    const int my_units = max(0, unit_end - unit_begin);
    const int num_stages = (my_units + kStageUnits - 1) / kStageUnits;
    const int units_per_page = page_size / kUnitTokens;
    const uint32_t* table = block_tables + static_cast<size_t>(row) * max_blocks;

    // Stale bytes of a partly filled stage are multiplied by zero probabilities, so they
    // must be finite: clear the value ring once.
    for (int i = threadIdx.x; i < kStages * kStageBytes / 16; i += kThreads) {
        reinterpret_cast<uint4*>(&sm.v[0][0])[i] = make_uint4(0, 0, 0, 0);
    }
    if (threadIdx.x == 0) {
        sm.failed = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
        }
        mbar_fence_init();
    }
    fence_proxy_async();
    __syncthreads();

    auto issue_stage = [&](int stage_index) {
        const int slot = stage_index % kStages;
        const int first = unit_begin + stage_index * kStageUnits;
        const int count = min(kStageUnits, unit_end - first);
        mbar_arrive_expect_tx(&sm.full[slot], static_cast<uint32_t>(count) * 2 * kUnitBytes);
        for (int u = 0; u < count; ++u) {
            const int unit = first + u;
            const uint32_t physical = table[unit / units_per_page];
            const size_t offset =
                ((static_cast<size_t>(physical) * kKvHeads + kv_head) * page_size +
                 static_cast<size_t>(unit % units_per_page) * kUnitTokens) *
                kHeadDim;
            bulk_g2s(&sm.k[slot][u * kUnitPitch], key_cache + offset, kUnitBytes, &sm.full[slot]);
            bulk_g2s(&sm.v[slot][u * kUnitPitch], value_cache + offset, kUnitBytes, &sm.full[slot]);
        }
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages && s < num_stages; ++s) {
            issue_stage(s);
        }
    }

    // Query A fragments for the 16 k-steps.  K fragment reads take 16-byte bank group
    // u(t, m) = 2t + (m & 1) + 8 (m >> 1) of a token row in load m, so k-step (m, s)
    // contracts dims 16 u + 4 s .. + 3 for t = 0..3: Q uses the same permutation.
    uint32_t qa[16][2];
    {
        const int head = kv_head * kGqaGroup + g;
        const __nv_bfloat16* qp = query + (static_cast<size_t>(row) * kQueryHeads + head) * kHeadDim;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int unit = 2 * t + (m & 1) + 8 * (m >> 1);
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                if (g < kGqaGroup) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(qp + 16 * unit + 4 * s);
                    qa[m * 4 + s][0] = pack_half2(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u));
                    qa[m * 4 + s][1] = pack_half2(__uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                } else {
                    qa[m * 4 + s][0] = 0;
                    qa[m * 4 + s][1] = 0;
                }
            }
        }
    }

    const float k_scale = key_scales ? key_scales[kv_head] : 1.0f;
    const float score_scale = softmax_scale * k_scale * kLog2e;

    float oacc[4][2][4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                oacc[a][b][c] = 0.0f;
            }
        }
    }
    float running_max = -INFINITY;  // log2 domain, shared by all warps
    float running_sum = 0.0f;       // this warp's tokens only

    const uint32_t v_base = smem_u32(&sm.v[0][0]);

    for (int stage_index = 0; stage_index < num_stages; ++stage_index) {
        const int slot = stage_index % kStages;
        if (!mbar_wait_bounded(&sm.full[slot], (stage_index / kStages) & 1, kStatusAttentionPageWait, status)) {
            sm.failed = 1;
        }
        const int first_token = (unit_begin + stage_index * kStageUnits) * kUnitTokens;

        // ---- S = Q K^T for this warp's four column tiles (token j of each unit) ----
        float sc[4][2];
        float local_max = -INFINITY;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int j = 4 * warp + jj;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const uint8_t* krow = &sm.k[slot][g * kUnitPitch + j * kHeadDim];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const int unit = 2 * t + (m & 1) + 8 * (m >> 1);
                const uint4 raw = *reinterpret_cast<const uint4*>(krow + 16 * unit);
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    uint32_t b0, b1;
                    cvt_e4m3x4(words[s], b0, b1);
                    mma_f16_16816(acc, qa[m * 4 + s][0], 0u, qa[m * 4 + s][1], 0u, b0, b1);
                }
            }
            // acc[0], acc[1]: head g, tokens (unit 2t, j) and (unit 2t + 1, j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int token = first_token + (2 * t + e) * kUnitTokens + j;
                const bool valid = token < context && (2 * t + e) < (unit_end - unit_begin - stage_index * kStageUnits);
                sc[jj][e] = valid ? acc[e] * score_scale : -INFINITY;
                local_max = fmaxf(local_max, sc[jj][e]);
            }
        }
        local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 1));
        local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 2));
        if (t == 0) {
            sm.warp_max[warp][g] = local_max;
        }
        __syncthreads();

        float new_max = running_max;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            new_max = fmaxf(new_max, sm.warp_max[w][g]);
        }
        const float rescale = new_max == -INFINITY ? 1.0f : exp2f(running_max - new_max);
        running_max = new_max;
        float row_sum = 0.0f;
        uint32_t pfrag[2][2];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const float p0 = new_max == -INFINITY ? 0.0f : exp2f(sc[jj][0] - new_max);
            const float p1 = new_max == -INFINITY ? 0.0f : exp2f(sc[jj][1] - new_max);
            row_sum += p0 + p1;
            pfrag[jj >> 1][jj & 1] = pack_half2(p0, p1);
        }
        running_sum = running_sum * rescale + row_sum;
        // PV k-step kk contracts tokens j = 2 kk and 2 kk + 1 of the eight units.
        sm.p[2 * warp][lane] = make_uint2(pfrag[0][0], pfrag[0][1]);
        sm.p[2 * warp + 1][lane] = make_uint2(pfrag[1][0], pfrag[1][1]);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                oacc[a][b][0] *= rescale;
                oacc[a][b][1] *= rescale;
            }
        }
        __syncthreads();

        // ---- O += P V for this warp's 64 output dims --------------------------------
        const uint32_t v_slot = v_base + slot * kStageBytes;
#pragma unroll
        for (int kk = 0; kk < kStageUnits; ++kk) {
            const uint2 pa = sm.p[kk][lane];
#pragma unroll
            for (int dp = 0; dp < 2; ++dp) {
                const int matrix = lane >> 3;
                const int token = 2 * kk + (matrix & 1);
                const int dblock = 4 * warp + 2 * dp + (matrix >> 1);
                uint32_t r[4];
                ldmatrix_x4_trans(r, v_slot + (lane & 7) * kUnitPitch + token * kHeadDim + dblock * 16);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    // bytes (b0, b2 | b1, b3): low pair feeds the even dim, high pair the odd dim
                    const uint32_t lo_tokens = __byte_perm(r[2 * half], 0, 0x3120);
                    const uint32_t hi_tokens = __byte_perm(r[2 * half + 1], 0, 0x3120);
                    uint32_t even0, odd0, even1, odd1;
                    cvt_e4m3x4(lo_tokens, even0, odd0);
                    cvt_e4m3x4(hi_tokens, even1, odd1);
                    mma_f16_16816(oacc[2 * dp + half][0], pa.x, 0u, pa.y, 0u, even0, even1);
                    mma_f16_16816(oacc[2 * dp + half][1], pa.x, 0u, pa.y, 0u, odd0, odd1);
                }
            }
        }
        __syncthreads();
        if (threadIdx.x == 0 && stage_index + kStages < num_stages) {
            issue_stage(stage_index + kStages);
        }
    }

    // ---- combine the warps' sums, normalise, write ------------------------------------
    running_sum += __shfl_xor_sync(0xffffffffu, running_sum, 1);
    running_sum += __shfl_xor_sync(0xffffffffu, running_sum, 2);
    if (t == 0) {
        sm.warp_sum[warp][g] = running_sum;
    }
    __syncthreads();
    if (sm.failed || g >= kGqaGroup) {
        return;
    }
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        total += sm.warp_sum[w][g];
    }
    const float v_scale = value_scales ? value_scales[kv_head] : 1.0f;
    const float inverse = total > 0.0f ? v_scale / total : 0.0f;
    const int head = kv_head * kGqaGroup + g;
    const size_t pair = static_cast<size_t>(row - row_base) * kQueryHeads + head;

    if (kSplit) {
        if (warp == 0 && t == 0) {
            float* stats = partial_stats + (pair * partitions + part) * kPartialFloats;
            stats[0] = running_max;
            stats[1] = total;
        }
        __half* po = partial_out + (pair * partitions + part) * kHeadDim;
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int d = 16 * (4 * warp + a) + 4 * t;
            const uint2 packed = make_uint2(pack_half2(oacc[a][0][0] * inverse, oacc[a][1][0] * inverse),
                                            pack_half2(oacc[a][0][1] * inverse, oacc[a][1][1] * inverse));
            *reinterpret_cast<uint2*>(po + d) = packed;
        }
    } else {
        __nv_bfloat16* op = output + (static_cast<size_t>(row) * kQueryHeads + head) * kHeadDim;
        const __nv_bfloat16* gp =
            query_gate_projection
                ? query_gate_projection + static_cast<size_t>(row) * gate_stride + head * (2 * kHeadDim) + kHeadDim
                : nullptr;
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int d = 16 * (4 * warp + a) + 4 * t;
            float values[4] = {oacc[a][0][0] * inverse, oacc[a][1][0] * inverse, oacc[a][0][1] * inverse,
                               oacc[a][1][1] * inverse};
            if (gp != nullptr) {
                const uint2 graw = *reinterpret_cast<const uint2*>(gp + d);
                const float gates[4] = {__uint_as_float(graw.x << 16), __uint_as_float(graw.x & 0xffff0000u),
                                        __uint_as_float(graw.y << 16), __uint_as_float(graw.y & 0xffff0000u)};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    values[i] *= 1.0f / (1.0f + __expf(-gates[i]));
                }
            }
            __nv_bfloat162 lo = __floats2bfloat162_rn(values[0], values[1]);
            __nv_bfloat162 hi = __floats2bfloat162_rn(values[2], values[3]);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(op + d) = packed;
        }
    }
}

// Log-sum-exp merge of the partitions, output gate, bf16 store: one warp per
// (row, head), eight dims per lane (as cuda/paged_attention.cu:1736-1823).
__global__ void __launch_bounds__(256) reduce_partitions_kernel(
    const float* __restrict__ partial_stats, const __half* __restrict__ partial_out,
    const __nv_bfloat16* __restrict__ query_gate_projection, __nv_bfloat16* __restrict__ output, int pairs,
    int partitions, int row_base, int gate_stride) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= pairs) {
        return;
    }
    const float* stats = partial_stats + static_cast<size_t>(warp) * partitions * kPartialFloats;
    float maximum = -INFINITY;
    for (int p = 0; p < partitions; ++p) {
        if (stats[2 * p + 1] > 0.0f) {
            maximum = fmaxf(maximum, stats[2 * p]);
        }
    }
    float denominator = 0.0f;
    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    for (int p = 0; p < partitions; ++p) {
        const float sum = stats[2 * p + 1];
        if (!(sum > 0.0f)) {
            continue;
        }
        const float weight = sum * exp2f(stats[2 * p] - maximum);
        denominator += weight;
        const uint4 raw =
            *reinterpret_cast<const uint4*>(partial_out + (static_cast<size_t>(warp) * partitions + p) * kHeadDim + 8 * lane);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            acc[2 * i] += weight * f.x;
            acc[2 * i + 1] += weight * f.y;
        }
    }
    const float inverse = denominator > 0.0f ? 1.0f / denominator : 0.0f;
    const int row = row_base + warp / kQueryHeads;
    const int head = warp % kQueryHeads;
    float gates[8] = {1.0f, 1.0f, 1.0f, 1.0f, 1.0f, 1.0f, 1.0f, 1.0f};
    if (query_gate_projection != nullptr) {
        const uint4 graw = *reinterpret_cast<const uint4*>(
            query_gate_projection + static_cast<size_t>(row) * gate_stride + head * (2 * kHeadDim) + kHeadDim + 8 * lane);
        const uint32_t words[4] = {graw.x, graw.y, graw.z, graw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            gates[2 * i] = 1.0f / (1.0f + __expf(-__uint_as_float(words[i] << 16)));
            gates[2 * i + 1] = 1.0f / (1.0f + __expf(-__uint_as_float(words[i] & 0xffff0000u)));
        }
    }
    uint32_t packed[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * i] * inverse * gates[2 * i],
                                                  acc[2 * i + 1] * inverse * gates[2 * i + 1]);
        packed[i] = *reinterpret_cast<uint32_t*>(&v);
    }
    *reinterpret_cast<uint4*>(output + (static_cast<size_t>(row) * kQueryHeads + head) * kHeadDim + 8 * lane) =
        make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

cudaError_t launch_attention(const void* query, const void* query_gate_projection, const void* key_cache,
                             const void* value_cache, const void* block_tables, const void* context_lengths,
                             const float* key_scales, const float* value_scales, void* output, void* workspace,
                             size_t workspace_bytes, int rows, int row_base, int max_blocks, int page_size,
                             int gate_stride, int partitions, float softmax_scale, cudaStream_t stream) {
    if (gate_stride == 0) {
        gate_stride = kQueryHeads * 2 * kHeadDim;
    }
    if (gate_stride < kQueryHeads * 2 * kHeadDim || gate_stride % 8 != 0) {
        return cudaErrorInvalidValue;
    }
    if (query == nullptr || key_cache == nullptr || value_cache == nullptr || block_tables == nullptr ||
        context_lengths == nullptr || output == nullptr || rows <= 0 || rows > kMaxStepRows || row_base < 0 ||
        max_blocks <= 0 || partitions <= 0 || partitions > 65535 || !isfinite(softmax_scale) ||
        softmax_scale <= 0.0f || (page_size != 16 && page_size != 64)) {
        return cudaErrorInvalidValue;
    }
    int* status = status_ptr();
    if (status == nullptr) {
        return cudaErrorInvalidValue;
    }
    const size_t shared = sizeof(Smem);
    static const cudaError_t opted_direct = cudaFuncSetAttribute(
        paged_attention_packed_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
    static const cudaError_t opted_split = cudaFuncSetAttribute(
        paged_attention_packed_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
    if (opted_direct != cudaSuccess) {
        return opted_direct;
    }
    if (opted_split != cudaSuccess) {
        return opted_split;
    }
    const dim3 grid(kKvHeads, rows, partitions);
    if (partitions == 1) {
        paged_attention_packed_kernel<false><<<grid, kThreads, shared, stream>>>(
            static_cast<const __nv_bfloat16*>(query), static_cast<const __nv_bfloat16*>(query_gate_projection),
            static_cast<const uint8_t*>(key_cache), static_cast<const uint8_t*>(value_cache),
            static_cast<const uint32_t*>(block_tables), static_cast<const uint32_t*>(context_lengths), key_scales,
            value_scales, static_cast<__nv_bfloat16*>(output), nullptr, nullptr, max_blocks, row_base, page_size,
            gate_stride, softmax_scale, status);
        return cudaGetLastError();
    }
    const size_t partials = static_cast<size_t>(rows) * kQueryHeads * partitions;
    if (workspace == nullptr || workspace_bytes < partials * kPartialBytes) {
        return cudaErrorInvalidValue;
    }
    // partials is a multiple of 24, so the f16 block starts on a 16-byte boundary.
    float* partial_stats = static_cast<float*>(workspace);
    __half* partial_out = reinterpret_cast<__half*>(partial_stats + partials * kPartialFloats);
    paged_attention_packed_kernel<true><<<grid, kThreads, shared, stream>>>(
        static_cast<const __nv_bfloat16*>(query), static_cast<const __nv_bfloat16*>(query_gate_projection),
        static_cast<const uint8_t*>(key_cache), static_cast<const uint8_t*>(value_cache),
        static_cast<const uint32_t*>(block_tables), static_cast<const uint32_t*>(context_lengths), key_scales,
        value_scales, static_cast<__nv_bfloat16*>(output), partial_stats, partial_out, max_blocks, row_base,
        page_size, gate_stride, softmax_scale, status);
    const cudaError_t launched = cudaGetLastError();
    if (launched != cudaSuccess) {
        return launched;
    }
    const int pairs = rows * kQueryHeads;
    reduce_partitions_kernel<<<(pairs + 7) / 8, 256, 0, stream>>>(
        partial_stats, partial_out, static_cast<const __nv_bfloat16*>(query_gate_projection),
        static_cast<__nv_bfloat16*>(output), pairs, partitions, row_base, gate_stride);
    return cudaGetLastError();
}

// ---- built-in scratch for callers that cannot allocate ------------------------------------
//
// Split-context partials normally live in a workspace the caller allocates.  Some callers have
// no way to do that: a process that handed its whole VRAM budget out at start-up and refuses
// any later cudaMalloc (the reference engine enforces such a ceiling), a thin foreign-language
// binding that can pass pointers it was given but owns no device allocator, or a diagnostic
// attached to a running server.  For them the library carries its own scratch: a fixed array
// in device memory, sized for kStaticPartialPairs (row, partition) pairs.  It exists once per
// GPU that loads the library and stays resident until the process exits.
constexpr int kStaticPartialPairs = 512;  // rows * partitions, e.g. 32 rows x 16 partitions
constexpr size_t kStaticScratchBytes = static_cast<size_t>(kStaticPartialPairs) * kQueryHeads * kPartialBytes;
static __device__ __align__(256) unsigned char g_static_partials[kStaticScratchBytes];

// Device address of the array above for the current device.  In host code the symbol's name is
// only a handle, never an address a kernel may be given, so the address is asked of the runtime
// once per device (with that device current) and remembered.
cudaError_t static_partials_address(void** out) {
    constexpr int kMaxDevices = 64;
    static void* cached[kMaxDevices] = {};
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) {
        return err;
    }
    if (device < 0 || device >= kMaxDevices) {
        return cudaErrorInvalidDevice;
    }
    if (cached[device] == nullptr) {
        void* address = nullptr;
        err = cudaGetSymbolAddress(&address, g_static_partials);
        if (err != cudaSuccess) {
            return err;
        }
        cached[device] = address;
    }
    *out = cached[device];
    return cudaSuccess;
}

}  // namespace
}  // namespace qwc

extern "C" size_t qwc_paged_attention_packed_workspace_bytes(int rows, int partitions) {
    if (rows <= 0 || partitions <= 1) {
        return 0;
    }
    return static_cast<size_t>(rows) * qwc::kQueryHeads * partitions * qwc::kPartialBytes;
}

extern "C" int qwc_paged_attention_packed_fp8(const void* query, const void* query_gate_projection,
                                              const void* key_cache, const void* value_cache,
                                              const void* block_tables, const void* context_lengths, void* output,
                                              void* workspace, size_t workspace_bytes, int rows, int row_base,
                                              int max_blocks, int tile_size, int partitions, float softmax_scale,
                                              cudaStream_t stream) {
    if (tile_size <= 0 || tile_size > 64) {
        return cudaErrorInvalidValue;
    }
    if (tile_size != qwc::kGqaGroup) {
        return cudaErrorNotSupported;  // segment tiles are prefill shapes
    }
    return qwc::launch_attention(query, query_gate_projection, key_cache, value_cache, block_tables,
                                 context_lengths, nullptr, nullptr, output, workspace, workspace_bytes, rows,
                                 row_base, max_blocks, qwc::current_shape().kv_page_size, 0, partitions,
                                 softmax_scale, stream);
}

extern "C" int qwc_paged_attention_packed_fp8_scaled(const void* query, const void* query_gate_projection,
                                                     const void* key_cache, const void* value_cache,
                                                     const void* block_tables, const void* context_lengths,
                                                     const float* key_scales, const float* value_scales,
                                                     void* output, void* workspace, size_t workspace_bytes,
                                                     int rows, int row_base, int max_blocks, int page_size,
                                                     int gate_stride, int partitions, float softmax_scale,
                                                     cudaStream_t stream) {
    return qwc::launch_attention(query, query_gate_projection, key_cache, value_cache, block_tables,
                                 context_lengths, key_scales, value_scales, output, workspace, workspace_bytes,
                                 rows, row_base, max_blocks, page_size, gate_stride, partitions, softmax_scale,
                                 stream);
}

extern "C" int qwc_paged_attention_packed_fp8_noalloc(const void* query, const void* query_gate_projection,
                                                      const void* key_cache, const void* value_cache,
                                                      const void* block_tables, const void* context_lengths,
                                                      const float* key_scales, const float* value_scales,
                                                      void* output, int rows, int row_base, int max_blocks,
                                                      int page_size, int gate_stride, int partitions,
                                                      float softmax_scale, cudaStream_t stream) {
    if (rows <= 0 || partitions <= 0) {
        return cudaErrorInvalidValue;
    }
    // The built-in scratch holds kStaticPartialPairs (row, partition) pairs and not one more.
    if (static_cast<long long>(rows) * partitions > qwc::kStaticPartialPairs) {
        return cudaErrorInvalidValue;
    }
    void* scratch = nullptr;
    const cudaError_t resolved = qwc::static_partials_address(&scratch);
    if (resolved != cudaSuccess) {
        return resolved;
    }
    // Every partial slot of this call is written by the CTA that owns it (an empty partition
    // stores sum = 0, which the merge skips), so nothing left over from an earlier call is read
    // and nothing needs clearing first.
    return qwc::launch_attention(query, query_gate_projection, key_cache, value_cache, block_tables,
                                 context_lengths, key_scales, value_scales, output, scratch,
                                 qwc::kStaticScratchBytes, rows, row_base, max_blocks, page_size, gate_stride,
                                 partitions, softmax_scale, stream);
}

extern "C" int qwc_paged_attention_packed_noalloc_max_pairs(void) { return qwc::kStaticPartialPairs; }
