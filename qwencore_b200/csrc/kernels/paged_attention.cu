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
//   * a persistent grid of one CTA per SM.  The rows of a ragged batch differ in context by
//     orders of magnitude, so the work is cut on the device into equal shares: the 16-token
//     units of all (row, kv head) pairs are laid end to end, CTA c owns positions
//     [c share, (c + 1) share) of that line, and a task is the piece of one pair inside one
//     CTA's share (its partial is merged by the second kernel).  Every CTA streams the same
//     number of bytes whatever the contexts are, and the launch shape depends only on the SM
//     count, so the step stays capturable in a CUDA graph;
//   * inside a CTA one producer warp and eight consumer warps.  KV moves in 4 KiB units (16
//     tokens x 256 B of one kv head: a whole 16-token page, or a quarter of a 64-token page)
//     by bulk-async copies (TMA 1-D) into a 3-stage ring of 8 units (128 tokens, 64 KiB of
//     K+V per stage) guarded by full/empty mbarriers; the producer runs ahead across task
//     boundaries, so the ring never drains between tasks;
//   * each unit lands 16 bytes further than a multiple of 4 KiB.  An MMA column tile is
//     "token j of 8 different units", so the eight rows an ldmatrix or a fragment load
//     touches fall in eight different 16-byte bank groups: conflict-free without a
//     swizzled tensor map;
//   * QK^T: the six heads of the group are rows of one m16 tile, e4m3 pairs are widened
//     by the hardware converter straight into B fragments; each warp owns two column tiles
//     and keeps four independent accumulation chains.  PV: V is transposed on the fly by
//     ldmatrix.trans on byte pairs and a byte permute; the eight warps split the 256 output
//     dims, exchanging P through 2 KiB of shared memory.
//
// Cache memory must hold finite e4m3 codes in every allocated page (a zero-initialised
// pool, as the reference allocates it): positions past the context are masked by
// zero probabilities, not skipped.

#include "common.cuh"

namespace qwc {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + the producer warp
constexpr int kUnitTokens = 16;
constexpr int kUnitBytes = kUnitTokens * kHeadDim;  // 4096
constexpr int kUnitPitch = kUnitBytes + 16;         // staggered landing offset
constexpr int kStageUnits = 8;
constexpr int kStages = 3;
constexpr int kStageBytes = kStageUnits * kUnitPitch;    // per K or V
constexpr int kPartialFloats = 2;
constexpr size_t kPartialBytes = 2 * sizeof(float) + kHeadDim * sizeof(__half);  // 520
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kMaxCtaTasks = 64;      // list capacity; the plan keeps a CTA far below it
constexpr int kPlanMinPadding = 16;   // units a task costs beyond its tokens (query load, epilogue, merge)
constexpr int kPlanPaddingDivisor = 24;  // padding = share / this at least: bounds the tasks of one CTA
constexpr int kPlanRows = 256;        // rows whose prefix fits the shared-memory table

struct Task {
    int row;
    int kv_head;
    int part;
    int unit_begin;
    int units;
    int context;  // tokens of the row, cut at the block table's capacity
};

struct Smem {
    uint8_t k[kStages][kStageBytes];
    uint8_t v[kStages][kStageBytes];
    uint2 p[kStageUnits][32];       // P as A fragments: [pv k-step][lane]
    float warp_max[kConsumerWarps][8];
    float warp_sum[kConsumerWarps][8];
    uint64_t full[kStages];
    uint64_t empty[kStages];
    int first_unit[kPlanRows + 1];  // prefix sum of the rows' units (a row without context counts one)
    Task tasks[kMaxCtaTasks];
    int task_count;
    int issued;                     // stages the producer has put in flight
    int consumed;                   // stages the consumers have finished
    int failed;                     // a consumer's wait gave up
    int producer_failed;            // the producer's wait gave up (written by the producer only)
    int leave[2];                   // what one consumer thread saw of the two flags before the barrier of stage n & 1
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

__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// The split plan.  Both kernels evaluate it from the same inputs.
//
// The (row, kv head) pairs are laid end to end, row-major, on a line of units; a pair takes
// max(units, 1) + padding positions (the padding stands for what a task costs beyond its tokens).
// Every CTA owns `share` consecutive positions and works on the tokens that fall inside: all CTAs
// stream the same amount, whatever the rows' lengths.  The piece of a pair inside CTA c is partial
// number c - (first CTA that touches the pair); a pair without context is one empty piece.
//   * padding >= share / kPlanPaddingDivisor, so that a CTA never holds more than
//     kPlanPaddingDivisor + pairs / CTAs + 2 tasks;
//   * share >= capacity / (partitions - 1): a row never has more pieces than the workspace has slots;
//   * share is a whole number of stages.
struct SplitPlan {
    long long share;
    int padding;
};

__device__ __forceinline__ SplitPlan make_split_plan(long long total_row_units, int rows, int capacity_units,
                                                     int partitions, int ctas) {
    const long long by_capacity = partitions > 1 ? (capacity_units + partitions - 2) / (partitions - 1) : 0;
    long long share = (total_row_units * kKvHeads + ctas - 1) / ctas;
    share = share > by_capacity ? share : by_capacity;
    const long long padding_wanted = (share + kPlanPaddingDivisor - 1) / kPlanPaddingDivisor;
    SplitPlan plan;
    plan.padding = static_cast<int>(padding_wanted > kPlanMinPadding ? padding_wanted : kPlanMinPadding);
    const long long line = (total_row_units + static_cast<long long>(rows) * plan.padding) * kKvHeads;
    share = (line + ctas - 1) / ctas;
    share = share > by_capacity ? share : by_capacity;
    plan.share = (share + kStageUnits - 1) / kStageUnits * kStageUnits;
    return plan;
}

// first position of pair (row, kv head); units_before = units of the rows before it
__device__ __forceinline__ long long pair_position(const SplitPlan& plan, int row, int kv_head, long long units_before,
                                                   int row_units) {
    return (units_before + static_cast<long long>(row) * plan.padding) * kKvHeads +
           static_cast<long long>(kv_head) * (row_units + plan.padding);
}

// A context longer than the block table can describe is cut at the table's capacity.
__device__ __forceinline__ int units_of_context(uint32_t context, int capacity_units) {
    const uint32_t units = (context + kUnitTokens - 1) / kUnitTokens;
    return static_cast<int>(units < static_cast<uint32_t>(capacity_units) ? units : capacity_units);
}

// Units a row occupies on the plan's line: a row without context still gets one task (it stores zeros).
__device__ __forceinline__ int plan_units(int units) { return units > 0 ? units : 1; }

template <bool kSplit>
__global__ void __launch_bounds__(kThreads, 1) paged_attention_packed_kernel(
    const __nv_bfloat16* __restrict__ query, const __nv_bfloat16* __restrict__ query_gate_projection,
    const uint8_t* __restrict__ key_cache, const uint8_t* __restrict__ value_cache,
    const uint32_t* __restrict__ block_tables, const uint32_t* __restrict__ context_lengths,
    const float* __restrict__ key_scales, const float* __restrict__ value_scales,
    __nv_bfloat16* __restrict__ output, __half* __restrict__ staged_output, int padded_rows,
    float* __restrict__ partial_stats, __half* __restrict__ partial_out, int rows, int max_blocks, int row_base,
    int page_size, int gate_stride, int partitions, float softmax_scale, int* status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);

    pdl_launch_dependents();
    if (status_is_set(status)) {
        return;
    }
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int units_per_page = page_size / kUnitTokens;
    const int capacity_units = max_blocks * units_per_page;

    // ---- plan: task size, the rows' task counts, this CTA's task list ---------------------
    // Stale bytes of a partly filled stage are multiplied by zero probabilities, so they
    // must be finite: clear the value ring once (every later byte comes from the cache).
    for (int i = threadIdx.x; i < kStages * kStageBytes / 16; i += kThreads) {
        reinterpret_cast<uint4*>(&sm.v[0][0])[i] = make_uint4(0, 0, 0, 0);
    }
    pdl_wait();  // context lengths, tables, query and the cache rows of this step come from earlier kernels
    if (warp == 0) {
        if (lane == 0) {
            sm.failed = 0;
            sm.producer_failed = 0;
            sm.leave[0] = 0;
            sm.leave[1] = 0;
            sm.consumed = 0;
            sm.issued = 0;
            for (int s = 0; s < kStages; ++s) {
                mbar_init(&sm.full[s], 1);
                mbar_init(&sm.empty[s], kConsumerWarps);
            }
            mbar_fence_init();
        }
        int count = 0;
        if (!kSplit) {
            // whole (row, kv head) pairs, dealt round: c, c + grid, ...
            for (int index = lane; index < kMaxCtaTasks; index += 32) {
                const long long id = static_cast<long long>(blockIdx.x) + static_cast<long long>(index) * gridDim.x;
                if (id < static_cast<long long>(rows) * kKvHeads) {
                    const int row = static_cast<int>(id / kKvHeads);
                    const uint32_t row_context = context_lengths[row_base + row];
                    Task task;
                    task.context = static_cast<int>(min(row_context, static_cast<uint32_t>(capacity_units) * kUnitTokens));
                    task.row = row_base + row;
                    task.kv_head = static_cast<int>(id % kKvHeads);
                    task.part = 0;
                    task.unit_begin = 0;
                    task.units = units_of_context(row_context, capacity_units);
                    sm.tasks[index] = task;
                    ++count;
                }
            }
            count = __reduce_add_sync(0xffffffffu, count);
        } else {
            // prefix of the rows' units: a warp scan per 32 rows
            int carry = 0;
            for (int base = 0; base < rows; base += 32) {
                const int r = base + lane;
                const int mine = r < rows ? plan_units(units_of_context(context_lengths[row_base + r], capacity_units)) : 0;
                int inclusive = mine;
#pragma unroll
                for (int offset = 1; offset < 32; offset <<= 1) {
                    const int other = __shfl_up_sync(0xffffffffu, inclusive, offset);
                    if (lane >= offset) {
                        inclusive += other;
                    }
                }
                if (r < rows) {
                    sm.first_unit[r] = carry + inclusive - mine;
                }
                carry += __shfl_sync(0xffffffffu, inclusive, 31);
            }
            if (lane == 0) {
                sm.first_unit[rows] = carry;
            }
            __syncwarp();
            const SplitPlan plan = make_split_plan(carry, rows, capacity_units, partitions, gridDim.x);
            const long long low = static_cast<long long>(blockIdx.x) * plan.share;
            const long long high = low + plan.share;
            // the pieces of this CTA, in (row, kv head) order: 32 rows at a time, a lane per row
            for (int base = 0; base < rows; base += 32) {
                const int r = base + lane;
                Task mine[kKvHeads];
                int found = 0;
                if (r < rows) {
                    const uint32_t row_context = context_lengths[row_base + r];
                    const int row_units = units_of_context(row_context, capacity_units);
                    const int occupied = plan_units(row_units);
#pragma unroll
                    for (int kv = 0; kv < kKvHeads; ++kv) {
                        const long long start = pair_position(plan, r, kv, sm.first_unit[r], occupied);
                        if (start < high && start + occupied > low) {
                            const long long begin = low > start ? low - start : 0;
                            const long long end = high - start < occupied ? high - start : occupied;
                            Task task;
                            task.context =
                                static_cast<int>(min(row_context, static_cast<uint32_t>(capacity_units) * kUnitTokens));
                            task.row = row_base + r;
                            task.kv_head = kv;
                            task.part = static_cast<int>(blockIdx.x - start / plan.share);
                            task.unit_begin = static_cast<int>(begin);
                            task.units = max(0, min(static_cast<int>(end), row_units) - static_cast<int>(begin));
                            mine[found++] = task;
                        }
                    }
                }
                int before = found;  // exclusive prefix over the lanes
#pragma unroll
                for (int offset = 1; offset < 32; offset <<= 1) {
                    const int other = __shfl_up_sync(0xffffffffu, before, offset);
                    if (lane >= offset) {
                        before += other;
                    }
                }
                const int all = __shfl_sync(0xffffffffu, before, 31);
                before -= found;
#pragma unroll
                for (int i = 0; i < kKvHeads; ++i) {
                    if (i < found && count + before + i < kMaxCtaTasks) {
                        sm.tasks[count + before + i] = mine[i];
                    }
                }
                count += all;
            }
            if (count > kMaxCtaTasks) {
                // cannot happen while the launcher's check of rows against the SM count holds
                if (lane == 0) {
                    atomicCAS(status, 0, kStatusAttentionPlanOverflow);
                }
                count = 0;
            }
        }
        if (lane == 0) {
            sm.task_count = count;
        }
    }
    fence_proxy_async();
    __syncthreads();
    const int task_count = sm.task_count;

    if (warp == kConsumerWarps) {
        // ---------------- producer ----------------------------------------------------------
        int n = 0;  // stages issued so far
        bool ok = true;
        for (int ti = 0; ti < task_count && ok; ++ti) {
            const Task task = sm.tasks[ti];
            const uint32_t* table = block_tables + static_cast<size_t>(task.row) * max_blocks;
            const int stages = (task.units + kStageUnits - 1) / kStageUnits;
            for (int st = 0; st < stages && ok; ++st, ++n) {
                const int slot = n % kStages;
                const int first = task.unit_begin + st * kStageUnits;
                const int count = min(kStageUnits, task.units - st * kStageUnits);
                // the page id is fetched before the wait for a free slot, which is the longer of the two
                const uint32_t physical = lane < count ? table[(first + lane) / units_per_page] : 0u;
                ok = mbar_wait_bounded(&sm.empty[slot], ((n / kStages) & 1) ^ 1, kStatusAttentionPageWait, status);
                // one lane reads the consumers' flag for the whole warp: the decision to leave is uniform
                const int consumers_left =
                    __shfl_sync(0xffffffffu, *reinterpret_cast<volatile int*>(&sm.failed), 0);
                ok = __all_sync(0xffffffffu, ok) && consumers_left == 0;
                if (!ok) {
                    break;
                }
                if (lane == 0) {
                    mbar_arrive_expect_tx(&sm.full[slot], static_cast<uint32_t>(count) * 2 * kUnitBytes);
                }
                __syncwarp();
                if (lane < count) {
                    const int unit = first + lane;
                    const size_t offset = ((static_cast<size_t>(physical) * kKvHeads + task.kv_head) * page_size +
                                           static_cast<size_t>(unit % units_per_page) * kUnitTokens) *
                                          kHeadDim;
                    bulk_g2s(&sm.k[slot][lane * kUnitPitch], key_cache + offset, kUnitBytes, &sm.full[slot]);
                    bulk_g2s(&sm.v[slot][lane * kUnitPitch], value_cache + offset, kUnitBytes, &sm.full[slot]);
                }
                __syncwarp();
                if (lane == 0) {
                    *reinterpret_cast<volatile int*>(&sm.issued) = n + 1;
                }
            }
        }
        if (!ok && lane == 0) {
            *reinterpret_cast<volatile int*>(&sm.producer_failed) = 1;
        }
    } else {
        // ---------------- consumers ---------------------------------------------------------
        const uint32_t v_base = smem_u32(&sm.v[0][0]);
        int n = 0;  // stages consumed so far
        bool ok = true;
        // bf16 words of this lane's query fragments (head g of the task's group; rows 6, 7 are padding)
        uint2 q_raw[16];
        auto load_query = [&](const Task& next) {
            const int head = next.kv_head * kGqaGroup + g;
            const __nv_bfloat16* qp = query + (static_cast<size_t>(next.row) * kQueryHeads + head) * kHeadDim;
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const int unit = 2 * t + (m & 1) + 8 * (m >> 1);
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    q_raw[m * 4 + s] = g < kGqaGroup ? *reinterpret_cast<const uint2*>(qp + 16 * unit + 4 * s)
                                                     : make_uint2(0u, 0u);
                }
            }
        };
        if (task_count > 0) {
            load_query(sm.tasks[0]);
        }
        for (int ti = 0; ti < task_count && ok; ++ti) {
            const Task task = sm.tasks[ti];
            const int row = task.row;
            const int kv_head = task.kv_head;
            const int context = task.context;

            // Query A fragments for the 16 k-steps.  K fragment reads take 16-byte bank group
            // u(t, m) = 2t + (m & 1) + 8 (m >> 1) of a token row in load m, so k-step (m, s)
            // contracts dims 16 u + 4 s .. + 3 for t = 0..3: Q uses the same permutation.
            // The raw bf16 words were fetched while the previous task was computed.
            uint32_t qa[16][2];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                qa[i][0] = pack_half2(__uint_as_float(q_raw[i].x << 16), __uint_as_float(q_raw[i].x & 0xffff0000u));
                qa[i][1] = pack_half2(__uint_as_float(q_raw[i].y << 16), __uint_as_float(q_raw[i].y & 0xffff0000u));
            }
            if (ti + 1 < task_count) {
                load_query(sm.tasks[ti + 1]);  // in flight during this task
            }
            const float k_scale = key_scales ? key_scales[kv_head] : 1.0f;
            const float score_scale = softmax_scale * k_scale * kLog2e;

            float oacc[2][2][4];
#pragma unroll
            for (int a = 0; a < 2; ++a) {
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

            const int stages = (task.units + kStageUnits - 1) / kStageUnits;
            for (int st = 0; st < stages; ++st, ++n) {
                const int slot = n % kStages;
                if (*reinterpret_cast<volatile int*>(&sm.failed) != 0 ||
                    !mbar_wait_bounded(&sm.full[slot], (n / kStages) & 1, kStatusAttentionPageWait, status)) {
                    *reinterpret_cast<volatile int*>(&sm.failed) = 1;  // acted on after the next barrier, by all
                }
                const int first_token = (task.unit_begin + st * kStageUnits) * kUnitTokens;
                const int units_here = task.units - st * kStageUnits;

                // ---- S = Q K^T for this warp's two column tiles (tokens 2w, 2w + 1 of each unit)
                float acc[2][2][4];
#pragma unroll
                for (int a = 0; a < 2; ++a) {
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            acc[a][b][c] = 0.0f;
                        }
                    }
                }
                const uint8_t* krow = &sm.k[slot][g * kUnitPitch + (2 * warp) * kHeadDim];
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    const int unit = 2 * t + (m & 1) + 8 * (m >> 1);
                    const uint4 raw0 = *reinterpret_cast<const uint4*>(krow + 16 * unit);
                    const uint4 raw1 = *reinterpret_cast<const uint4*>(krow + kHeadDim + 16 * unit);
                    const uint32_t words[2][4] = {{raw0.x, raw0.y, raw0.z, raw0.w}, {raw1.x, raw1.y, raw1.z, raw1.w}};
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
#pragma unroll
                        for (int tile = 0; tile < 2; ++tile) {
                            uint32_t b0, b1;
                            cvt_e4m3x4(words[tile][s], b0, b1);
                            mma_f16_16816(acc[tile][s & 1], qa[m * 4 + s][0], 0u, qa[m * 4 + s][1], 0u, b0, b1);
                        }
                    }
                }
                // acc[tile][.][0], [1]: head g, tokens (unit 2t, j) and (unit 2t + 1, j), j = 2w + tile
                float sc[2][2];
                float local_max = -INFINITY;
#pragma unroll
                for (int tile = 0; tile < 2; ++tile) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int token = first_token + (2 * t + e) * kUnitTokens + 2 * warp + tile;
                        const bool valid = token < context && (2 * t + e) < units_here;
                        sc[tile][e] = valid ? (acc[tile][0][e] + acc[tile][1][e]) * score_scale : -INFINITY;
                        local_max = fmaxf(local_max, sc[tile][e]);
                    }
                }
                local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 1));
                local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 2));
                if (t == 0) {
                    sm.warp_max[warp][g] = local_max;
                }
                // The flags can change at any moment (the producer raises its own asynchronously), so a
                // consumer that read them for itself after the barrier could leave while another stays and
                // waits at the next barrier for ever.  One thread samples them before the barrier into the
                // word of this stage; every consumer acts on that word only.  A failure that thread 0 has
                // not seen yet is acted on one stage later.
                if (threadIdx.x == 0) {
                    sm.leave[n & 1] = *reinterpret_cast<volatile int*>(&sm.failed) |
                                      *reinterpret_cast<volatile int*>(&sm.producer_failed);
                }
                consumer_sync();
                ok = *reinterpret_cast<volatile int*>(&sm.leave[n & 1]) == 0;
                if (!ok) {
                    break;  // the same word for every consumer: they leave together
                }

                float new_max = running_max;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) {
                    new_max = fmaxf(new_max, sm.warp_max[w][g]);
                }
                const float rescale = new_max == -INFINITY ? 1.0f : exp2f(running_max - new_max);
                running_max = new_max;
                float row_sum = 0.0f;
                uint32_t pfrag[2];
#pragma unroll
                for (int tile = 0; tile < 2; ++tile) {
                    const float p0 = new_max == -INFINITY ? 0.0f : exp2f(sc[tile][0] - new_max);
                    const float p1 = new_max == -INFINITY ? 0.0f : exp2f(sc[tile][1] - new_max);
                    row_sum += p0 + p1;
                    pfrag[tile] = pack_half2(p0, p1);
                }
                running_sum = running_sum * rescale + row_sum;
                // PV k-step kk contracts tokens j = 2 kk and 2 kk + 1 of the eight units: this warp's two tiles.
                sm.p[warp][lane] = make_uint2(pfrag[0], pfrag[1]);
#pragma unroll
                for (int a = 0; a < 2; ++a) {
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        oacc[a][b][0] *= rescale;
                        oacc[a][b][1] *= rescale;
                    }
                }
                consumer_sync();

                // ---- O += P V for this warp's 32 output dims --------------------------------
                const uint32_t v_slot = v_base + slot * kStageBytes;
                const int matrix = lane >> 3;
                const uint32_t v_lane = v_slot + (lane & 7) * kUnitPitch + (matrix & 1) * kHeadDim +
                                        (2 * warp + (matrix >> 1)) * 16;
#pragma unroll
                for (int kk = 0; kk < kStageUnits; ++kk) {
                    const uint2 pa = sm.p[kk][lane];
                    uint32_t r[4];
                    ldmatrix_x4_trans(r, v_lane + 2 * kk * kHeadDim);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        // bytes (b0, b2 | b1, b3): low pair feeds the even dim, high pair the odd dim
                        const uint32_t lo_tokens = __byte_perm(r[2 * half], 0, 0x3120);
                        const uint32_t hi_tokens = __byte_perm(r[2 * half + 1], 0, 0x3120);
                        uint32_t even0, odd0, even1, odd1;
                        cvt_e4m3x4(lo_tokens, even0, odd0);
                        cvt_e4m3x4(hi_tokens, even1, odd1);
                        mma_f16_16816(oacc[half][0], pa.x, 0u, pa.y, 0u, even0, even1);
                        mma_f16_16816(oacc[half][1], pa.x, 0u, pa.y, 0u, odd0, odd1);
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&sm.empty[slot]);
                }
            }
            if (!ok) {
                break;
            }

            // ---- combine the warps' sums, normalise, write --------------------------------
            running_sum += __shfl_xor_sync(0xffffffffu, running_sum, 1);
            running_sum += __shfl_xor_sync(0xffffffffu, running_sum, 2);
            if (t == 0) {
                sm.warp_sum[warp][g] = running_sum;
            }
            consumer_sync();
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                total += sm.warp_sum[w][g];
            }
            consumer_sync();  // the sums are read before the next task overwrites them
            if (g < kGqaGroup) {
                const float v_scale = value_scales ? value_scales[kv_head] : 1.0f;
                const float inverse = total > 0.0f ? v_scale / total : 0.0f;
                const int head = kv_head * kGqaGroup + g;
                const size_t pair = static_cast<size_t>(row - row_base) * kQueryHeads + head;
                if (kSplit) {
                    const size_t slot_index = pair * partitions + task.part;
                    if (warp == 0 && t == 0) {
                        float* stats = partial_stats + slot_index * kPartialFloats;
                        stats[0] = running_max;
                        stats[1] = total;
                    }
                    __half* po = partial_out + slot_index * kHeadDim;
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const int d = 16 * (2 * warp + a) + 4 * t;
                        const uint2 packed = make_uint2(pack_half2(oacc[a][0][0] * inverse, oacc[a][1][0] * inverse),
                                                        pack_half2(oacc[a][0][1] * inverse, oacc[a][1][1] * inverse));
                        *reinterpret_cast<uint2*>(po + d) = packed;
                    }
                } else {
                    __nv_bfloat16* op = output + (static_cast<size_t>(row) * kQueryHeads + head) * kHeadDim;
                    const __nv_bfloat16* gp = query_gate_projection
                                                  ? query_gate_projection + static_cast<size_t>(row) * gate_stride +
                                                        head * (2 * kHeadDim) + kHeadDim
                                                  : nullptr;
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const int d = 16 * (2 * warp + a) + 4 * t;
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
                        if (output != nullptr) {
                            *reinterpret_cast<uint2*>(op + d) = packed;
                        }
                        if (staged_output != nullptr) {
                            // the same values as f16 in the operand layout of the output projection
                            const int feature = head * kHeadDim + d;
                            *reinterpret_cast<uint2*>(staged_output +
                                                      (static_cast<size_t>(feature >> 3) * padded_rows + row) * 8 +
                                                      (feature & 7)) =
                                make_uint2(bf16x2_to_f16x2(packed.x), bf16x2_to_f16x2(packed.y));
                        }
                    }
                }
            }
        }
        if (threadIdx.x == 0) {
            sm.consumed = n;
        }
    }
    __syncthreads();
    // After a failed wait the CTA must not return while copies it issued are still landing:
    // one thread waits (bounded) for the stages that were put in flight and never consumed.
    if (threadIdx.x == 0 && (sm.failed | sm.producer_failed) != 0) {
        for (int i = sm.consumed; i < sm.issued; ++i) {
            mbar_wait_bounded(&sm.full[i % kStages], (i / kStages) & 1, kStatusAttentionPageWait, status);
        }
    }
}

// Log-sum-exp merge of the partitions, output gate, bf16 store (as cuda/paged_attention.cu:1736-1823).
// One CTA of four warps per (row, head): the longest row of a ragged batch has dozens of partials,
// and a single warp walking them is a chain of dependent memory round trips.  Warp w takes the
// partials w, w + 4, ... (eight dims per lane), the four sums meet in shared memory in warp order.
constexpr int kMergeWarps = 4;

__global__ void __launch_bounds__(kMergeWarps * 32) reduce_partitions_kernel(
    const float* __restrict__ partial_stats, const __half* __restrict__ partial_out,
    const __nv_bfloat16* __restrict__ query_gate_projection, const uint32_t* __restrict__ context_lengths,
    __nv_bfloat16* __restrict__ output, __half* __restrict__ staged_output, int padded_rows, int rows, int partitions,
    int row_base, int gate_stride, int capacity_units, int plan_ctas) {
    pdl_launch_dependents();  // the output projection may start streaming its weights
    pdl_wait();
    __shared__ float sums[kMergeWarps][kHeadDim];
    __shared__ float denominators[kMergeWarps];
    const int pair = blockIdx.x;  // (row, head)
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // The same plan as the attention kernel made: this pair has `used` partials, the rest of its
    // slots were never written.
    const int plan_row = pair / kQueryHeads;
    long long total_units = 0, units_before = 0;
    for (int r = lane; r < rows; r += 32) {
        const int units = plan_units(units_of_context(context_lengths[row_base + r], capacity_units));
        total_units += units;
        units_before += r < plan_row ? units : 0;
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        total_units += __shfl_xor_sync(0xffffffffu, total_units, offset);
        units_before += __shfl_xor_sync(0xffffffffu, units_before, offset);
    }
    const SplitPlan plan = make_split_plan(total_units, rows, capacity_units, partitions, plan_ctas);
    const int occupied = plan_units(units_of_context(context_lengths[row_base + plan_row], capacity_units));
    const long long start = pair_position(plan, plan_row, (pair % kQueryHeads) / kGqaGroup, units_before, occupied);
    const int used = static_cast<int>((start + occupied - 1) / plan.share - start / plan.share) + 1;
    const float* stats = partial_stats + static_cast<size_t>(pair) * partitions * kPartialFloats;
    // every warp finds the maximum over all partials (lanes side by side) ...
    float maximum = -INFINITY;
    for (int p = lane; p < used; p += 32) {
        const float2 pair_stats = *reinterpret_cast<const float2*>(stats + 2 * p);
        if (pair_stats.y > 0.0f) {
            maximum = fmaxf(maximum, pair_stats.x);
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
    }
    // ... and sums its own quarter of them, four outputs in flight at a time
    float denominator = 0.0f;
    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    const __half* outs = partial_out + static_cast<size_t>(pair) * partitions * kHeadDim + 8 * lane;
    for (int first = warp; first < used; first += 4 * kMergeWarps) {
        uint4 raw[4];
        float weight[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int p = first + j * kMergeWarps;
            weight[j] = 0.0f;
            raw[j] = make_uint4(0, 0, 0, 0);
            if (p < used) {
                const float2 pair_stats = *reinterpret_cast<const float2*>(stats + 2 * p);
                weight[j] = pair_stats.y > 0.0f ? pair_stats.y * exp2f(pair_stats.x - maximum) : 0.0f;
                raw[j] = *reinterpret_cast<const uint4*>(outs + static_cast<size_t>(p) * kHeadDim);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            denominator += weight[j];
            const __half2* h = reinterpret_cast<const __half2*>(&raw[j]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                acc[2 * i] += weight[j] * f.x;
                acc[2 * i + 1] += weight[j] * f.y;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        sums[warp][8 * lane + i] = acc[i];
    }
    if (lane == 0) {
        denominators[warp] = denominator;
    }
    __syncthreads();
    if (warp != 0) {
        return;
    }
    denominator = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        acc[i] = 0.0f;
    }
#pragma unroll
    for (int w = 0; w < kMergeWarps; ++w) {
        denominator += denominators[w];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            acc[i] += sums[w][8 * lane + i];
        }
    }
    const float inverse = denominator > 0.0f ? 1.0f / denominator : 0.0f;
    const int row = row_base + pair / kQueryHeads;
    const int head = pair % kQueryHeads;
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
    if (output != nullptr) {
        *reinterpret_cast<uint4*>(output + (static_cast<size_t>(row) * kQueryHeads + head) * kHeadDim + 8 * lane) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    if (staged_output != nullptr) {
        // the same values as f16 in the operand layout of the output projection: this lane's eight
        // dims are one K core
        const int core = head * (kHeadDim / 8) + lane;
        *reinterpret_cast<uint4*>(staged_output + (static_cast<size_t>(core) * padded_rows + row) * 8) =
            make_uint4(bf16x2_to_f16x2(packed[0]), bf16x2_to_f16x2(packed[1]), bf16x2_to_f16x2(packed[2]),
                       bf16x2_to_f16x2(packed[3]));
    }
}

cudaError_t launch_attention(const void* query, const void* query_gate_projection, const void* key_cache,
                             const void* value_cache, const void* block_tables, const void* context_lengths,
                             const float* key_scales, const float* value_scales, void* output, void* workspace,
                             size_t workspace_bytes, int rows, int row_base, int max_blocks, int page_size,
                             int gate_stride, int partitions, float softmax_scale, cudaStream_t stream,
                             void* staged_output = nullptr) {
    if (gate_stride == 0) {
        gate_stride = kQueryHeads * 2 * kHeadDim;
    }
    if (gate_stride < kQueryHeads * 2 * kHeadDim || gate_stride % 8 != 0) {
        return cudaErrorInvalidValue;
    }
    if (query == nullptr || key_cache == nullptr || value_cache == nullptr || block_tables == nullptr ||
        context_lengths == nullptr || (output == nullptr && staged_output == nullptr) ||
        (staged_output != nullptr && row_base + rows > 32) || rows <= 0 || rows > kPlanRows || row_base < 0 ||
        max_blocks <= 0 || partitions <= 0 || partitions > 65535 || !isfinite(softmax_scale) ||
        softmax_scale <= 0.0f || (page_size != 16 && page_size != 64)) {
        return cudaErrorInvalidValue;
    }
    int* status = status_ptr();
    if (status == nullptr) {
        return cudaErrorInvalidValue;
    }
    const size_t shared = sizeof(Smem);
    static PerDevice<cudaError_t> opted_per_device;
    const cudaError_t* opted = opted_per_device.get([shared]() {
        const cudaError_t direct =
            cudaFuncSetAttribute(paged_attention_packed_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(shared));
        if (direct != cudaSuccess) {
            return direct;
        }
        return cudaFuncSetAttribute(paged_attention_packed_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(shared));
    });
    if (opted == nullptr) {
        return cudaErrorInvalidDevice;
    }
    if (*opted != cudaSuccess) {
        return *opted;
    }
    // One CTA per SM, whatever the batch: the task list is cut on the device.  A CTA's list holds
    // kMaxCtaTasks entries; the plan gives it at most kPlanPaddingDivisor + 2 plus one per row and
    // kv head and CTA (undivided rows: one per row and kv head and CTA).
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
        return cudaErrorInvalidDevice;
    }
    if ((rows * kKvHeads + sms - 1) / sms + kPlanPaddingDivisor + 2 > kMaxCtaTasks) {
        return cudaErrorInvalidValue;
    }
    const dim3 grid(sms);
    const int padded_rows = row_base + rows <= 16 ? 16 : 32;  // of the staged output
    if (partitions == 1) {
        return qwc::launch_chained(paged_attention_packed_kernel<false>, dim3(grid), dim3(kThreads), shared, stream, 
            static_cast<const __nv_bfloat16*>(query), static_cast<const __nv_bfloat16*>(query_gate_projection),
            static_cast<const uint8_t*>(key_cache), static_cast<const uint8_t*>(value_cache),
            static_cast<const uint32_t*>(block_tables), static_cast<const uint32_t*>(context_lengths), key_scales,
            value_scales, static_cast<__nv_bfloat16*>(output), static_cast<__half*>(staged_output), padded_rows,
            nullptr, nullptr, rows, max_blocks, row_base, page_size, gate_stride, 1, softmax_scale, status);
    }
    const size_t partials = static_cast<size_t>(rows) * kQueryHeads * partitions;
    if (workspace == nullptr || workspace_bytes < partials * kPartialBytes) {
        return cudaErrorInvalidValue;
    }
    // partials is a multiple of 24, so the f16 block starts on a 16-byte boundary.
    float* partial_stats = static_cast<float*>(workspace);
    __half* partial_out = reinterpret_cast<__half*>(partial_stats + partials * kPartialFloats);
    const cudaError_t launched = qwc::launch_chained(paged_attention_packed_kernel<true>, dim3(grid), dim3(kThreads), shared, stream, 
        static_cast<const __nv_bfloat16*>(query), static_cast<const __nv_bfloat16*>(query_gate_projection),
        static_cast<const uint8_t*>(key_cache), static_cast<const uint8_t*>(value_cache),
        static_cast<const uint32_t*>(block_tables), static_cast<const uint32_t*>(context_lengths), key_scales,
        value_scales, static_cast<__nv_bfloat16*>(output), nullptr, padded_rows, partial_stats, partial_out, rows,
        max_blocks, row_base, page_size, gate_stride, partitions, softmax_scale, status);
    if (launched != cudaSuccess) {
        return launched;
    }
    const int pairs = rows * kQueryHeads;
    return qwc::launch_chained(reduce_partitions_kernel, dim3(pairs), dim3(kMergeWarps * 32), 0, stream, 
        partial_stats, partial_out, static_cast<const __nv_bfloat16*>(query_gate_projection),
        static_cast<const uint32_t*>(context_lengths), static_cast<__nv_bfloat16*>(output),
        static_cast<__half*>(staged_output), padded_rows, rows, partitions, row_base, gate_stride,
        max_blocks * (page_size / kUnitTokens), sms);
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

extern "C" int qwc_paged_attention_packed_fp8_staged(const void* query, const void* query_gate_projection,
                                                     const void* key_cache, const void* value_cache,
                                                     const void* block_tables, const void* context_lengths,
                                                     const float* key_scales, const float* value_scales,
                                                     void* output, void* staged_output, void* workspace,
                                                     size_t workspace_bytes, int rows, int row_base, int max_blocks,
                                                     int page_size, int gate_stride, int partitions,
                                                     float softmax_scale, cudaStream_t stream) {
    return qwc::launch_attention(query, query_gate_projection, key_cache, value_cache, block_tables,
                                 context_lengths, key_scales, value_scales, output, workspace, workspace_bytes,
                                 rows, row_base, max_blocks, page_size, gate_stride, partitions, softmax_scale,
                                 stream, staged_output);
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
    // Every partial slot the merge reads was written by this call (the merge recomputes which of
    // a row's slots the attention kernel used), so nothing left over from an earlier call is read
    // and nothing needs clearing first.
    return qwc::launch_attention(query, query_gate_projection, key_cache, value_cache, block_tables,
                                 context_lengths, key_scales, value_scales, output, scratch,
                                 qwc::kStaticScratchBytes, rows, row_base, max_blocks, page_size, gate_stride,
                                 partitions, softmax_scale, stream);
}

extern "C" int qwc_paged_attention_packed_noalloc_max_pairs(void) { return qwc::kStaticPartialPairs; }
