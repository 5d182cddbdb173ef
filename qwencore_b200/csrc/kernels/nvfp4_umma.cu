// NVFP4 W4A16 skinny GEMM for up to 32 activation rows on the 5th-generation tensor cores, and the
// FP8 vocabulary head through the same pipeline.
//
// Same contract as nvfp4_gemv.cu (crates/qwc-cuda/cuda/nvfp4.cu:489-537, :585-643); this file
// serves the batches where the legacy mma.sync path runs out of tensor throughput: a profile of
// that kernel shows its HMMA pipe at 15 % for 8 rows at 40 % of HBM bandwidth, i.e. above 100 %
// for 32 rows at full bandwidth.  Here the product runs as tcgen05.mma (M = 128 weight rows,
// N = 16 or 32 activation rows, K = 16 per instruction, f16 inputs, fp32 accumulators in TMEM).
//
// One CTA per SM works on two 128-row tiles (plain GEMV: 256 consecutive rows; SwiGLU: the gate
// rows and the up rows of the same 128 outputs) and a K slice; K slices of one row group form a
// thread-block cluster and are reduced through distributed shared memory.  K is walked in stages
// of 256 elements (two 128-element chunks).
//
//   warps 0-15  dequantise.  Thread = one weight row = one TMEM lane; warps 0-7 take the even
//               chunks, warps 8-15 the odd ones.  A thread reads 64 bytes of its row per chunk
//               from the shared-memory ring, widens e2m1 pairs with the hardware converter,
//               multiplies by the e4m3 block scale in f16 (exact) and writes the 128 scaled
//               weights as the A operand into one of three TMEM buffers with tcgen05.st.
//   warp 16     producer: per stage one tiled TMA copy per tile (a box of 128 rows x 128 bytes,
//               128-byte swizzle, so that the row-per-thread reads above are free of bank
//               conflicts) and one bulk copy of the swizzled scale tiles (contiguous over K for a
//               128-row block), into a four-stage ring.  One instruction moves 16 KiB: a copy
//               per weight row is limited by the copy issue rate, not by HBM.
//   warps 17-18 issue tcgen05.mma, one warp per tile: A from TMEM, B (activations, K-major core
//               matrices) from shared memory, and tcgen05.commit to hand buffers back.  The
//               instructions sit in an elect.sync region: issued from `lane == 0` they cost three
//               times as many cycles each.
//   warps 19-26 convert the activation rows bf16 -> f16 into the B layout; two warps share operand
//               stage w and every fourth chunk, and the first of them fetches the bf16 rows of the
//               next chunk with two tiled TMA copies as soon as both have read the current one.
//
// Vocabulary-head mode (crates/qwc-cuda/cuda/vocab_fp8.cu:255: e4m3 bytes [vocab][hidden], one fp32
// scale per row, fp32 logits): a stage is one 128-element chunk (the same 128-byte box), there are
// no block scales, each dequantising set reads every other stage, and the row scale multiplies the
// accumulator in the epilogue.
//
// When the caller has named the projection that follows (qwc_nvfp4_prefetch_next), the producer's
// last act is to ask L2 for the first stages of that launch's CTAs (tiled TMA prefetches without a
// shared-memory destination), so that HBM keeps streaming while this launch works off its ring and
// the next launch finds its first boxes in L2.
//
// Every wait is bounded; a wait that gives up records a code in the status word, the CTA skips
// its stores, frees its TMEM and returns.

#include <cooperative_groups.h>

#include "tcgen05.cuh"

namespace cg = cooperative_groups;

namespace qwc {
namespace {

constexpr int kChunkK = 128;                  // K elements per chunk
constexpr int kStageChunks = 2;               // chunks per weight stage: 128 bytes of nibbles per row
constexpr int kBoxRowBytes = 128;
constexpr int kTileRows = 128;
constexpr int kTiles = 2;
constexpr int kBoxBytes = kTileRows * kBoxRowBytes;       // 16 KiB, multiple of the 1 KiB swizzle period
constexpr int kScaleStageBytes = kStageChunks * 2 * 512;  // scale tiles of 512 bytes per 128-row block and 64 K
constexpr int kTileStageBytes = kBoxBytes + kScaleStageBytes;
constexpr int kWeightStages = 4;
constexpr int kXStages = 4;
constexpr int kRawBuffers = 1;  // bf16 chunks in flight per converting warp (cp.async)
constexpr int kABuffers = 3;
constexpr int kRowWarps = 8;                     // one thread per weight row of the two tiles
constexpr int kDequantSets = 2;                  // set s dequantises the chunks with index = s (mod 2)
constexpr int kDequantWarps = kRowWarps * kDequantSets;
constexpr int kProducerWarp = kDequantWarps;
constexpr int kMmaWarp = kDequantWarps + 1;
static_assert(kDequantSets == kStageChunks, "each dequantising warp reads one chunk of every stage");
constexpr int kConvertWarps = 8;               // two per operand stage: each converts half of a chunk's units
constexpr int kMmaWarps = 2;  // one issuing warp per tile
constexpr int kFirstConvertWarp = kMmaWarp + kMmaWarps;
constexpr int kThreads = (kDequantWarps + 1 + kMmaWarps + kConvertWarps) * 32;
constexpr int kTmemColumns = 512;
constexpr int kAccumulatorColumn = kABuffers * 64;
constexpr int kAccumulators = 1;  // independent accumulation chains per tile, summed in the epilogue
constexpr int kTileColumns = kAccumulatorColumn + 32 * kAccumulators;  // three 64-column A buffers + the accumulators
static_assert(kTiles * kTileColumns <= kTmemColumns, "tensor memory budget");
static_assert(kTileStageBytes % 1024 == 0, "swizzled boxes start on 1 KiB boundaries");

struct UmmaParams {
    const uint8_t* packed[2];
    const uint8_t* scales[2];
    const __nv_bfloat16* x;
    __nv_bfloat16* y;
    float inverse_scale[2];
    int out_features;
    int in_features;
    int batch;
    int n_pad;       // 16 or 32
    int swiglu;
    int row_groups;  // 128-row (swiglu) or 256-row groups
    int splits;
    int* status;
    // FP8 rows (the vocabulary head): e4m3 weights, one byte per element, no block scales; a stage
    // then holds one 128-element chunk per row instead of two; fp32 output times a per-row scale.
    int fp8;
    const float* row_scales;
    float* y_f32;
    // The projection that this stream runs next, when the caller has named it: every CTA asks L2 for
    // the first stages of some of that launch's CTAs once its own last stage is on its way, so that
    // HBM keeps streaming while this launch drains its ring and the next one starts.
    struct Next {
        int valid;
        int swiglu;
        int nvfp4;  // block scales to fetch as well
        int out_features;
        int ctas;       // row groups x splits of that launch
        int splits;
        int stages_in_k;
        int group_blocks;
        const uint8_t* scales[2];
    } next;
};


struct Barriers {
    uint64_t w_full[kWeightStages];
    uint64_t w_empty[kWeightStages];
    uint64_t a_ready[kTiles][kABuffers];
    uint64_t a_free[kTiles][kABuffers];
    uint64_t x_full[kXStages];
    uint64_t x_free[kXStages];
    uint64_t d_ready;
    uint64_t tmem_ready;
    uint64_t raw_full[kXStages];
    uint32_t tmem_base;
    int failed;
};

// The polling loop is kept out of line: it is inlined at no call site, so the roles' main loops stay
// short for the instruction caches; a wait that is already satisfied costs one test.
__device__ __noinline__ bool wait_or_fail_slow(uint64_t* bar, uint32_t parity, Barriers* b, int* status) {
    const long long start = clock64();
    for (;;) {
#pragma unroll 1
        for (int spin = 0; spin < 64; ++spin) {
            if (mbar_try_wait(bar, parity)) {
                return true;
            }
        }
        if (*reinterpret_cast<volatile int*>(&b->failed) != 0) {
            return false;
        }
        if (clock64() - start > 40000000ll) {
            break;
        }
    }
    atomicCAS(status, 0, kStatusGemvWait);
    *reinterpret_cast<volatile int*>(&b->failed) = 1;
    return false;
}

__device__ __forceinline__ bool wait_or_fail(uint64_t* bar, uint32_t parity, Barriers* b, int* status) {
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    return wait_or_fail_slow(bar, parity, b, status);
}

// The mode (vocabulary head, SwiGLU pair), the padded batch and whether K is split are template parameters: every
// instantiation carries only its own code, which the instruction caches of an SM with five kinds of
// warps per scheduler repay.
template <bool kFp8, bool kSwiglu, int kPad, bool kSplit>
__global__ void __launch_bounds__(kThreads, 1)
    nvfp4_umma_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                      const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap next_map0,
                      const __grid_constant__ CUtensorMap next_map1, const UmmaParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ Barriers bars;
    // 128-byte-swizzled boxes need a 1 KiB-aligned shared address.
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int splits = kSplit ? p.splits : 1;  // K slices of a row group = CTAs of the cluster
    const int row_group = blockIdx.x / splits;
    const int split = blockIdx.x - row_group * splits;
    const int K = p.in_features;
    // K is cut into stages of 256 elements; a slice is a whole number of stages.
    const int stage_chunks = kFp8 ? 1 : kStageChunks;  // 128 bytes per row and stage either way
    const int stages_in_k = K / (kChunkK * stage_chunks);
    // stages_in_k * 8 fits 32 bits for every K an int can hold
    const int s_begin = stages_in_k * split / splits;
    const int s_end = stages_in_k * (split + 1) / splits;
    const int num_wstages = s_end - s_begin;
    const int total_chunks = num_wstages * stage_chunks;
    const int group_blocks = K / 64;
    constexpr int n_pad = kPad;  // activation rows padded to 16 or 32
    const int x_stage_bytes = n_pad * kChunkK * 2;

    unsigned char* weight_ring = smem;                                                   // [stage][tile][box | scales]
    unsigned char* x_ring = smem + kWeightStages * kTiles * kTileStageBytes;             // [xstage][...]
    unsigned char* raw_ring = x_ring + kXStages * 32 * kChunkK * 2;                      // [warp][two boxes of 32 rows x 128 B, swizzled]

    // First row of each tile and the matrix it comes from.
    int tile_row0[kTiles];
    const uint8_t* tile_scales[kTiles];
#pragma unroll
    for (int t = 0; t < kTiles; ++t) {
        tile_row0[t] = kSwiglu ? row_group * kTileRows : (row_group * kTiles + t) * kTileRows;
        tile_scales[t] = p.scales[t];  // the launcher repeats matrix 0 when there is no second one
    }

    // One stage of the weight ring: a box per tile and the tiles' block scales (issued by one thread).
    auto issue_stage = [&](int wstage) {
        const int slot = wstage % kWeightStages;
        const int first = (s_begin + wstage) * kStageChunks;  // first 128-element chunk of this stage
        constexpr int n = kStageChunks;
        // A box is always delivered whole (rows or bytes outside the matrix arrive as zeros)
        // and the scale storage is padded to whole 128-row blocks; a tile that starts past
        // the matrix has no scale block at all and keeps whatever the slot held (its rows
        // are never stored).
        int scale_tiles_present = 0;
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {
            scale_tiles_present += tile_row0[t] < p.out_features ? 1 : 0;
        }
        if (kFp8) {
            scale_tiles_present = 0;  // one float per row, applied in the epilogue
        }
        mbar_arrive_expect_tx(&bars.w_full[slot], kTiles * kBoxBytes + scale_tiles_present * n * 1024);
        // Byte offset of the stage within a row: 64 bytes per 128 four-bit elements, or one
        // 128-byte box per 128 e4m3 elements.
        const int byte0 = kFp8 ? (s_begin + wstage) * 128 : first * 64;
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {
            unsigned char* stage = weight_ring + (slot * kTiles + t) * kTileStageBytes;
            tma_box_g2s(stage, t == 1 ? &map1 : &map0, byte0, tile_row0[t], &bars.w_full[slot]);
            if (!kFp8 && tile_row0[t] < p.out_features) {
                bulk_g2s(stage + kBoxBytes,
                         tile_scales[t] + (static_cast<size_t>(tile_row0[t] >> 7) * group_blocks + 2 * first) * 512,
                         n * 1024, &bars.w_full[slot]);
            }
        }
    };
    // The first trip round the weight ring does not wait for the rest of the CTA: the producer's
    // thread sets up the ring's own barriers and asks for the first stages before the CTA-wide barrier
    // (weights are never written during a step, so nothing has to be waited for either).
    const int early_stages = num_wstages < kWeightStages ? num_wstages : kWeightStages;
    if (threadIdx.x == kProducerWarp * 32) {
        for (int s = 0; s < kWeightStages; ++s) {
            mbar_init(&bars.w_full[s], 1);
            mbar_init(&bars.w_empty[s], kFp8 ? kRowWarps : kDequantWarps);  // warps that read a stage
        }
        mbar_fence_init();
        for (int wstage = 0; wstage < early_stages; ++wstage) {
            issue_stage(wstage);
        }
    }
    if (threadIdx.x == 0) {
        for (int t = 0; t < kTiles; ++t) {
            for (int b = 0; b < kABuffers; ++b) {
                mbar_init(&bars.a_ready[t][b], 4);
                mbar_init(&bars.a_free[t][b], 1);
            }
        }
        for (int s = 0; s < kXStages; ++s) {
            mbar_init(&bars.x_full[s], kConvertWarps / kXStages);
            mbar_init(&bars.x_free[s], kMmaWarps);
        }
        mbar_init(&bars.d_ready, kMmaWarps);
        mbar_init(&bars.tmem_ready, 1);
        for (int s = 0; s < kXStages; ++s) {
            mbar_init(&bars.raw_full[s], 1);
        }
        bars.failed = status_is_set(p.status) ? 1 : 0;
        bars.tmem_base = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // Tensor memory is allocated while the producer already fetches weights and the converting warps
    // activations; the warps that use it wait for the address below.
    uint32_t tmem_base = 0;
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars.tmem_base)),
                     "r"(kTmemColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(&bars.tmem_ready);
        }
    }
    bool tmem_ok = true;
    if (warp < kFirstConvertWarp && warp != kProducerWarp) {
        tmem_ok = wait_or_fail(&bars.tmem_ready, 0, &bars, p.status);
        tmem_ok = __all_sync(0xffffffffu, tmem_ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars.tmem_base);
    }

    float result[32];
    bool have_result = false;

    if (warp < kDequantWarps) {
        // ---------------- dequantise: thread = row ----------------
        const int set = warp / kRowWarps;
        const int tile = (warp >> 2) & 1;
        const int quarter = warp & 3;
        const int local_row = quarter * 32 + lane;
        const uint32_t lane_address = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + tile * kTileColumns;
        const int row_offset = local_row * kBoxRowBytes;
        const int row_swizzle = local_row & 7;
        const int scale_offset = (local_row & 31) * 16 + (local_row >> 5) * 4;
        bool ok = tmem_ok;
        int previous_buf = -1;
        int previous_slot = -1;  // >= 0: the previous chunk was the last reader of that ring slot
        // Hands a finished chunk to the tensor-core warp and its ring slot back to the producer.
        auto retire_previous = [&]() {
            if (previous_buf >= 0) {
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars.a_ready[tile][previous_buf]);
                    if (previous_slot >= 0) {
                        mbar_arrive(&bars.w_empty[previous_slot]);
                    }
                }
                previous_buf = -1;
                previous_slot = -1;
            }
        };
        for (int c = set; c < total_chunks && ok; c += kDequantSets) {
            const int wstage = kFp8 ? c : c / kStageChunks;
            const int slot = wstage % kWeightStages;
            const int q = set;
            ok = wait_or_fail(&bars.w_full[slot], (wstage / kWeightStages) & 1, &bars, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            const unsigned char* stage = weight_ring + (slot * kTiles + tile) * kTileStageBytes;
            const unsigned char* row = stage + row_offset;
            const int buf = c % kABuffers;
            if (kFp8) {
                // 128 e4m3 bytes of this row: one conversion per pair, no block scale (the per-row
                // scale is applied to the accumulator in the epilogue)
                uint4 bytes[8];
#pragma unroll
                for (int piece = 0; piece < 8; ++piece) {
                    bytes[piece] = *reinterpret_cast<const uint4*>(row + ((piece ^ row_swizzle) << 4));
                }
                ok = wait_or_fail(&bars.a_free[tile][buf], ((c / kABuffers) & 1) ^ 1, &bars, p.status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int part = 0; part < 4; ++part) {
                    uint32_t out[16];
#pragma unroll
                    for (int piece = 0; piece < 2; ++piece) {
                        const uint4 raw = bytes[2 * part + piece];
                        cvt_e4m3x4_to_f16x2(raw.x, out[8 * piece + 0], out[8 * piece + 1]);
                        cvt_e4m3x4_to_f16x2(raw.y, out[8 * piece + 2], out[8 * piece + 3]);
                        cvt_e4m3x4_to_f16x2(raw.z, out[8 * piece + 4], out[8 * piece + 5]);
                        cvt_e4m3x4_to_f16x2(raw.w, out[8 * piece + 6], out[8 * piece + 7]);
                    }
                    tmem_store16(lane_address + buf * 64 + part * 16, out);
                }
            } else {
            const unsigned char* scale_tiles = stage + kBoxBytes + q * 1024 + scale_offset;
            uint4 raw[4];
#pragma unroll
            for (int part = 0; part < 4; ++part) {
                raw[part] = *reinterpret_cast<const uint4*>(row + (((q * 4 + part) ^ row_swizzle) << 4));
            }
            // 8 block scales of this chunk: two words of four e4m3 (cuda/nvfp4.cu:33-39 layout)
            const uint32_t scale_word0 = *reinterpret_cast<const uint32_t*>(scale_tiles);
            const uint32_t scale_word1 = *reinterpret_cast<const uint32_t*>(scale_tiles + 512);
            ok = wait_or_fail(&bars.a_free[tile][buf], ((c / kABuffers) & 1) ^ 1, &bars, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t scale2[8];
#pragma unroll
            for (int gb = 0; gb < 2; ++gb) {
                uint32_t lo, hi;
                cvt_e4m3x4_to_f16x2(gb == 0 ? scale_word0 : scale_word1, lo, hi);
                scale2[gb * 4 + 0] = __byte_perm(lo, 0, 0x1010);
                scale2[gb * 4 + 1] = __byte_perm(lo, 0, 0x3232);
                scale2[gb * 4 + 2] = __byte_perm(hi, 0, 0x1010);
                scale2[gb * 4 + 3] = __byte_perm(hi, 0, 0x3232);
            }
#pragma unroll
            for (int part = 0; part < 4; ++part) {
                const uint32_t words[4] = {raw[part].x, raw[part].y, raw[part].z, raw[part].w};
                uint32_t out[16];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t h[4];
                    cvt_e2m1x8_to_f16x2(words[i], h);
                    const uint32_t s = scale2[part * 2 + (i >> 1)];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        out[i * 4 + j] = hmul2_bits(h[j], s);
                    }
                }
                tmem_store16(lane_address + buf * 64 + part * 16, out);
            }
            }
            previous_buf = buf;
            previous_slot = slot;  // this warp reads one chunk per stage
            retire_previous();
        }
        if (ok && set == 0) {
            ok = wait_or_fail(&bars.d_ready, 0, &bars, p.status);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok && set == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // n_pad == 16 reads 32 columns too; the upper half is unused TMEM of this tile
            tmem_load32(lane_address + kAccumulatorColumn, result);
#pragma unroll
            for (int extra = 1; extra < kAccumulators; ++extra) {
                float more[32];
                tmem_load32(lane_address + kAccumulatorColumn + extra * 32, more);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    result[i] += more[i];
                }
            }
            have_result = true;
        }
    } else if (warp == kProducerWarp) {
        // ---------------- producer: weights and scales ----------------
        bool ok = true;
        for (int wstage = early_stages; wstage < num_wstages && ok; ++wstage) {
            const int slot = wstage % kWeightStages;
            ok = wait_or_fail(&bars.w_empty[slot], ((wstage / kWeightStages) & 1) ^ 1, &bars, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            if (elect_one()) {
                issue_stage(wstage);
            }
            __syncwarp();
        }
        if (ok && p.next.valid && elect_one()) {
            for (int cta = blockIdx.x; cta < p.next.ctas; cta += gridDim.x) {
                const int group = cta / p.next.splits;
                const int slice = cta - group * p.next.splits;
                const int first_stage =
                    static_cast<int>(static_cast<long long>(p.next.stages_in_k) * slice / p.next.splits);
                const int end_stage =
                    static_cast<int>(static_cast<long long>(p.next.stages_in_k) * (slice + 1) / p.next.splits);
                const int stages = min(kWeightStages, end_stage - first_stage);
#pragma unroll
                for (int t = 0; t < kTiles; ++t) {
                    const int row0 = p.next.swiglu ? group * kTileRows : (group * kTiles + t) * kTileRows;
                    if (row0 >= p.next.out_features) {
                        continue;
                    }
                    for (int st = 0; st < stages; ++st) {
                        tma_box_prefetch_l2(t == 1 ? &next_map1 : &next_map0, (first_stage + st) * kBoxRowBytes, row0);
                        if (p.next.nvfp4) {
                            bulk_prefetch_l2(p.next.scales[t] + (static_cast<size_t>(row0 >> 7) * p.next.group_blocks +
                                                                 2 * kStageChunks * (first_stage + st)) * 512,
                                             kStageChunks * 1024);
                        }
                    }
                }
            }
        }
    } else if (warp < kFirstConvertWarp) {
        // ---------------- tensor-core issue ----------------
        // One warp per tile.  The whole warp waits; only the instructions themselves sit in the
        // elected lane's region, which the compiler then runs on the uniform datapath.
        const int t = warp - kMmaWarp;
        const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(n_pad >> 3) << 17) | (8u << 24);
        // K cores are n_pad * 16 bytes apart, 8-row groups 128 bytes; one instruction takes two K cores
        const uint64_t desc_base = smem_descriptor(smem_u32(x_ring), n_pad * 16, 128);
        const uint64_t desc_step = static_cast<uint64_t>((2 * n_pad * 16) >> 4);
        const uint64_t desc_stage = static_cast<uint64_t>(x_stage_bytes >> 4);
        const uint32_t a_tile = tmem_base + t * kTileColumns;
        const uint32_t d_tile = a_tile + kAccumulatorColumn;
        bool ok = tmem_ok;
        int buf = 0, xs = 0;
        uint32_t a_parity = 0, x_parity = 0;
        for (int c = 0; c < total_chunks && ok; ++c) {
            ok = wait_or_fail(&bars.x_full[xs], x_parity, &bars, p.status);
            if (ok) {
                ok = wait_or_fail(&bars.a_ready[t][buf], a_parity, &bars, p.status);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (elect_one()) {
                uint64_t b_desc = desc_base + desc_stage * xs;
                const uint32_t a0 = a_tile + buf * 64;
                const uint32_t later = c > 0 ? 1u : 0u;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    umma_f16(d_tile + (s % kAccumulators) * 32, a0 + s * 8, b_desc, idesc, s >= kAccumulators ? 1u : later);
                    b_desc += desc_step;
                }
                umma_commit(&bars.a_free[t][buf]);
                umma_commit(&bars.x_free[xs]);
                if (c == total_chunks - 1) {
                    umma_commit(&bars.d_ready);
                }
            }
            __syncwarp();
            if (++buf == kABuffers) {
                buf = 0;
                a_parity ^= 1;
            }
            if (++xs == kXStages) {
                xs = 0;
                x_parity ^= 1;
            }
        }
    } else {
        // ---------------- activation rows: bf16 -> f16, K-major core matrices ----------------
        // Converting warp w owns operand stage w and the chunks w, w + 4, ...  The bf16 rows of a
        // chunk come by two tiled TMA copies (boxes of 32 rows x 64 elements with the 128-byte
        // swizzle; rows past the batch arrive as zeros) which the warp itself issues for its next
        // chunk as soon as it has read the current one: no load instruction and no address
        // arithmetic per element is spent on fetching.  Then lane = activation row (two half-warps
        // take the two halves of the K cores when only 16 rows are padded in): load 16 bytes,
        // convert, store in the operand layout (K cores n_pad * 16 bytes apart, rows 16 bytes apart).
        static_assert(kConvertWarps == 2 * kXStages, "two converting warps per operand stage");
        static_assert(kRawBuffers == 1, "the staging slot is refilled after it has been read");
        const int w = (warp - kFirstConvertWarp) % kXStages;   // operand stage and staging slot
        const int part = (warp - kFirstConvertWarp) / kXStages;  // which half of the units this warp converts
        const int token = lane & (n_pad - 1);
        const int half = n_pad == 16 ? lane >> 4 : 0;
        const int units = n_pad == 16 ? 8 : 16;          // 16-byte units per lane and chunk, both warps together
        const int unit_step = n_pad == 16 ? 2 : 1;       // K cores between a lane's units
        unsigned char* raw_slot = raw_ring + w * (32 * kChunkK * 2);
        const uint32_t raw_row = smem_u32(raw_slot) + token * 128;
        unsigned char* stage = x_ring + w * x_stage_bytes + half * (n_pad * 16) + (token >> 3) * 128 + (token & 7) * 16;
        auto fetch = [&](int c) {  // chunk c of this CTA's slice, c = w (mod 4); issued by the part-0 warp
            if (part == 0 && c < total_chunks && elect_one()) {
                const int k0 = (s_begin * stage_chunks + c) * kChunkK;
                mbar_arrive_expect_tx(&bars.raw_full[w], 32 * kChunkK * 2);
                tma_box_g2s(raw_slot, &x_map, k0, 0, &bars.raw_full[w]);
                tma_box_g2s(raw_slot + 32 * 128, &x_map, k0 + 64, 0, &bars.raw_full[w]);
            }
            __syncwarp();
        };
        bool ok = true;
        // Weights, scales and the whole pipeline above start before the kernel that produces the
        // activations has finished; only these loads wait for it.
        pdl_wait();
        fetch(w);
        uint32_t parity = 1;      // the first use of an operand stage finds it free
        uint32_t raw_parity = 0;
        for (int c = w; c < total_chunks && ok; c += kXStages) {
            ok = wait_or_fail(&bars.raw_full[w], raw_parity, &bars, p.status);
            if (ok) {
                ok = wait_or_fail(&bars.x_free[w], parity, &bars, p.status);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = 2 * j + part;  // the two warps of a stage take alternate units
                if (i < units) {
                    const int kcore = i * unit_step + half;  // 16-byte piece of the row's 256-byte chunk
                    uint4 raw;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                                 : "r"(raw_row + (kcore >> 3) * (32 * 128) + (((kcore & 7) ^ (token & 7)) << 4)));
                    *reinterpret_cast<uint4*>(stage + i * 512) = make_uint4(
                        bf16x2_to_f16x2(raw.x), bf16x2_to_f16x2(raw.y), bf16x2_to_f16x2(raw.z), bf16x2_to_f16x2(raw.w));
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars.x_full[w]);
            }
            if (part == 0 && c + kXStages < total_chunks) {
                // the staging slot may be refilled once both warps have read it: that is when the
                // operand stage's barrier completes its phase
                ok = wait_or_fail(&bars.x_full[w], parity ^ 1, &bars, p.status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    break;
                }
            }
            parity ^= 1;
            raw_parity ^= 1;
            fetch(c + kXStages);
        }
    }

    // ---------------- split-K reduction, epilogue ----------------
    // Every CTA of the cluster parks its accumulators in its own shared memory ([token][row], fp32;
    // the weight ring is idle now).  Then the tokens are dealt out: CTA s sums, over all slices and in
    // slice order, the tokens s, s + splits, ... and stores them, eight consecutive rows (16 bytes of
    // bf16) per thread.  One CTA reading every peer for all tokens takes several microseconds.
    __syncthreads();
    const bool failed = *reinterpret_cast<volatile int*>(&bars.failed) != 0;
    cg::cluster_group cluster = cg::this_cluster();
    float* parked = reinterpret_cast<float*>(smem);  // [32][256]
    constexpr int kParkedRows = kRowWarps * 32;
    if (have_result) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            parked[i * kParkedRows + threadIdx.x] = result[i];
        }
    }
    if (kSplit) {
        cluster.sync();
    } else {
        __syncthreads();
    }
    // Every warp of the CTA takes part: the loop is a chain of dependent instructions per unit (and a
    // division and an exponential per output for SwiGLU), so the more units run side by side the
    // sooner the CTA leaves.
    if (!failed) {
        const int unit_shift = kSwiglu ? 4 : 5;  // 8-row units per token: 16 (128 outputs) or 32 (256)
        const int row0 = kSwiglu ? row_group * kTileRows : row_group * kTiles * kTileRows;
        const int owned = split < p.batch ? (p.batch - split + splits - 1) / splits : 0;
        const auto slice_base = [&](int r) -> const float* {
            return kSplit ? cluster.map_shared_rank(parked, r) : parked;
        };
        for (int u = threadIdx.x; u < (owned << unit_shift); u += kThreads) {
            const int token = split + (u >> unit_shift) * splits;
            const int r8 = (u & ((1 << unit_shift) - 1)) * 8;
            float first[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            float second[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};  // the up rows of a SwiGLU pair
            // A load from a peer's shared memory is a round trip through the cluster network: the loads
            // of four slices are issued together and only then summed (in slice order, as before), so a
            // six-way split waits for two round trips instead of six.
            const int offset = token * kParkedRows + r8;
            for (int base = 0; base < splits; base += 4) {
                float4 a[4], b[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (base + j < splits) {
                        const float* peer = slice_base(base + j) + offset;
                        a[j] = *reinterpret_cast<const float4*>(peer);
                        b[j] = *reinterpret_cast<const float4*>(peer + 4);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (base + j < splits) {
                        first[0] += a[j].x; first[1] += a[j].y; first[2] += a[j].z; first[3] += a[j].w;
                        first[4] += b[j].x; first[5] += b[j].y; first[6] += b[j].z; first[7] += b[j].w;
                    }
                }
                if (kSwiglu) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (base + j < splits) {
                            const float* peer = slice_base(base + j) + offset + kTileRows;
                            a[j] = *reinterpret_cast<const float4*>(peer);
                            b[j] = *reinterpret_cast<const float4*>(peer + 4);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (base + j < splits) {
                            second[0] += a[j].x; second[1] += a[j].y; second[2] += a[j].z; second[3] += a[j].w;
                            second[4] += b[j].x; second[5] += b[j].y; second[6] += b[j].z; second[7] += b[j].w;
                        }
                    }
                }
            }
            const int row = row0 + r8;
            if (row < p.out_features && kFp8) {
                // vocabulary head: fp32 logits, one scale per weight row
                const float4 s_lo = *reinterpret_cast<const float4*>(p.row_scales + row);
                const float4 s_hi = *reinterpret_cast<const float4*>(p.row_scales + row + 4);
                float* out = p.y_f32 + static_cast<size_t>(token) * p.out_features + row;
                *reinterpret_cast<float4*>(out) =
                    make_float4(first[0] * s_lo.x, first[1] * s_lo.y, first[2] * s_lo.z, first[3] * s_lo.w);
                *reinterpret_cast<float4*>(out + 4) =
                    make_float4(first[4] * s_hi.x, first[5] * s_hi.y, first[6] * s_hi.z, first[7] * s_hi.w);
            } else if (row < p.out_features) {  // out_features is a multiple of 8: a unit is inside or outside
                uint32_t packed[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float lo = first[2 * i] * p.inverse_scale[0];
                    float hi = first[2 * i + 1] * p.inverse_scale[0];
                    if (kSwiglu) {
                        lo = lo / (1.0f + __expf(-lo)) * (second[2 * i] * p.inverse_scale[1]);
                        hi = hi / (1.0f + __expf(-hi)) * (second[2 * i + 1] * p.inverse_scale[1]);
                    }
                    const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
                    packed[i] = *reinterpret_cast<const uint32_t*>(&pair);
                }
                *reinterpret_cast<uint4*>(p.y + static_cast<size_t>(token) * p.out_features + row) =
                    make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
        }
    }
    if (kSplit) {
        cluster.sync();  // nobody leaves while a peer may still read its shared memory
    }

    // A CTA that gave up must not return while the stages it asked for before the barrier are still
    // landing in its shared memory: their thread waits for them, with a limit of 0.2 ms per ring slot
    // (a stage that was consumed has completed its first phase long ago and the wait falls through).
    if (failed && threadIdx.x == kProducerWarp * 32) {
        for (int slot = 0; slot < kWeightStages; ++slot) {
            const long long start = clock64();
            while (!mbar_try_wait(&bars.w_full[slot], 0) && clock64() - start < 400000ll) {
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
    }
}

int sm_count_umma() {
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) {
        int value = 0;
        if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && value > 0) {
            sms = value;
        }
    }
    return sms;
}

}  // namespace


namespace {

// Fills the launch-dependent fields of p (its operand pointers and mode are the caller's) and launches.
cudaError_t launch_umma(UmmaParams p, const void* x, int out_features, int in_features, int batch, bool swiglu,
                        cudaStream_t stream) {
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.out_features = out_features;
    p.in_features = in_features;
    p.batch = batch;
    p.n_pad = batch <= 16 ? 16 : 32;
    p.swiglu = swiglu ? 1 : 0;
    const int rows_per_group = swiglu ? kTileRows : kTiles * kTileRows;
    p.row_groups = (out_features + rows_per_group - 1) / rows_per_group;
    // bytes of one weight row: two elements per byte, or one e4m3 byte each
    const int row_bytes = p.fp8 ? in_features : in_features / 2;
    CUtensorMap map0, map1;
    cudaError_t encoded = encode_weight_map(&map0, p.packed[0], out_features, row_bytes);
    if (encoded == cudaSuccess) {
        encoded = encode_weight_map(&map1, p.packed[1], out_features, row_bytes);
    }
    if (encoded != cudaSuccess) {
        return encoded;
    }
    // The activation rows as a [batch][K] bf16 matrix, fetched in boxes of 32 rows x 64 elements.
    CUtensorMap x_map;
    {
        const EncodeTiled encode = tensor_map_encoder();
        if (encode == nullptr) {
            return cudaErrorNotSupported;
        }
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(in_features), static_cast<cuuint64_t>(batch)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(in_features) * 2};
        const cuuint32_t box[2] = {64, 32};
        const cuuint32_t element_strides[2] = {1, 1};
        if (encode(&x_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box,
                   element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            return cudaErrorInvalidValue;
        }
    }
    const int smem_bytes =
        kWeightStages * kTiles * kTileStageBytes + (kXStages + kXStages * kRawBuffers) * 32 * kChunkK * 2 + 1024;
    using Kernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                            const CUtensorMap, const UmmaParams);
    static const Kernel kernels[12] = {
        nvfp4_umma_kernel<false, false, 16, false>, nvfp4_umma_kernel<false, false, 32, false>,
        nvfp4_umma_kernel<false, true, 16, false>,  nvfp4_umma_kernel<false, true, 32, false>,
        nvfp4_umma_kernel<true, false, 16, false>,  nvfp4_umma_kernel<true, false, 32, false>,
        nvfp4_umma_kernel<false, false, 16, true>,  nvfp4_umma_kernel<false, false, 32, true>,
        nvfp4_umma_kernel<false, true, 16, true>,   nvfp4_umma_kernel<false, true, 32, true>,
        nvfp4_umma_kernel<true, false, 16, true>,   nvfp4_umma_kernel<true, false, 32, true>};
    static PerDevice<cudaError_t> opted_per_device;
    const cudaError_t* opted_found = opted_per_device.get([smem_bytes]() {
        for (const Kernel kernel : kernels) {
            const cudaError_t error =
                cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
            if (error != cudaSuccess) {
                return error;
            }
        }
        return cudaSuccess;
    });
    if (opted_found == nullptr) {
        return cudaErrorInvalidDevice;
    }
    if (*opted_found != cudaSuccess) {
        return *opted_found;
    }
    // K split: the slices of a row group form a cluster, and a cluster must sit inside one GPC, so
    // the number of clusters resident at once is asked of the driver per cluster size.  The cost of
    // a plan is its waves times the chunks per slice, plus a term for the reduction.
    struct Residency {
        int clusters[9];
    };
    static PerDevice<Residency> residency_per_device;
    const Residency* residency_found = residency_per_device.get([smem_bytes]() {
        Residency r = {};
        for (int size = 1; size <= 8; ++size) {
            cudaLaunchConfig_t probe = {};
            probe.gridDim = dim3(size * 64);
            probe.blockDim = dim3(kThreads);
            probe.dynamicSmemBytes = smem_bytes;
            cudaLaunchAttribute attribute[1];
            attribute[0].id = cudaLaunchAttributeClusterDimension;
            attribute[0].val.clusterDim.x = size;
            attribute[0].val.clusterDim.y = 1;
            attribute[0].val.clusterDim.z = 1;
            probe.attrs = attribute;
            probe.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, kernels[7], &probe) != cudaSuccess) {
                clusters = 0;
                (void)cudaGetLastError();
            }
            r.clusters[size] = clusters;
        }
        return r;
    });
    if (residency_found == nullptr) {
        return cudaErrorInvalidDevice;
    }
    const Residency& residency = *residency_found;
    const auto plan_splits = [&](int row_groups, int features_in, bool fp8) {
        const int chunks = features_in / kChunkK;
        const int stage_chunks = fp8 ? 1 : kStageChunks;
        int best = 1;
        double best_cost = 1e30;
        for (int size = 1; size <= 8; ++size) {
            const int clusters = size == 1 ? sm_count_umma() : residency.clusters[size];
            if (clusters <= 0 || (size > 1 && chunks / size < 2 * stage_chunks)) {
                continue;
            }
            const int waves = (row_groups + clusters - 1) / clusters;
            const double cost = waves * (static_cast<double>((chunks + size - 1) / size) + 6.0) + 1.5 * (size - 1);
            if (cost < best_cost) {
                best_cost = cost;
                best = size;
            }
        }
        return best;
    };
    const int splits = plan_splits(p.row_groups, in_features, p.fp8 != 0);
    p.splits = splits;
    // The caller's hint about the projection that follows (one use): its plan is made the way its own
    // launch will make it, so that this launch's CTAs ask for the boxes that launch starts with.
    CUtensorMap next_map0 = map0, next_map1 = map1;
    p.next.valid = 0;
    const NextProjection hint = take_next_projection();
    if (hint.packed[0] != nullptr && hint.out_features > 0 && hint.in_features > 0) {
        const bool next_fp8 = hint.kind == 2;
        const bool next_swiglu = hint.kind == 1 || hint.kind == 4;
        const int next_row_bytes = next_fp8 ? hint.in_features : hint.in_features / 2;
        const int next_rows_per_group = next_swiglu ? kTileRows : kTiles * kTileRows;
        const int next_groups = (hint.out_features + next_rows_per_group - 1) / next_rows_per_group;
        if (encode_weight_map(&next_map0, hint.packed[0], hint.out_features, next_row_bytes) == cudaSuccess &&
            encode_weight_map(&next_map1, hint.packed[next_swiglu ? 1 : 0], hint.out_features, next_row_bytes) ==
                cudaSuccess) {
            p.next.valid = 1;
            p.next.swiglu = next_swiglu ? 1 : 0;
            p.next.nvfp4 = next_fp8 ? 0 : 1;
            p.next.out_features = hint.out_features;
            p.next.splits = plan_splits(next_groups, hint.in_features, next_fp8);
            p.next.ctas = next_groups * p.next.splits;
            p.next.stages_in_k = hint.in_features / (kChunkK * (next_fp8 ? 1 : kStageChunks));
            p.next.group_blocks = hint.in_features / 64;
            p.next.scales[0] = static_cast<const uint8_t*>(hint.scales[0]);
            p.next.scales[1] = static_cast<const uint8_t*>(hint.scales[next_swiglu ? 1 : 0]);
        }
    }
    p.status = status_ptr();
    if (p.status == nullptr) {
        return cudaErrorInvalidValue;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(p.row_groups * splits);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = splits;
    attribute[1].val.clusterDim.y = 1;
    attribute[1].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = splits > 1 ? 2 : 1;
    const Kernel kernel = kernels[(splits > 1 ? 6 : 0) + (p.fp8 ? 4 : (p.swiglu ? 2 : 0)) + (p.n_pad == 32 ? 1 : 0)];
    return cudaLaunchKernelEx(&config, kernel, map0, map1, x_map, next_map0, next_map1, p);
}

}  // namespace

cudaError_t launch_nvfp4_umma(const void* packed0, const void* scales0, const void* packed1, const void* scales1,
                              const void* x, void* y, int out_features, int in_features, int batch, float inverse0,
                              float inverse1, bool swiglu, cudaStream_t stream) {
    UmmaParams p = {};
    p.packed[0] = static_cast<const uint8_t*>(packed0);
    p.scales[0] = static_cast<const uint8_t*>(scales0);
    p.packed[1] = static_cast<const uint8_t*>(swiglu ? packed1 : packed0);
    p.scales[1] = static_cast<const uint8_t*>(swiglu ? scales1 : scales0);
    p.y = static_cast<__nv_bfloat16*>(y);
    p.inverse_scale[0] = inverse0;
    p.inverse_scale[1] = inverse1;
    return launch_umma(p, x, out_features, in_features, batch, swiglu, stream);
}

// The vocabulary head through the same pipeline: e4m3 weight bytes [vocab][hidden], one fp32 scale per
// row, fp32 logits [batch][vocab].  hidden a multiple of 128, vocab of 8, logits 16-byte aligned.
cudaError_t launch_fp8_umma(const void* weights, const float* row_scales, const void* x, float* logits,
                            int out_features, int in_features, int batch, cudaStream_t stream) {
    UmmaParams p = {};
    p.packed[0] = p.packed[1] = static_cast<const uint8_t*>(weights);
    p.scales[0] = p.scales[1] = nullptr;
    p.fp8 = 1;
    p.row_scales = row_scales;
    p.y_f32 = logits;
    p.inverse_scale[0] = p.inverse_scale[1] = 1.0f;
    return launch_umma(p, x, out_features, in_features, batch, false, stream);
}

}  // namespace qwc
