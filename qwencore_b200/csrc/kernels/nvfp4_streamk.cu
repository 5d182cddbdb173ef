// NVFP4 W4A16 projections and the FP8 vocabulary head on the 5th-generation tensor cores, with the
// work of one launch cut into equal shares for every SM.
//
// Same arithmetic as nvfp4_umma.cu (crates/qwc-cuda/cuda/nvfp4.cu:489-537, :585-643;
// cuda/vocab_fp8.cu:255): weights are widened to f16 times their e4m3 block scale (exact) and
// written to tensor memory as the A operand of tcgen05.mma.kind::f16 (M = 128 weight rows, N = 16 or
// 32 activation rows, K = 16), fp32 accumulators in tensor memory.  What differs is who does what:
//
//   * Staged activations.  The kernels that produce activations (RMSNorm, gated RMSNorm, the
//     attention merge, the SwiGLU epilogue of this kernel) also store them as f16 in the layout the
//     tensor core reads its B operand in - K-major core matrices, [K / 8][rows padded to 16 or 32][8]
//     - so a 128-element chunk of all rows is one contiguous block of 4 or 8 KiB that a single bulk
//     copy lands in shared memory, ready for the MMA.  No warp of this kernel converts activations.
//   * Equal shares.  A launch is a line of units, (pair of 128-row tiles) x (256-element K stage),
//     pair-major.  CTA c of G (G = SM count) owns units [U c / G, U (c + 1) / G): every SM streams the
//     same number of bytes whatever the matrix shape is.  A share crosses pair boundaries, so a CTA
//     works through a list of segments; a segment that does not cover all of K leaves an fp32 partial
//     tile in a workspace in global memory (L2-resident) and takes a ticket; whoever takes the last
//     ticket of a tile sums the partials in a fixed order (bit-reproducible) and stores the result.
//     Nobody waits for anybody: there is no cluster and no barrier between CTAs.  The piece a CTA
//     ends its share with is the first piece of its pair, and the other pieces are usually long
//     finished by then: while the main loop still runs, the (idle) epilogue warps look at the
//     ticket, and if everybody else has arrived they fetch the sum of the other pieces into shared
//     memory, so that the end of the launch is one TMEM read, one addition and the stores.
//   * A drain that does not stop the stream.  Accumulators are double-buffered in tensor memory and
//     eight epilogue warps read them, so the dequantising warps and the tensor core go on with the
//     next segment while the previous one is scaled, combined (SwiGLU) and stored.
//
//   warps 0-15  dequantise.  Thread = one weight row = one TMEM lane; warps 0-7 take the even
//               128-element chunks, warps 8-15 the odd ones; three 64-column A buffers per tile.
//   warp 16     weight producer: per stage one tiled TMA copy per tile (128 rows x 128 bytes,
//               128-byte swizzle) and one bulk copy of the tile's swizzled scale blocks; 4-stage ring.
//   warps 17-18 issue tcgen05.mma, one warp per tile (elect.sync region).
//   warp 19     activation producer: one bulk copy per chunk into a 6-chunk ring; the only warp
//               besides the epilogue that waits for the previous kernel (programmatic launch).
//   warps 20-27 epilogue: warp e reads TMEM lanes 32 (e % 4) .. + 31 (those output rows) of both tiles
//               for half of the activation rows (e / 4).  Both tiles in one thread means the gate and up
//               values of a SwiGLU output meet in registers.
//
// Vocabulary head (e4m3 rows, one fp32 scale per row): a stage is one 128-element chunk, the row
// scale multiplies the accumulator in the epilogue, and the epilogue keeps, per activation row, the
// best (logit, index) it has seen, so that greedy sampling needs no logits in memory.
//
// Every wait is bounded; a wait that gives up records a code in the status word, the CTA skips its
// stores, frees its TMEM and returns.  A launch that ends that way leaves tickets taken: the
// workspace must be cleared (qwc_streamk_workspace_init) before it is used again.

#include "exchange.cuh"
#include "tcgen05.cuh"

namespace qwc {
namespace {

constexpr int kChunkK = 128;                  // K elements per chunk
constexpr int kStageChunks = 2;               // chunks per NVFP4 weight stage: 128 bytes of nibbles per row
constexpr int kBoxRowBytes = 128;
constexpr int kTileRows = 128;
constexpr int kTiles = 2;
constexpr int kBoxBytes = kTileRows * kBoxRowBytes;       // 16 KiB, multiple of the 1 KiB swizzle period
constexpr int kScaleStageBytes = kStageChunks * 2 * 512;  // scale blocks of 512 bytes per 128 rows and 64 K
constexpr int kTileStageBytes = kBoxBytes + kScaleStageBytes;
constexpr int kWeightStages = 4;
constexpr int kXStages = 5;                   // activation chunks in flight
constexpr int kXStageBytes = 32 * kChunkK * 2;  // a chunk of 32 rows; 16 rows use half of it
constexpr int kABuffers = 3;
constexpr int kRowWarps = 8;                  // one thread per weight row of the two tiles
constexpr int kDequantSets = 2;               // set s dequantises the chunks with index = s (mod 2)
constexpr int kDequantWarps = kRowWarps * kDequantSets;
constexpr int kProducerWarp = kDequantWarps;
constexpr int kMmaWarp = kDequantWarps + 1;
constexpr int kMmaWarps = kTiles;
constexpr int kXWarp = kMmaWarp + kMmaWarps;
constexpr int kFirstEpilogueWarp = kXWarp + 1;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;
static_assert(kFirstEpilogueWarp % 4 == 0, "an epilogue warp reads the TMEM lanes 32 (warp % 4) ..");
constexpr int kTmemColumns = 512;
constexpr int kAccumulatorColumn = kABuffers * 64;
constexpr int kAccumulatorBuffers = 2;
constexpr int kTileColumns = kAccumulatorColumn + 32 * kAccumulatorBuffers;
static_assert(kTiles * kTileColumns <= kTmemColumns, "tensor memory budget");
static_assert(kTileStageBytes % 1024 == 0, "swizzled boxes start on 1 KiB boundaries");
constexpr int kStashPitch = 33;  // floats per column of a warp's stash: a lane reads a whole column without bank conflicts
constexpr int kStashWarpFloats = kTiles * 16 * kStashPitch + 64;  // a tile pair's accumulators, and 64 row scales
constexpr int kStashBytes = 8 * kStashWarpFloats * 4;
constexpr int kSmemBytes =
    kWeightStages * kTiles * kTileStageBytes + kXStages * kXStageBytes + kStashBytes + 1024;

// Workspace in global memory: partial tiles, then tickets, then the vocabulary head's candidates.
constexpr int kMaxCtas = 160;
constexpr int kPartialWarpFloats = kTiles * 16 * 32;  // one epilogue warp: 2 tiles x 16 columns x 32 lanes
constexpr int kPartialSlotFloats = kEpilogueWarps * kPartialWarpFloats;  // 32 KiB
constexpr size_t kPartialBytes = static_cast<size_t>(kMaxCtas) * 2 * kPartialSlotFloats * sizeof(float);
constexpr int kMaxPairTiles = 2048;
constexpr size_t kTicketBytes = static_cast<size_t>(kMaxPairTiles) * kEpilogueWarps * sizeof(int);
constexpr int kCandidateSlots = kMaxCtas * 4;         // per activation row: one per CTA and lane quarter
constexpr size_t kCandidateBytes = static_cast<size_t>(32) * kCandidateSlots * 8;
constexpr size_t kWorkspaceBytes = kPartialBytes + kTicketBytes + kCandidateBytes;

struct StreamKParams {
    const uint8_t* scales[2];
    const __half* x;          // staged activations: [K / 8][n_pad][8] f16
    __nv_bfloat16* y;         // bf16 rows [batch][N], or null
    __half* y_staged;         // the same values staged for the next projection: [N / 8][n_pad][8] f16, or null
    float* y_f32;             // vocabulary head: fp32 logits [batch][N], or null
    const float* row_scales;  // vocabulary head: one per weight row
    float inverse_scale[2];
    int out_features;
    int in_features;
    int batch;
    int pair_tiles;   // tile pairs: 256 rows (plain, head) or the gate and up rows of 128 outputs (SwiGLU)
    int stages_in_k;  // K / 256, or K / 128 for the head
    int units;        // pair_tiles * stages_in_k
    float* partials;
    int* tickets;
    // Regular K split: CTA = pair * splits + slice, no tickets.  With more than one slice every CTA
    // stores its fp32 partial rows [slice][batch][N] in split_out and the consumer sums them; with one
    // slice (a CTA per tile pair: matrices with about as many pairs as SMs) the CTA finishes its pair
    // itself.  0 splits: equal shares with tickets.
    int splits;
    float* split_out;
    // Latency mode (one activation row, weight rows split over ranks): the slices go to every rank's
    // exchange block as tagged words instead (exchange.cuh); split_out is null then.
    ExchangeTarget exchange;  // ranks == 0: not in latency mode
    uint32_t index_offset;  // vocabulary head in latency mode: this rank's first row in the whole vocabulary
    float* candidate_values;     // vocabulary head with sampling: [32][kCandidateSlots]
    uint32_t* candidate_indices;
    int* status;
    // The projection that this stream runs next, when the caller has named it: every CTA asks L2 for
    // the first stages of that launch's shares once its own last stage is on its way.
    struct Next {
        int valid;
        int swiglu;
        int nvfp4;  // block scales to fetch as well
        int out_features;
        int ctas;
        int units;
        int splits;  // 0: equal shares
        int stages_in_k;
        int group_blocks;
        const uint8_t* scales[2];
    } next;
};

// Optional timeline of every CTA of the last launch (compile with -DQWC_STREAMK_TRACE): nanosecond
// stamps of the global timer at the events named in trace_names(), read back with qwc_streamk_trace.
#ifdef QWC_STREAMK_TRACE
constexpr int kTraceSlots = 32;
__device__ unsigned long long g_trace[kMaxCtas * kTraceSlots];
__device__ __forceinline__ void trace_stamp(int slot) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now)::"memory");
    g_trace[blockIdx.x * kTraceSlots + slot] = now;
}
#define QWC_TRACE(slot) trace_stamp(slot)
#define QWC_TRACE_LANE0(slot) \
    do {                      \
        if (lane == 0) {      \
            trace_stamp(slot); \
        }                     \
    } while (0)
#else
#define QWC_TRACE(slot)
#define QWC_TRACE_LANE0(slot)
#endif

// Where the stores of the epilogue's rehearsal go (see the kernel): a line per lane of every epilogue
// warp, so that the rehearsals of different warps do not queue for the same line; nobody reads it.
__device__ float g_rehearsal_sink[kMaxCtas * kEpilogueWarps * 32];

struct Barriers {
    uint64_t w_full[kWeightStages];
    uint64_t w_empty[kWeightStages];
    uint64_t a_ready[kTiles][kABuffers];
    uint64_t a_free[kTiles][kABuffers];
    uint64_t x_full[kXStages];
    uint64_t x_free[kXStages];
    uint64_t d_ready[kAccumulatorBuffers];
    uint64_t d_free[kAccumulatorBuffers];
    uint64_t tmem_ready;
    uint32_t tmem_base;
    int failed;
};

// The polling loop is kept out of line so that the roles' main loops stay short for the instruction
// caches; a wait that is already satisfied costs one test.
__device__ __noinline__ bool sk_wait_slow(uint64_t* bar, uint32_t parity, Barriers* b, int* status) {
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

__device__ __forceinline__ bool sk_wait(uint64_t* bar, uint32_t parity, Barriers* b, int* status) {
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    return sk_wait_slow(bar, parity, b, status);
}

// One look at a barrier phase, without the hardware's own wait that try_wait includes.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// First unit of CTA `cta` when `units` units are shared by `ctas` CTAs.
__device__ __forceinline__ int share_begin(int units, int cta, int ctas) {
    return static_cast<int>(static_cast<long long>(units) * cta / ctas);
}

// The CTA whose share holds unit `unit` (ctas <= units, so no share is empty).
__device__ __forceinline__ int share_owner(int units, int unit, int ctas) {
    return static_cast<int>(((static_cast<long long>(unit) + 1) * ctas - 1) / units);
}

// A ticket is taken with release (the partial stored before it is visible to whoever sees the count)
// and acquire (the one who takes the last ticket sees every partial stored before the others).
__device__ __forceinline__ int ticket_take(int* ticket) {
    int taken;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(taken) : "l"(ticket) : "memory");
    return taken;
}

// A look that orders nothing (polled in a loop: an acquire per look would be a fence per look) ...
__device__ __forceinline__ int ticket_look(const int* ticket) {
    int count;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(count) : "l"(ticket) : "memory");
    return count;
}

// ... and the acquire that follows the look that found everybody in.
__device__ __forceinline__ void ticket_acquire() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

__device__ __forceinline__ bool better_candidate(float value, uint32_t index, float best, uint32_t best_index) {
    return value > best || (value == best && index < best_index);
}

// Where the partial of CTA `owner` for tile pair `pair` lies, for epilogue warp `e` (see the kernel:
// slot 0 when the owner's share starts with that piece, slot 1 when it ends with it).
__device__ __forceinline__ const float* piece_of(const float* partials, int units, int ctas, int S, int pair,
                                                 int owner, int e) {
    const int slot = share_begin(units, owner, ctas) >= pair * S ? 0 : 1;
    return partials + (static_cast<size_t>(owner * 2 + slot) * kEpilogueWarps + e) * kPartialWarpFloats;
}

// Sums `count` pieces of a tile pair into this warp's stash (shared memory), in the fixed order
// first + 1, first + 2, .., last, first (the first piece comes last because its owner is the one who
// usually finishes the sum, with that piece still on chip).  The piece of CTA `own` (-1: none) is
// taken from the stash itself, where it already lies, the others from the workspace; kPieces x kWidth
// loads are in flight at a time: the sum costs L2 round trips, not bandwidth.
template <int kCols, int kPieces, int kWidth>
__device__ __forceinline__ void sum_pieces_to_stash(const float* partials, int units, int ctas, int S, int pair,
                                                    int first_cta, int last_cta, int count, int own, int e,
                                                    int lane, float* stash) {
    const int pieces = last_cta - first_cta + 1;
#pragma unroll 1
    for (int base = 0; base < 2 * kCols; base += kWidth) {
        float total[kWidth];
#pragma unroll
        for (int i = 0; i < kWidth; ++i) {
            total[i] = 0.0f;
        }
#pragma unroll 1
        for (int q0 = 0; q0 < count; q0 += kPieces) {
            float piece[kPieces][kWidth];
#pragma unroll
            for (int j = 0; j < kPieces; ++j) {
                // a batch that reaches past the last piece reads the last piece again and adds nothing
                const int q = min(q0 + j, count - 1);
                const int owner = q < pieces - 1 ? first_cta + 1 + q : first_cta;
                const float* theirs = piece_of(partials, units, ctas, S, pair, owner, e) + lane;
#pragma unroll
                for (int i = 0; i < kWidth; ++i) {
                    const int flat = base + i;  // tile * kCols + column
                    piece[j][i] = owner == own ? stash[flat * kStashPitch + lane]
                                               : __ldcg(theirs + ((flat / kCols) * 16 + flat % kCols) * 32);
                }
            }
#pragma unroll
            for (int j = 0; j < kPieces; ++j) {
                const bool valid = q0 + j < count;
#pragma unroll
                for (int i = 0; i < kWidth; ++i) {
                    total[i] += valid ? piece[j][i] : 0.0f;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kWidth; ++i) {
            stash[(base + i) * kStashPitch + lane] = total[i];
        }
    }
}

template <bool kFp8, bool kSwiglu, int kPad, bool kSplitOut>
__global__ void __launch_bounds__(kThreads, 1)
    nvfp4_streamk_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                         const __grid_constant__ CUtensorMap next_map0, const __grid_constant__ CUtensorMap next_map1,
                         const StreamKParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ Barriers bars;
    // 128-byte-swizzled boxes need a 1 KiB-aligned shared address.
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        QWC_TRACE(0);  // entry
    }
    const int cta = blockIdx.x;
    const int ctas = gridDim.x;
    const int S = p.stages_in_k;
    constexpr int stage_chunks = kFp8 ? 1 : kStageChunks;  // 128 bytes per row and stage either way
    int u_begin, u_end;
    if (kSplitOut) {
        const int pair = cta / p.splits;
        const int slice = cta - pair * p.splits;
        u_begin = pair * S + S * slice / p.splits;
        u_end = pair * S + S * (slice + 1) / p.splits;
    } else {
        u_begin = share_begin(p.units, cta, ctas);
        u_end = share_begin(p.units, cta + 1, ctas);
    }
    const int num_units = u_end - u_begin;
    const int total_chunks = num_units * stage_chunks;
    const int pair_first = u_begin / S;
    const int stage_first = u_begin - pair_first * S;
    const int group_blocks = p.in_features / 64;
    constexpr int x_chunk_bytes = kPad * kChunkK * 2;

    unsigned char* weight_ring = smem;                                       // [stage][tile][box | scales]
    unsigned char* x_ring = smem + kWeightStages * kTiles * kTileStageBytes;  // [chunk][K core][row][8] f16
    float* stash_base = reinterpret_cast<float*>(x_ring + kXStages * kXStageBytes);  // [epilogue warp][4 KiB]

    // One stage of the weight ring: a box per tile and the tiles' block scales (issued by one thread).
    auto issue_stage = [&](int index, int pair, int stage) {
        const int slot = index % kWeightStages;
        int tile_row0[kTiles];
        int scale_tiles_present = 0;
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {
            tile_row0[t] = kSwiglu ? pair * kTileRows : (pair * kTiles + t) * kTileRows;
            // A box is always delivered whole (rows outside the matrix arrive as zeros) and the scale
            // storage is padded to whole 128-row blocks; a tile that starts past the matrix has no
            // scale block at all and keeps whatever the slot held (its rows are never stored).
            scale_tiles_present += (!kFp8 && tile_row0[t] < p.out_features) ? 1 : 0;
        }
        mbar_arrive_expect_tx(&bars.w_full[slot], kTiles * kBoxBytes + scale_tiles_present * kScaleStageBytes);
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {
            unsigned char* dst = weight_ring + (slot * kTiles + t) * kTileStageBytes;
            tma_box_g2s(dst, t == 1 ? &map1 : &map0, stage * kBoxRowBytes, tile_row0[t], &bars.w_full[slot]);
            if (!kFp8 && tile_row0[t] < p.out_features) {
                bulk_g2s(dst + kBoxBytes,
                         p.scales[t] + (static_cast<size_t>(tile_row0[t] >> 7) * group_blocks + 4 * stage) * 512,
                         kScaleStageBytes, &bars.w_full[slot]);
            }
        }
    };
    // The first trip round the weight ring does not wait for the rest of the CTA: the producer's
    // thread sets up the ring's own barriers and asks for the first stages before the CTA-wide barrier
    // (weights are never written during a step, so nothing has to be waited for either).
    const int early_stages = num_units < kWeightStages ? num_units : kWeightStages;
    if (threadIdx.x == kProducerWarp * 32) {
        for (int s = 0; s < kWeightStages; ++s) {
            mbar_init(&bars.w_full[s], 1);
            mbar_init(&bars.w_empty[s], kFp8 ? kRowWarps : kDequantWarps);  // warps that read a stage
        }
        mbar_fence_init();
        int pair = pair_first, stage = stage_first;
        for (int index = 0; index < early_stages; ++index) {
            issue_stage(index, pair, stage);
            if (++stage == S) {
                stage = 0;
                ++pair;
            }
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
            mbar_init(&bars.x_full[s], 1);
            mbar_init(&bars.x_free[s], kMmaWarps);
        }
        for (int b = 0; b < kAccumulatorBuffers; ++b) {
            mbar_init(&bars.d_ready[b], kMmaWarps);
            mbar_init(&bars.d_free[b], kEpilogueWarps);
        }
        mbar_init(&bars.tmem_ready, 1);
        bars.failed = status_is_set(p.status) ? 1 : 0;
        bars.tmem_base = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        QWC_TRACE(1);  // barriers set up
    }
    // Tensor memory is allocated while the producer already fetches weights; the warps that use it
    // wait for the address below.
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
    if (warp != kProducerWarp && warp != kXWarp) {
        tmem_ok = sk_wait(&bars.tmem_ready, 0, &bars, p.status);
        tmem_ok = __all_sync(0xffffffffu, tmem_ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars.tmem_base);
    }

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
        for (int c = set; c < total_chunks && ok; c += kDequantSets) {
            const int wstage = kFp8 ? c : c / kStageChunks;
            const int slot = wstage % kWeightStages;
            ok = sk_wait(&bars.w_full[slot], (wstage / kWeightStages) & 1, &bars, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            if (warp == 0 && c == 0) {
                QWC_TRACE_LANE0(2);  // first weights landed
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
                ok = sk_wait(&bars.a_free[tile][buf], ((c / kABuffers) & 1) ^ 1, &bars, p.status);
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
                const int q = set;  // which half of the stage's 128 bytes per row
                const unsigned char* scale_tiles = stage + kBoxBytes + q * 1024 + scale_offset;
                uint4 raw[4];
#pragma unroll
                for (int part = 0; part < 4; ++part) {
                    raw[part] = *reinterpret_cast<const uint4*>(row + (((q * 4 + part) ^ row_swizzle) << 4));
                }
                // 8 block scales of this chunk: two words of four e4m3 (cuda/nvfp4.cu:33-39 layout)
                const uint32_t scale_word0 = *reinterpret_cast<const uint32_t*>(scale_tiles);
                const uint32_t scale_word1 = *reinterpret_cast<const uint32_t*>(scale_tiles + 512);
                ok = sk_wait(&bars.a_free[tile][buf], ((c / kABuffers) & 1) ^ 1, &bars, p.status);
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
            // hand the chunk to the tensor-core warp and the ring slot back to the producer
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars.a_ready[tile][buf]);
                mbar_arrive(&bars.w_empty[slot]);  // this warp reads one chunk per stage
            }
        }
        if (warp == 0) {
            QWC_TRACE_LANE0(6);  // last chunk dequantised
        }
    } else if (warp == kProducerWarp) {
        // ---------------- producer: weights and scales ----------------
        bool ok = true;
        int pair = pair_first, stage = stage_first + early_stages;
        while (stage >= S) {
            stage -= S;
            ++pair;
        }
        for (int index = early_stages; index < num_units && ok; ++index) {
            const int slot = index % kWeightStages;
            ok = sk_wait(&bars.w_empty[slot], ((index / kWeightStages) & 1) ^ 1, &bars, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            if (elect_one()) {
                issue_stage(index, pair, stage);
            }
            __syncwarp();
            if (++stage == S) {
                stage = 0;
                ++pair;
            }
        }
        QWC_TRACE_LANE0(7);  // last stage requested
        if (ok && p.next.valid && elect_one()) {
            // the first stages of the shares of the launch that follows, dealt over this launch's CTAs
            for (int other = cta; other < p.next.ctas; other += ctas) {
                int first, end;
                if (p.next.splits > 0) {
                    const int its_pair = other / p.next.splits;
                    const int its_slice = other - its_pair * p.next.splits;
                    first = its_pair * p.next.stages_in_k + p.next.stages_in_k * its_slice / p.next.splits;
                    end = its_pair * p.next.stages_in_k + p.next.stages_in_k * (its_slice + 1) / p.next.splits;
                } else {
                    first = share_begin(p.next.units, other, p.next.ctas);
                    end = share_begin(p.next.units, other + 1, p.next.ctas);
                }
                const int count = min(kWeightStages, end - first);
                int next_pair = first / p.next.stages_in_k;
                int next_stage = first - next_pair * p.next.stages_in_k;
                for (int i = 0; i < count; ++i) {
#pragma unroll
                    for (int t = 0; t < kTiles; ++t) {
                        const int row0 = p.next.swiglu ? next_pair * kTileRows : (next_pair * kTiles + t) * kTileRows;
                        if (row0 < p.next.out_features) {
                            tma_box_prefetch_l2(t == 1 ? &next_map1 : &next_map0, next_stage * kBoxRowBytes, row0);
                            if (p.next.nvfp4) {
                                bulk_prefetch_l2(p.next.scales[t] + (static_cast<size_t>(row0 >> 7) * p.next.group_blocks +
                                                                     4 * next_stage) * 512,
                                                 kScaleStageBytes);
                            }
                        }
                    }
                    if (++next_stage == p.next.stages_in_k) {
                        next_stage = 0;
                        ++next_pair;
                    }
                }
            }
        }
    } else if (warp < kXWarp) {
        // ---------------- tensor-core issue ----------------
        // One warp per tile.  The whole warp waits; only the instructions themselves sit in the
        // elected lane's region, which the compiler then runs on the uniform datapath.
        const int t = warp - kMmaWarp;
        const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(kPad >> 3) << 17) | (8u << 24);
        // K cores are kPad * 16 bytes apart, 8-row groups 128 bytes; one instruction takes two K cores
        const uint64_t desc_base = smem_descriptor(smem_u32(x_ring), kPad * 16, 128);
        const uint64_t desc_step = static_cast<uint64_t>((2 * kPad * 16) >> 4);
        const uint64_t desc_stage = static_cast<uint64_t>(kXStageBytes >> 4);
        const uint32_t a_tile = tmem_base + t * kTileColumns;
        const uint32_t d_tile = a_tile + kAccumulatorColumn;
        bool ok = tmem_ok;
        int buf = 0, xs = 0;
        uint32_t a_parity = 0, x_parity = 0;
        int stage = stage_first;
        int segment = 0;
        for (int c = 0; c < total_chunks && ok; ++c) {
            const int in_stage = kFp8 ? 0 : (c & 1);
            const bool fresh = c == 0 || (stage == 0 && in_stage == 0);  // first chunk of a segment
            const bool last = c == total_chunks - 1 || (stage == S - 1 && in_stage == stage_chunks - 1);
            const int acc = segment & 1;
            if (fresh && segment >= kAccumulatorBuffers) {
                // the epilogue must have read what this accumulator held two segments ago
                ok = sk_wait(&bars.d_free[acc], ((segment >> 1) & 1) ^ 1, &bars, p.status);
            }
            if (ok) {
                ok = sk_wait(&bars.x_full[xs], x_parity, &bars, p.status);
            }
            if (t == 0 && c == 0) {
                QWC_TRACE_LANE0(3);  // first activations landed
            }
            if (ok) {
                ok = sk_wait(&bars.a_ready[t][buf], a_parity, &bars, p.status);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            if (t == 0 && c == 0) {
                QWC_TRACE_LANE0(4);  // first MMA
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (elect_one()) {
                uint64_t b_desc = desc_base + desc_stage * xs;
                const uint32_t a0 = a_tile + buf * 64;
                const uint32_t d0 = d_tile + acc * 32;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    umma_f16(d0, a0 + s * 8, b_desc, idesc, (s > 0 || !fresh) ? 1u : 0u);
                    b_desc += desc_step;
                }
                umma_commit(&bars.a_free[t][buf]);
                umma_commit(&bars.x_free[xs]);
                if (last) {
                    umma_commit(&bars.d_ready[acc]);
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
            if (in_stage == stage_chunks - 1 && ++stage == S) {
                stage = 0;
            }
            segment += last ? 1 : 0;
        }
        if (t == 0) {
            QWC_TRACE_LANE0(5);  // last MMA issued
        }
    } else if (warp == kXWarp) {
        // ---------------- activation chunks ----------------
        // Everything above starts before the kernel that produces the activations has finished; these
        // loads (and the epilogue's stores) wait for it.
        pdl_wait();
        QWC_TRACE_LANE0(22);  // the previous kernel has finished
        bool ok = true;
        int stage = stage_first;
        for (int c = 0; c < total_chunks && ok; ++c) {
            const int xs = c % kXStages;
            const int in_stage = kFp8 ? 0 : (c & 1);
            if (c >= kXStages) {
                ok = sk_wait(&bars.x_free[xs], ((c / kXStages) & 1) ^ 1, &bars, p.status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    break;
                }
            }
            if (elect_one()) {
                const int k_chunk = stage * stage_chunks + in_stage;
                mbar_arrive_expect_tx(&bars.x_full[xs], x_chunk_bytes);
                bulk_g2s(x_ring + xs * kXStageBytes,
                         reinterpret_cast<const unsigned char*>(p.x) + static_cast<size_t>(k_chunk) * x_chunk_bytes,
                         x_chunk_bytes, &bars.x_full[xs]);
            }
            __syncwarp();
            if (in_stage == stage_chunks - 1 && ++stage == S) {
                stage = 0;
            }
        }
    } else {
        // ---------------- epilogue ----------------
        // Warp e: output rows 32 (e % 4) .. + 31 of both tiles, activation rows (e / 4) * kPad / 2 .. .
        // Everything goes through the warp's 4 KiB stash in shared memory ([tile * kCols + column][lane]),
        // eight columns at a time, so that no step holds more than a few registers.
        constexpr int kCols = kPad / 2;  // accumulator columns per tile and warp
        const int e = warp - kFirstEpilogueWarp;
        const int quarter = e & 3;
        const int first_token = (e >> 2) * kCols;
        const uint32_t lane_address = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kAccumulatorColumn +
                                      (e >> 2) * kCols;
        float best_value = -INFINITY;      // lane i: best logit of activation row first_token + i
        uint32_t best_index = UINT32_MAX;
        const bool sampling = kFp8 && p.candidate_values != nullptr;
        float* stash = stash_base + e * kStashWarpFloats + lane;
        bool ok = tmem_ok;

        // Scales the finished tile pair in the stash, combines (SwiGLU), rounds and stores the activation
        // rows below `batch`.  batch == 0 is the rehearsal (below): every instruction runs, for every
        // row, but the stores go to a sink and nothing is sampled.
        auto finalize = [&](int pair, int batch) {
            const bool rehearsal = batch == 0;
            const int rows_stored = rehearsal ? kPad : batch;
            float* const sink = g_rehearsal_sink + (cta * kEpilogueWarps + e) * 32;
            __nv_bfloat16* const y = rehearsal ? reinterpret_cast<__nv_bfloat16*>(sink) : p.y;
            __half* const y_staged = rehearsal ? reinterpret_cast<__half*>(sink) : p.y_staged;
            float* const y_f32 = rehearsal ? sink : p.y_f32;
            const size_t row_pitch = rehearsal ? 0 : static_cast<size_t>(p.out_features);
            const size_t staged_pitch = rehearsal ? 0 : static_cast<size_t>(kPad) * 8;
#pragma unroll 1
            for (int c0 = 0; c0 < kCols; c0 += 8) {
                float v0[8], v1[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v0[i] = stash[(c0 + i) * kStashPitch];
                    v1[i] = stash[(kCols + c0 + i) * kStashPitch];
                }
                if (kSwiglu) {
                    const int row = pair * kTileRows + quarter * 32 + lane;
                    if (row < p.out_features) {
                        const size_t column = rehearsal ? lane : row;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int token = first_token + c0 + i;
                            if (token < rows_stored) {
                                const float gate = v0[i] * p.inverse_scale[0];
                                const float up = v1[i] * p.inverse_scale[1];
                                // (the fast division: an IEEE one leaves the fast path for every gate below
                                // -88, where the exponential is infinite, and costs microseconds at the very
                                // end of the launch; the two differ by two units in the last place of fp32)
                                const __nv_bfloat16 rounded =
                                    __float2bfloat16(__fdividef(gate, 1.0f + __expf(-gate)) * up);
                                if (p.y != nullptr) {
                                    y[token * row_pitch + column] = rounded;
                                }
                                if (p.y_staged != nullptr) {
                                    y_staged[(column >> 3) * staged_pitch + token * 8 + (column & 7)] =
                                        __float2half_rn(fminf(fmaxf(__bfloat162float(rounded), -65504.0f), 65504.0f));
                                }
                            }
                        }
                    }
                    continue;
                }
#pragma unroll
                for (int t = 0; t < kTiles; ++t) {
                    const int row = (pair * kTiles + t) * kTileRows + quarter * 32 + lane;
                    const bool inside = row < p.out_features;
                    const size_t column = rehearsal ? lane : row;
                    const float row_scale = kFp8 ? (inside ? p.row_scales[row] : 0.0f) : p.inverse_scale[0];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int token = first_token + c0 + i;
                        const float value = (t == 0 ? v0[i] : v1[i]) * row_scale;
                        if (kFp8) {
                            if (inside && token < rows_stored && p.y_f32 != nullptr) {
                                y_f32[token * row_pitch + column] = value;
                            }
                        } else if (inside && token < rows_stored) {
                            const __nv_bfloat16 rounded = __float2bfloat16(value);
                            if (p.y != nullptr) {
                                y[token * row_pitch + column] = rounded;
                            }
                            if (p.y_staged != nullptr) {
                                y_staged[(column >> 3) * staged_pitch + token * 8 + (column & 7)] =
                                    __float2half_rn(fminf(fmaxf(__bfloat162float(rounded), -65504.0f), 65504.0f));
                            }
                        }
                    }
                }
            }
        };
        // Greedy sampling without logits: the best (logit, row) of the tile pair in the stash for every
        // activation row this warp holds.  A lane takes one column of the stash (lanes below kCols: tile 0,
        // the next kCols lanes: tile 1) and walks down its 32 rows - no exchange between lanes but the
        // row scales, which every lane fetches for its own row and leaves in shared memory.
        auto sample_pair = [&](int pair, bool rehearsal) {
            float* scales = stash - lane + kTiles * 16 * kStashPitch;  // [tile][row of this quarter]
#pragma unroll
            for (int t = 0; t < kTiles; ++t) {
                const int row = (pair * kTiles + t) * kTileRows + quarter * 32 + lane;
                // a row past the vocabulary can never win: its logit is -inf whatever the accumulator holds
                scales[t * 32 + lane] = row < p.out_features ? p.row_scales[row] : NAN;
            }
            __syncwarp();
            const int t = lane / kCols;
            float candidate = -INFINITY;
            uint32_t index = UINT32_MAX;
            if (t < kTiles) {
                const float* column = stash - lane + lane * kStashPitch;  // (t * kCols + lane % kCols) == lane
                const uint32_t row0 = static_cast<uint32_t>((pair * kTiles + t) * kTileRows + quarter * 32);
#pragma unroll 8
                for (int r = 0; r < 32; ++r) {
                    const float scale = scales[t * 32 + r];
                    const float value = scale == scale ? column[r] * scale : -INFINITY;
                    if (value > candidate) {  // rows ascend: a later equal value never replaces an earlier one
                        candidate = value;
                        index = row0 + r;
                    }
                }
            }
            // the two tiles' winners of a column meet in the lane that keeps the column's running best
            const float other = __shfl_down_sync(0xffffffffu, candidate, kCols);
            const uint32_t other_index = __shfl_down_sync(0xffffffffu, index, kCols);
            if (better_candidate(other, other_index, candidate, index)) {
                candidate = other;
                index = other_index;
            }
            if (!rehearsal && lane < kCols && better_candidate(candidate, index, best_value, best_index)) {
                best_value = candidate;
                best_index = index;
            }
            __syncwarp();
        };
        // A slice of a regular K split: fp32 rows [slice][batch][N] for the consumer to sum, this lane's two
        // rows (batch == 0: the rehearsal, as above).
        auto store_slice = [&](int pair, int batch) {
            const bool rehearsal = batch == 0;
            const int slice = kSplitOut ? cta - pair * p.splits : 0;
            if (p.exchange.ranks > 0) {
                // Latency mode, one activation row (the first column of the warps that hold the first
                // rows): this rank's columns of the row go to every rank's copy of the slice array, its
                // own included, as tagged words (exchange.cuh).
                if (first_token != 0) {
                    return;
                }
                const uint32_t tag = rehearsal ? 0u : exchange_tag(p.exchange.epoch, p.exchange.instance);
                uint2* const sink = reinterpret_cast<uint2*>(g_rehearsal_sink + (cta * kEpilogueWarps + e) * 32);
#pragma unroll
                for (int t = 0; t < kTiles; ++t) {
                    const int row = kSwiglu ? pair * kTileRows + quarter * 32 + lane
                                            : (pair * kTiles + t) * kTileRows + quarter * 32 + lane;
                    if (row < p.out_features) {
                        // SwiGLU pair: the row is [gate | up], each half holding all ranks' columns
                        const size_t element = static_cast<size_t>(slice) * p.exchange.width +
                                               (kSwiglu ? t * (p.exchange.width / 2) : 0) + p.exchange.first_column +
                                               row;
                        const float value = stash[(t * kCols) * kStashPitch];
                        for (int r = 0; r < p.exchange.ranks; ++r) {
                            store_tagged(rehearsal ? sink + (lane >> 1) : p.exchange.copies[r] + element, value, tag);
                        }
                    }
                }
                return;
            }
            const int rows_stored = rehearsal ? kPad : batch;
            float* const out = rehearsal ? g_rehearsal_sink + (cta * kEpilogueWarps + e) * 32
                                         : p.split_out + static_cast<size_t>(slice) * p.batch * p.out_features;
            const size_t row_pitch = rehearsal ? 0 : static_cast<size_t>(p.out_features);
#pragma unroll
            for (int t = 0; t < kTiles; ++t) {
                const int row = (pair * kTiles + t) * kTileRows + quarter * 32 + lane;
                if (row < p.out_features) {
                    const size_t column = rehearsal ? lane : row;
#pragma unroll
                    for (int i = 0; i < kCols; ++i) {
                        const int token = first_token + i;
                        if (token < rows_stored) {
                            out[token * row_pitch + column] = stash[(t * kCols + i) * kStashPitch];
                        }
                    }
                }
            }
        };
        // Rehearsal.  What this warp runs at the very end of the launch - after the last MMA, with every
        // SM waiting for it - it has not run before, so its instructions would come from L2 one cache
        // line at a time.  It has nothing to do until the first accumulators are complete: it walks
        // through the same code once now, its stores aimed at a sink, and finds it in the instruction cache
        // later (measured on the K-split in-projection: accumulators read -> slice stored 1.6 -> 0.6 us).
        // (It is the first pass of the segment loop below, so that it is the same code, not a copy.)
        // `count` pieces in the fixed order; `own`: this CTA when its piece lies in the stash, else -1
        const auto sum_to_stash = [&](int pair, int first_cta, int last_cta, int count, int own) {
            if (count <= 2) {
                sum_pieces_to_stash<kCols, 2, kCols>(p.partials, p.units, ctas, S, pair, first_cta, last_cta, count, own,
                                                     e, lane, stash - lane);
            } else {
                sum_pieces_to_stash<kCols, 4, 8>(p.partials, p.units, ctas, S, pair, first_cta, last_cta, count, own, e,
                                                 lane, stash - lane);
            }
        };
        int u = u_begin;
        int segment = -1;  // -1: the rehearsal
        while (segment < 0 || (u < u_end && ok)) {
            const bool rehearsal = segment < 0;
            const int pair = u / S;
            const int s0 = u - pair * S;
            const int s1 = min(S, s0 + (u_end - u));
            const int acc = segment & 1;
            const bool whole = !kSplitOut && s0 == 0 && s1 == S;
            const bool ticketed = !kSplitOut && !whole;
            const int first_cta = ticketed ? share_owner(p.units, pair * S, ctas) : cta;
            const int last_cta = ticketed ? share_owner(p.units, pair * S + S - 1, ctas) : cta;
            int* ticket = p.tickets + pair * kEpilogueWarps + e;
            int limit = p.batch;       // activation rows that are stored
            bool complete = false;     // the pair is finished here: scale, combine, store
            bool slice = false;        // the segment is a slice for the consumer to sum
            bool parked = false;
            if (rehearsal) {
                limit = 0;  // the stores go to a sink
                asm volatile("" : "+r"(limit));  // opaque: one copy of the code below serves both passes
                slice = kSplitOut && (p.split_out != nullptr || p.exchange.ranks > 0);
                complete = !slice;
            } else {
                // The first piece of a pair is what its CTA ends its share with, so it usually arrives
                // last: its owner looks at the ticket while it waits for its own accumulators (the epilogue
                // warps have nothing else to do), and once all the others are in, it parks their sum in
                // the stash.  The end of the launch is then one TMEM read, one addition and the stores.
                const bool may_look = ticketed && s0 == 0 && u + (s1 - s0) == u_end;
                if (may_look) {
                    const long long start = clock64();
                    while (!mbar_test(&bars.d_ready[acc], (segment >> 1) & 1)) {
                        int count = 0;
                        if (lane == 0) {
                            count = ticket_look(ticket);  // an L2 round trip
                        }
                        count = __shfl_sync(0xffffffffu, count, 0);
                        if (count == last_cta - first_cta) {
                            ticket_acquire();
                            __syncwarp();
                            sum_to_stash(pair, first_cta, last_cta, count, -1);
                            parked = true;
                            break;
                        }
                        if (clock64() - start > 40000000ll || *reinterpret_cast<volatile int*>(&bars.failed) != 0) {
                            break;  // the bounded wait below gives the verdict
                        }
                        __nanosleep(400);  // the look is not urgent and must not crowd the memory pipeline
                    }
                }
                ok = sk_wait(&bars.d_ready[acc], (segment >> 1) & 1, &bars, p.status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    break;
                }
                if (e == 0) {
                    QWC_TRACE_LANE0(8 + 3 * min(segment, 3));  // accumulators of the segment complete
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // tensor memory -> stash (added to the parked sum of the other pieces when there is one)
#pragma unroll
                for (int t = 0; t < kTiles; ++t) {
#pragma unroll
                    for (int c0 = 0; c0 < kCols; c0 += 8) {
                        uint32_t r[8];
                        tmem_load8_issue(lane_address + t * kTileColumns + acc * 32 + c0, r);
                        tmem_load_wait();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float* slot = stash + (t * kCols + c0 + i) * kStashPitch;
                            *slot = parked ? *slot + __uint_as_float(r[i]) : __uint_as_float(r[i]);
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars.d_free[acc]);
                }
                if (e == 0) {
                    QWC_TRACE_LANE0(9 + 3 * min(segment, 3));  // accumulators read
                }
                complete = whole || parked;
                if (kSplitOut) {
                    slice = p.split_out != nullptr || p.exchange.ranks > 0;
                    complete = !slice;  // one CTA per tile pair: nothing to sum
                } else if (parked) {
                    if (lane == 0) {
                        *ticket = 0;  // everybody else arrived long ago: the tickets go back
                    }
                } else if (!whole) {
                    // A piece of the pair's K range: the partial goes to this CTA's slot (0: the share
                    // starts with it, 1: the share ends with it), then a ticket.  Tickets are per (pair,
                    // epilogue warp): a warp never has to wait for the other warps of its CTA.
                    const int slot = u == u_begin ? 0 : 1;
                    float* mine =
                        p.partials + (static_cast<size_t>(cta * 2 + slot) * kEpilogueWarps + e) * kPartialWarpFloats + lane;
#pragma unroll
                    for (int i = 0; i < kCols; ++i) {
                        mine[i * 32] = stash[i * kStashPitch];
                        mine[(16 + i) * 32] = stash[(kCols + i) * kStashPitch];
                    }
                    __syncwarp();  // every lane's stores are ordered before the ticket that lane 0 takes
                    int taken = 0;
                    if (lane == 0) {
                        taken = ticket_take(ticket);
                    }
                    taken = __shfl_sync(0xffffffffu, taken, 0);
                    if (taken == last_cta - first_cta) {
                        // the last piece to arrive sums all of them, in the fixed order
                        if (lane == 0) {
                            *ticket = 0;  // ready for the next launch
                        }
                        sum_to_stash(pair, first_cta, last_cta, last_cta - first_cta + 1, cta);
                        complete = true;
                    }
                }
            }
            if (slice) {
                store_slice(pair, limit);
            }
            if (complete) {
                __syncwarp();
                if (sampling) {
                    sample_pair(pair, rehearsal);
                }
                if (!sampling || p.y_f32 != nullptr) {
                    finalize(pair, limit);
                }
            }
            if (rehearsal) {
                pdl_wait();  // from here on the warp touches what earlier kernels wrote and read
                if (e == 0) {
                    QWC_TRACE_LANE0(23);
                }
                segment = 0;
                continue;
            }
            if (e == 0) {
                QWC_TRACE_LANE0(10 + 3 * min(segment, 3));  // segment stored (partial or final); the fourth slot: the last
#ifdef QWC_STREAMK_TRACE
                if (lane == 0) {
                    g_trace[blockIdx.x * kTraceSlots + 24 + min(segment, 3)] =
                        (whole ? 1 : 0) | (parked ? 2 : 0) | (complete ? 4 : 0) | ((last_cta - first_cta + 1) << 8) |
                        (static_cast<unsigned long long>(s1 - s0) << 16);
                }
#endif
            }
            u += s1 - s0;
            ++segment;
        }
        if (sampling && ok && p.exchange.ranks > 0) {
            // latency mode: the one row's candidate of this warp goes to every rank, as two tagged words
            // (value, then the row's number in the whole vocabulary)
            if (first_token == 0 && lane == 0) {
                const uint32_t tag = exchange_tag(p.exchange.epoch, p.exchange.instance);
                const size_t element = static_cast<size_t>(p.exchange.first_column + cta * 4 + quarter) * 2;
                const uint32_t index = best_index == UINT32_MAX ? UINT32_MAX : best_index + p.index_offset;
                for (int r = 0; r < p.exchange.ranks; ++r) {
                    store_tagged(p.exchange.copies[r] + element, best_value, tag);
                    store_tagged(p.exchange.copies[r] + element + 1, __uint_as_float(index), tag);
                }
            }
        } else if (sampling && ok && lane < kCols && first_token + lane < 32) {
            const size_t slot = static_cast<size_t>(first_token + lane) * kCandidateSlots + cta * 4 + quarter;
            p.candidate_values[slot] = best_value;
            p.candidate_indices[slot] = best_index;
        }
    }

    // A CTA that gave up must not return while the stages it asked for before the barrier are still
    // landing in its shared memory: their thread waits for them, with a limit of 0.2 ms per ring slot
    // (a stage that was consumed has completed its first phase long ago and the wait falls through).
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
        QWC_TRACE(21);  // every role done
    }
    const bool failed = *reinterpret_cast<volatile int*>(&bars.failed) != 0;
    if (failed && threadIdx.x == kProducerWarp * 32) {
        for (int slot = 0; slot < early_stages; ++slot) {
            const long long start = clock64();
            while (!mbar_try_wait(&bars.w_full[slot], 0) && clock64() - start < 400000ll) {
            }
        }
    }
    if (failed && threadIdx.x == kXWarp * 32) {
        for (int slot = 0; slot < kXStages; ++slot) {
            const long long start = clock64();
            while (!mbar_try_wait(&bars.x_full[slot], 0) && clock64() - start < 400000ll) {
            }
        }
    }
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
    }
}

// Greedy sampling from the candidates the vocabulary head left: one CTA per activation row, ties to
// the smaller index (cuda/sampling.cu:11-14).  Also stores the device status word next to the tokens.
constexpr int kSampleThreads = 128;

__global__ void __launch_bounds__(kSampleThreads) sample_candidates_kernel(const float* __restrict__ values,
                                                                           const uint32_t* __restrict__ indices,
                                                                           uint32_t* __restrict__ output, int slots,
                                                                           const int* __restrict__ status,
                                                                           uint32_t* __restrict__ status_out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float shared_values[kSampleThreads / 32];
    __shared__ uint32_t shared_indices[kSampleThreads / 32];
    const int row = blockIdx.x;
    float best = -INFINITY;
    uint32_t best_index = UINT32_MAX;
    for (int i = threadIdx.x; i < slots; i += kSampleThreads) {
        const float value = values[static_cast<size_t>(row) * kCandidateSlots + i];
        const uint32_t index = indices[static_cast<size_t>(row) * kCandidateSlots + i];
        if (better_candidate(value, index, best, best_index)) {
            best = value;
            best_index = index;
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const uint32_t other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
        if (better_candidate(other, other_index, best, best_index)) {
            best = other;
            best_index = other_index;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        shared_values[threadIdx.x >> 5] = best;
        shared_indices[threadIdx.x >> 5] = best_index;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kSampleThreads / 32; ++w) {
            if (better_candidate(shared_values[w], shared_indices[w], best, best_index)) {
                best = shared_values[w];
                best_index = shared_indices[w];
            }
        }
        output[row] = best_index;
        if (row == 0 && status_out != nullptr) {
            *status_out = static_cast<uint32_t>(*reinterpret_cast<const volatile int*>(status));
        }
    }
}

// Latency mode: the same choice over the candidates that all ranks stored into this rank's block (two
// tagged words each: value, vocabulary row), after a bounded wait for this step's words.  Every rank
// sees the same candidates in the same places and stores the same token.
__global__ void __launch_bounds__(kSampleThreads) sample_exchanged_kernel(const TaggedRow candidates, int slots,
                                                                          uint32_t* __restrict__ output,
                                                                          uint32_t* __restrict__ status_out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float shared_values[kSampleThreads / 32];
    __shared__ uint32_t shared_indices[kSampleThreads / 32];
    const uint32_t tag = exchange_tag(candidates.epoch, candidates.instance);
    float best = -INFINITY;
    uint32_t best_index = UINT32_MAX;
    for (int i = threadIdx.x; i < slots; i += kSampleThreads) {
        const uint2* at = candidates.words + 2 * i;
        const uint4 pair = load_tagged_pair(at);
        const float value = ((pair.y ^ tag) & candidates.tag_mask) == 0
                                ? __uint_as_float(pair.x)
                                : await_tagged(at, tag, candidates.status, candidates.wait_profile);
        const uint32_t index =
            ((pair.w ^ tag) & candidates.tag_mask) == 0
                ? pair.z
                : __float_as_uint(await_tagged(at + 1, tag, candidates.status, candidates.wait_profile));
        if (better_candidate(value, index, best, best_index)) {
            best = value;
            best_index = index;
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const uint32_t other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
        if (better_candidate(other, other_index, best, best_index)) {
            best = other;
            best_index = other_index;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        shared_values[threadIdx.x >> 5] = best;
        shared_indices[threadIdx.x >> 5] = best_index;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kSampleThreads / 32; ++w) {
            if (better_candidate(shared_values[w], shared_indices[w], best, best_index)) {
                best = shared_values[w];
                best_index = shared_indices[w];
            }
        }
        output[0] = best_index;
        if (status_out != nullptr) {
            *status_out = static_cast<uint32_t>(*reinterpret_cast<const volatile int*>(candidates.status));
        }
    }
}

// bf16 rows -> the staged f16 operand layout [K / 8][n_pad][8]; one thread per 8 elements.
__global__ void __launch_bounds__(256) stage_activations_kernel(const __nv_bfloat16* __restrict__ x,
                                                                __half* __restrict__ staged, int batch, int in_features,
                                                                int n_pad) {
    pdl_launch_dependents();
    pdl_wait();
    const int cores = in_features / 8;
    const int index = blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= cores * batch) {
        return;
    }
    const int token = index / cores;
    const int core = index - token * cores;
    const uint4 raw = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(token) * in_features + core * 8);
    *reinterpret_cast<uint4*>(staged + (static_cast<size_t>(core) * n_pad + token) * 8) =
        make_uint4(bf16x2_to_f16x2(raw.x), bf16x2_to_f16x2(raw.y), bf16x2_to_f16x2(raw.z), bf16x2_to_f16x2(raw.w));
}

int sm_count_streamk() {
    static PerDevice<int> count_per_device;
    const int* found = count_per_device.get([]() {
        int device = 0, value = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || value <= 0) {
            value = 148;
        }
        return value;
    });
    return found == nullptr ? 148 : *found;
}

struct LaunchShape {
    int pair_tiles;
    int stages_in_k;
    int units;
    int ctas;
    int splits;  // of the regular K split whose sum is left to the consumer; 0: equal shares with tickets
};

// Tile pairs that nearly fill the SMs once are not cut at all: one CTA per pair.
bool prefers_whole_pairs(int pair_tiles, int ctas) { return pair_tiles <= ctas && pair_tiles * 20 >= ctas * 17; }

// What a consumer can have in flight per output at once: more slices would cost it a second round trip.
constexpr int kMaxKSlices = 8;
static_assert(kMaxKSlices == kExchangeMaxSlices, "exchange rows are sized for this many slices");

LaunchShape shape_of(int out_features, int in_features, bool swiglu, bool fp8, bool split_out = false) {
    LaunchShape shape;
    const int rows_per_pair = swiglu ? kTileRows : kTiles * kTileRows;
    shape.pair_tiles = (out_features + rows_per_pair - 1) / rows_per_pair;
    shape.stages_in_k = in_features / (fp8 ? kChunkK : kChunkK * kStageChunks);
    shape.units = shape.pair_tiles * shape.stages_in_k;
    shape.splits = 0;
    const int sms = sm_count_streamk();
    shape.ctas = sms < kMaxCtas ? sms : kMaxCtas;
    if (!split_out && !fp8 && prefers_whole_pairs(shape.pair_tiles, shape.ctas)) {
        shape.splits = 1;
        shape.ctas = shape.pair_tiles;
        return shape;
    }
    if (split_out) {
        // as many K slices per tile pair as fill the SMs once; a slice holds at least one stage
        int splits = shape.ctas / shape.pair_tiles;
        splits = splits < 1 ? 1 : splits;
        splits = splits > shape.stages_in_k ? shape.stages_in_k : splits;
        splits = splits > kMaxKSlices ? kMaxKSlices : splits;

        shape.splits = splits;
        shape.ctas = shape.pair_tiles * splits;
        return shape;
    }
    if (shape.ctas > shape.units) {
        shape.ctas = shape.units;
    }
    return shape;
}

cudaError_t launch_streamk(StreamKParams p, const void* packed0, const void* packed1, bool swiglu, bool fp8,
                           void* workspace, cudaStream_t stream) {
    const bool split_out = p.split_out != nullptr || (p.exchange.ranks > 0 && !fp8);
    const LaunchShape shape = shape_of(p.out_features, p.in_features, swiglu, fp8, split_out);
    if (shape.pair_tiles > kMaxPairTiles || shape.units <= 0 || shape.ctas > 4 * kMaxCtas) {
        (void)take_next_projection();
        return cudaErrorInvalidValue;
    }
    p.pair_tiles = shape.pair_tiles;
    p.stages_in_k = shape.stages_in_k;
    p.units = shape.units;
    p.splits = shape.splits;
    unsigned char* base = static_cast<unsigned char*>(workspace);
    p.partials = reinterpret_cast<float*>(base);
    p.tickets = shape.splits > 0 ? nullptr : reinterpret_cast<int*>(base + kPartialBytes);
    const int row_bytes = fp8 ? p.in_features : p.in_features / 2;
    CUtensorMap map0, map1;
    cudaError_t encoded = encode_weight_map(&map0, packed0, p.out_features, row_bytes);
    if (encoded == cudaSuccess) {
        encoded = encode_weight_map(&map1, packed1, p.out_features, row_bytes);
    }
    if (encoded != cudaSuccess) {
        (void)take_next_projection();
        return encoded;
    }
    using Kernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                            const StreamKParams);
    static const Kernel kernels[10] = {
        nvfp4_streamk_kernel<false, false, 16, false>, nvfp4_streamk_kernel<false, false, 32, false>,
        nvfp4_streamk_kernel<false, true, 16, false>,  nvfp4_streamk_kernel<false, true, 32, false>,
        nvfp4_streamk_kernel<true, false, 16, false>,  nvfp4_streamk_kernel<true, false, 32, false>,
        nvfp4_streamk_kernel<false, false, 16, true>,  nvfp4_streamk_kernel<false, false, 32, true>,
        nvfp4_streamk_kernel<false, true, 16, true>,   nvfp4_streamk_kernel<false, true, 32, true>};
    static PerDevice<cudaError_t> opted_per_device;
    const cudaError_t* opted = opted_per_device.get([]() {
        for (const Kernel kernel : kernels) {
            const cudaError_t error =
                cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
            if (error != cudaSuccess) {
                return error;
            }
        }
        return cudaSuccess;
    });
    if (opted == nullptr || *opted != cudaSuccess) {
        (void)take_next_projection();
        return opted == nullptr ? cudaErrorInvalidDevice : *opted;
    }
    // The caller's hint about the projection that follows (one use).
    CUtensorMap next_map0 = map0, next_map1 = map1;
    p.next.valid = 0;
    const NextProjection hint = take_next_projection();
    if (hint.packed[0] != nullptr && hint.out_features > 0 && hint.in_features > 0) {
        const bool next_fp8 = hint.kind == 2;
        const bool next_swiglu = hint.kind == 1 || hint.kind == 4;
        const int next_row_bytes = next_fp8 ? hint.in_features : hint.in_features / 2;
        // kinds 3 and 4: a matrix / a SwiGLU pair that will run as a regular K split (qwc_nvfp4_w4a16_split,
        // the latency-mode projections)
        const LaunchShape next =
            shape_of(hint.out_features, hint.in_features, next_swiglu, next_fp8, hint.kind == 3 || hint.kind == 4);
        if (next.units > 0 &&
            encode_weight_map(&next_map0, hint.packed[0], hint.out_features, next_row_bytes) == cudaSuccess &&
            encode_weight_map(&next_map1, hint.packed[next_swiglu ? 1 : 0], hint.out_features, next_row_bytes) ==
                cudaSuccess) {
            p.next.valid = 1;
            p.next.swiglu = next_swiglu ? 1 : 0;
            p.next.nvfp4 = next_fp8 ? 0 : 1;
            p.next.out_features = hint.out_features;
            p.next.ctas = next.ctas;
            p.next.units = next.units;
            p.next.splits = next.splits;
            p.next.stages_in_k = next.stages_in_k;
            p.next.group_blocks = hint.in_features / 64;
            p.next.scales[0] = static_cast<const uint8_t*>(hint.scales[0]);
            p.next.scales[1] = static_cast<const uint8_t*>(hint.scales[next_swiglu ? 1 : 0]);
        }
    }
    p.status = status_ptr();
    if (p.status == nullptr) {
        return cudaErrorInvalidValue;
    }
    const int n_pad = p.batch <= 16 ? 16 : 32;
    const bool regular = shape.splits > 0;  // no tickets: slices for the consumer, or whole pairs
    const Kernel kernel =
        kernels[(regular ? (swiglu ? 8 : 6) : (fp8 ? 4 : (swiglu ? 2 : 0))) + (n_pad == 32 ? 1 : 0)];
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(shape.ctas);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, map0, map1, next_map0, next_map1, p);
}

bool aligned16(const void* pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15) == 0; }

}  // namespace
}  // namespace qwc

using namespace qwc;

extern "C" size_t qwc_streamk_workspace_bytes(void) { return kWorkspaceBytes; }

// Timeline of the last launch: kMaxCtas x 32 nanosecond stamps (see QWC_STREAMK_TRACE above); returns the
// number of 64-bit words copied, 0 when the library was built without the trace.
extern "C" int qwc_streamk_trace(unsigned long long* host, int capacity_words) {
#ifdef QWC_STREAMK_TRACE
    const int words = kMaxCtas * kTraceSlots;
    if (host == nullptr || capacity_words < words ||
        cudaMemcpyFromSymbol(host, g_trace, sizeof(unsigned long long) * words) != cudaSuccess) {
        return -1;
    }
    return words;
#else
    (void)host;
    (void)capacity_words;
    return 0;
#endif
}

extern "C" int qwc_streamk_workspace_init(void* workspace, cudaStream_t stream) {
    if (workspace == nullptr || !aligned16(workspace)) {
        return cudaErrorInvalidValue;
    }
    return cudaMemsetAsync(workspace, 0, kWorkspaceBytes, stream);
}

extern "C" size_t qwc_staged_activation_bytes(int batch, int features) {
    if (batch <= 0 || batch > 32 || features <= 0 || features % 8 != 0) {
        return 0;
    }
    return static_cast<size_t>(features / 8) * (batch <= 16 ? 16 : 32) * 8 * sizeof(__half);
}

extern "C" int qwc_stage_activations(const void* input, void* staged, int batch, int in_features, cudaStream_t stream) {
    if (input == nullptr || staged == nullptr || batch <= 0 || batch > 32 || in_features <= 0 ||
        in_features % 8 != 0 || !aligned16(input) || !aligned16(staged)) {
        return cudaErrorInvalidValue;
    }
    const int threads = (in_features / 8) * batch;
    return launch_chained(stage_activations_kernel, dim3((threads + 255) / 256), dim3(256), 0, stream,
                          static_cast<const __nv_bfloat16*>(input), static_cast<__half*>(staged), batch, in_features,
                          batch <= 16 ? 16 : 32);
}

extern "C" int qwc_nvfp4_w4a16_staged(const void* packed, const void* scales, const void* staged_input, void* output,
                                      void* staged_output, int out_features, int in_features, int batch,
                                      float weight_global_scale, void* workspace, cudaStream_t stream) {
    if (packed == nullptr || scales == nullptr || staged_input == nullptr ||
        (output == nullptr && staged_output == nullptr) || workspace == nullptr || out_features <= 0 ||
        out_features % 8 != 0 || in_features <= 0 || in_features % 256 != 0 || batch <= 0 || batch > 32 ||
        !(weight_global_scale > 0.0f) || !aligned16(packed) || !aligned16(scales) || !aligned16(staged_input) ||
        !aligned16(workspace)) {
        (void)take_next_projection();  // a hint is good for one call, also for one that is refused
        return cudaErrorInvalidValue;
    }
    StreamKParams p = {};
    p.scales[0] = p.scales[1] = static_cast<const uint8_t*>(scales);
    p.x = static_cast<const __half*>(staged_input);
    p.y = static_cast<__nv_bfloat16*>(output);
    p.y_staged = static_cast<__half*>(staged_output);
    p.inverse_scale[0] = p.inverse_scale[1] = 1.0f / weight_global_scale;
    p.out_features = out_features;
    p.in_features = in_features;
    p.batch = batch;
    return launch_streamk(p, packed, packed, false, false, workspace, stream);
}

extern "C" int qwc_nvfp4_split_count(int out_features, int in_features) {
    if (out_features <= 0 || in_features <= 0 || in_features % 256 != 0) {
        return 0;
    }
    return shape_of(out_features, in_features, false, false, true).splits;
}

extern "C" int qwc_nvfp4_w4a16_split(const void* packed, const void* scales, const void* staged_input,
                                     float* partial_sums, int out_features, int in_features, int batch,
                                     cudaStream_t stream) {
    if (packed == nullptr || scales == nullptr || staged_input == nullptr || partial_sums == nullptr ||
        out_features <= 0 || in_features <= 0 || in_features % 256 != 0 || batch <= 0 || batch > 32 ||
        !aligned16(packed) || !aligned16(scales) || !aligned16(staged_input)) {
        (void)take_next_projection();
        return cudaErrorInvalidValue;
    }
    StreamKParams p = {};
    p.scales[0] = p.scales[1] = static_cast<const uint8_t*>(scales);
    p.x = static_cast<const __half*>(staged_input);
    p.inverse_scale[0] = p.inverse_scale[1] = 1.0f;
    p.out_features = out_features;
    p.in_features = in_features;
    p.batch = batch;
    p.split_out = partial_sums;
    return launch_streamk(p, packed, packed, false, false, nullptr, stream);
}

extern "C" int qwc_nvfp4_swiglu_w4a16_staged(const void* gate_packed, const void* gate_scales, const void* up_packed,
                                             const void* up_scales, const void* staged_input, void* output,
                                             void* staged_output, int out_features, int in_features, int batch,
                                             float gate_global_scale, float up_global_scale, void* workspace,
                                             cudaStream_t stream) {
    if (gate_packed == nullptr || gate_scales == nullptr || up_packed == nullptr || up_scales == nullptr ||
        staged_input == nullptr || (output == nullptr && staged_output == nullptr) || workspace == nullptr ||
        out_features <= 0 || out_features % 8 != 0 || in_features <= 0 || in_features % 256 != 0 || batch <= 0 ||
        batch > 32 || !(gate_global_scale > 0.0f) || !(up_global_scale > 0.0f) || !aligned16(gate_packed) ||
        !aligned16(gate_scales) || !aligned16(up_packed) || !aligned16(up_scales) || !aligned16(staged_input) ||
        !aligned16(workspace)) {
        (void)take_next_projection();
        return cudaErrorInvalidValue;
    }
    StreamKParams p = {};
    p.scales[0] = static_cast<const uint8_t*>(gate_scales);
    p.scales[1] = static_cast<const uint8_t*>(up_scales);
    p.x = static_cast<const __half*>(staged_input);
    p.y = static_cast<__nv_bfloat16*>(output);
    p.y_staged = static_cast<__half*>(staged_output);
    p.inverse_scale[0] = 1.0f / gate_global_scale;
    p.inverse_scale[1] = 1.0f / up_global_scale;
    p.out_features = out_features;
    p.in_features = in_features;
    p.batch = batch;
    return launch_streamk(p, gate_packed, up_packed, true, false, workspace, stream);
}

extern "C" int qwc_fp8_lm_head_staged(const void* weights, const void* row_scales, const void* staged_input,
                                      void* logits, void* sampled, void* status_out, int batch, int hidden_size,
                                      int vocab, void* workspace, cudaStream_t stream) {
    if (weights == nullptr || row_scales == nullptr || staged_input == nullptr ||
        (logits == nullptr && sampled == nullptr) || workspace == nullptr || batch <= 0 || batch > 32 ||
        hidden_size <= 0 || hidden_size % 256 != 0 || vocab <= 0 || !aligned16(weights) ||
        !aligned16(staged_input) || !aligned16(workspace)) {
        (void)take_next_projection();
        return cudaErrorInvalidValue;
    }
    StreamKParams p = {};
    p.scales[0] = p.scales[1] = nullptr;
    p.x = static_cast<const __half*>(staged_input);
    p.y_f32 = static_cast<float*>(logits);
    p.row_scales = static_cast<const float*>(row_scales);
    p.inverse_scale[0] = p.inverse_scale[1] = 1.0f;
    p.out_features = vocab;
    p.in_features = hidden_size;
    p.batch = batch;
    unsigned char* base = static_cast<unsigned char*>(workspace);
    float* candidate_values = reinterpret_cast<float*>(base + kPartialBytes + kTicketBytes);
    uint32_t* candidate_indices = reinterpret_cast<uint32_t*>(candidate_values + 32 * kCandidateSlots);
    if (sampled != nullptr) {
        p.candidate_values = candidate_values;
        p.candidate_indices = candidate_indices;
    }
    const cudaError_t launched = launch_streamk(p, weights, weights, false, true, workspace, stream);
    if (launched != cudaSuccess || sampled == nullptr) {
        return launched;
    }
    int* status = status_ptr();
    if (status == nullptr) {
        return cudaErrorInvalidValue;
    }
    const LaunchShape shape = shape_of(vocab, hidden_size, false, true);
    return launch_chained(sample_candidates_kernel, dim3(batch), dim3(kSampleThreads), 0, stream, candidate_values,
                          candidate_indices, static_cast<uint32_t*>(sampled), shape.ctas * 4,
                          static_cast<const int*>(status), static_cast<uint32_t*>(status_out));
}

// ---- latency mode: projections that hand their slices to every rank (exchange.cuh) ----------------

extern "C" int qwc_nvfp4_exchange_slices(int out_features, int in_features, int swiglu) {
    if (out_features <= 0 || in_features <= 0 || in_features % 256 != 0) {
        return 0;
    }
    return shape_of(out_features, in_features, swiglu != 0, false, true).splits;
}

extern "C" size_t qwc_exchange_candidate_bytes(int ranks) {
    if (ranks < 1 || ranks > kMaxPeers) {
        return 0;
    }
    return static_cast<size_t>(ranks) * kMaxCtas * 4 * 2 * sizeof(uint2);
}

extern "C" int qwc_nvfp4_w4a16_exchange(const void* packed, const void* scales, const void* staged_input,
                                        const qwc_exchange_row* row, int out_features, int in_features,
                                        cudaStream_t stream) {
    if (packed == nullptr || scales == nullptr || staged_input == nullptr || !valid_exchange_row(row) ||
        out_features <= 0 || out_features % 8 != 0 || in_features <= 0 || in_features % 256 != 0 ||
        row->width != row->ranks * out_features || !aligned16(packed) || !aligned16(scales) || !aligned16(staged_input)) {
        (void)take_next_projection();
        return cudaErrorInvalidValue;
    }
    StreamKParams p = {};
    p.scales[0] = p.scales[1] = static_cast<const uint8_t*>(scales);
    p.x = static_cast<const __half*>(staged_input);
    p.inverse_scale[0] = p.inverse_scale[1] = 1.0f;
    p.out_features = out_features;
    p.in_features = in_features;
    p.batch = 1;
    p.exchange = exchange_target(*row, row->rank * out_features);
    return launch_streamk(p, packed, packed, false, false, nullptr, stream);
}

extern "C" int qwc_nvfp4_swiglu_w4a16_exchange(const void* gate_packed, const void* gate_scales, const void* up_packed,
                                               const void* up_scales, const void* staged_input,
                                               const qwc_exchange_row* row, int out_features, int in_features,
                                               cudaStream_t stream) {
    if (gate_packed == nullptr || gate_scales == nullptr || up_packed == nullptr || up_scales == nullptr ||
        staged_input == nullptr || !valid_exchange_row(row) || out_features <= 0 || out_features % 8 != 0 ||
        in_features <= 0 || in_features % 256 != 0 || row->width != 2 * row->ranks * out_features || !aligned16(gate_packed) ||
        !aligned16(gate_scales) || !aligned16(up_packed) || !aligned16(up_scales) || !aligned16(staged_input)) {
        (void)take_next_projection();
        return cudaErrorInvalidValue;
    }
    StreamKParams p = {};
    p.scales[0] = static_cast<const uint8_t*>(gate_scales);
    p.scales[1] = static_cast<const uint8_t*>(up_scales);
    p.x = static_cast<const __half*>(staged_input);
    p.inverse_scale[0] = p.inverse_scale[1] = 1.0f;
    p.out_features = out_features;
    p.in_features = in_features;
    p.batch = 1;
    p.exchange = exchange_target(*row, row->rank * out_features);
    return launch_streamk(p, gate_packed, up_packed, true, false, nullptr, stream);
}

extern "C" int qwc_fp8_lm_head_exchange(const void* weights, const void* row_scales, const void* staged_input,
                                        void* logits, const qwc_exchange_row* candidates, void* sampled,
                                        void* status_out,
                                        int hidden_size, int vocab_local, void* workspace, cudaStream_t stream) {
    int* status = status_ptr();
    if (weights == nullptr || row_scales == nullptr || staged_input == nullptr || !valid_exchange_row(candidates) ||
        workspace == nullptr || hidden_size <= 0 || hidden_size % 256 != 0 || vocab_local <= 0 ||
        !aligned16(weights) || !aligned16(staged_input) || !aligned16(workspace) || status == nullptr) {
        (void)take_next_projection();
        return cudaErrorInvalidValue;
    }
    const LaunchShape shape = shape_of(vocab_local, hidden_size, false, true);
    const int slots_per_rank = shape.ctas * 4;
    StreamKParams p = {};
    p.scales[0] = p.scales[1] = nullptr;
    p.x = static_cast<const __half*>(staged_input);
    p.y_f32 = static_cast<float*>(logits);  // this rank's columns only, or null
    p.row_scales = static_cast<const float*>(row_scales);
    p.inverse_scale[0] = p.inverse_scale[1] = 1.0f;
    p.out_features = vocab_local;
    p.in_features = hidden_size;
    p.batch = 1;
    unsigned char* base = static_cast<unsigned char*>(workspace);
    p.candidate_values = reinterpret_cast<float*>(base + kPartialBytes + kTicketBytes);  // marks the sampling form
    p.candidate_indices = reinterpret_cast<uint32_t*>(p.candidate_values + 32 * kCandidateSlots);
    p.exchange = exchange_target(*candidates, candidates->rank * slots_per_rank);
    p.index_offset = static_cast<uint32_t>(candidates->rank) * static_cast<uint32_t>(vocab_local);
    const cudaError_t launched = launch_streamk(p, weights, weights, false, true, workspace, stream);
    if (launched != cudaSuccess || sampled == nullptr) {
        return launched;  // sampled == NULL: the candidates only (another launch picks the token)
    }
    return launch_chained(sample_exchanged_kernel, dim3(1), dim3(kSampleThreads), 0, stream,
                          tagged_row(*candidates, 1, status), candidates->ranks * slots_per_rank,
                          static_cast<uint32_t*>(sampled), static_cast<uint32_t*>(status_out));
}
