// NVFP4 W4A16 weight-streaming GEMV / skinny GEMM for 1..32 activation rows.
//
// Replaces the launchers of crates/qwc-cuda/cuda/nvfp4.cu:489-537 and :585-643 behind the
// same C signatures.  The arithmetic contract is the reference's
// (crates/qwc-cuda/src/nvfp4.rs:597-635): W[n,k] = e2m1(nibble) * e4m3(scale[n, k/16]) /
// global, fp32 accumulation, bf16 output.
//
// Design for sm_100a.  The op is HBM-bound (4.5 bits per weight, read once), so the
// kernel is organised around keeping ~50 KB of 128-bit weight loads in flight per SM:
//   * one CTA per SM; each warp owns 16 or 32 weight rows and a private two-stage ring
//     in shared memory; every stage is filled by bulk-async copies (TMA 1-D) of 256
//     contiguous bytes per weight row plus the 128-byte pieces of the swizzled block
//     scales, completing on the warp's own mbarrier.  256-byte runs per row matter:
//     a probe on this part reads 64-byte runs over 34816 rows at 3.6 TB/s and 256-byte
//     runs at 5.4 TB/s (DRAM page locality), and the copies cost no registers;
//   * the e2m1 nibbles are expanded to f16 by the hardware converter and multiplied by
//     their e4m3 block scale in f16 - the product has at most six significant bits, so
//     it is exact - directly into mma.sync A fragments: the dequantised weights never
//     touch shared memory;
//   * the activation rows are the B operand: converted bf16 -> f16 once per CTA into a
//     double-buffered shared tile laid out so every B-fragment read is a conflict-free
//     16-byte access, and shared by all warps; 8, 16 or 32 rows cost the same weight
//     traffic (one pass over W for every row of the batch);
//   * narrow outputs (N = 5120) do not give 148 SMs enough rows, so K is split across a
//     thread-block cluster and the partial sums are reduced through distributed shared
//     memory: split-K across SMs without a global workspace or atomics.
//
// Row / scale mapping.  The block scales arrive in the 128x4 swizzled layout
// (cuda/nvfp4.cu:33-39): one 16-byte unit holds rows {r, r+32, r+64, r+96} x 4 groups.
// A thread's MMA rows are chosen from exactly that set, so one 16-byte load brings the
// scales of all its rows for a 64-element K span.
//
// Activations with |x| > 65504 saturate in the f16 conversion; the weights themselves
// are exact.

#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace qwc {

// tcgen05 paths (nvfp4_umma.cu): NVFP4 projections, and the e4m3 vocabulary head.
cudaError_t launch_nvfp4_umma(const void* packed0, const void* scales0, const void* packed1, const void* scales1,
                              const void* x, void* y, int out_features, int in_features, int batch, float inverse0,
                              float inverse1, bool swiglu, cudaStream_t stream);
cudaError_t launch_fp8_umma(const void* weights, const float* row_scales, const void* x, float* logits,
                            int out_features, int in_features, int batch, cudaStream_t stream);

namespace {

constexpr int kChunk = 128;   // K elements per chunk: 64 bytes of nibbles (128 of e4m3) per row
constexpr int kRowRun = 256;  // bytes of one weight row fetched by one bulk copy
constexpr int kRowPitch = 320;  // shared-memory pitch of a row: 16-byte groups of rows g, g+1 differ by 4
constexpr int kWeightStages = 2;
constexpr int kMaxWarps = 16;
constexpr int kMaxBatch = 32;
constexpr int kSmemLimit = 232448 - 1024;  // 227 KiB opt-in limit minus static barriers

struct GemvParams {
    const uint8_t* packed[2];
    const uint8_t* scales[2];
    const __nv_bfloat16* x;
    __nv_bfloat16* y;
    const float* row_scales;  // kFp8Rows: per-row fp32 scale
    float* y_f32;             // kFp8Rows: fp32 output
    float inverse_scale[2];
    int out_features;
    int in_features;
    int batch;
    int num_tiles;
    int tiles_per_cta;
    int splits;
    int* status;
};

// Weight formats served by the one streaming kernel.
constexpr int kNvfp4 = 0;        // e2m1 nibbles + e4m3 block scales, bf16 out
constexpr int kNvfp4Swiglu = 1;  // two such matrices, silu(gate) * up epilogue
constexpr int kFp8Rows = 2;      // e4m3 bytes + one fp32 scale per row, fp32 out (lm_head)

template <int NT, int MT, int MODE>
struct Config {
    static constexpr bool SWIGLU = MODE == kNvfp4Swiglu;
    static constexpr bool FP8 = MODE == kFp8Rows;
    static constexpr int kRows = SWIGLU ? 4 : 2 * MT;  // weight rows per thread
    static constexpr int kMTiles = SWIGLU ? 2 : MT;    // m16 tiles per warp
    static constexpr int kUnits = FP8 ? 0 : (SWIGLU ? 2 : 1);  // scale sets per warp
    static constexpr int kVec = FP8 ? 2 : 1;           // 16-byte weight reads per row per chunk
    static constexpr int kChunkBytes = FP8 ? 128 : 64; // bytes of one row per chunk
    static constexpr int kStageChunks = kRowRun / kChunkBytes;  // chunks per weight stage: 4 or 2
    static constexpr int kWarpRows = 8 * kRows;        // weight rows staged per warp: 16 or 32
    static constexpr int kScaleBytes = kUnits * kStageChunks * 2 * 128;
    static constexpr int kWarpStageBytes = kWarpRows * kRowPitch + kScaleBytes;
    static constexpr int kWarpBytes = kWeightStages * kWarpStageBytes;
    static constexpr int kXChunks = (NT == 4 || FP8) ? 2 : 4;   // chunks per activation stage
    static constexpr int kXStageBytes = kXChunks * NT * 4 * 512;
    static constexpr int kXBytes = 2 * kXStageBytes;
    static constexpr int kMaxTiles =
        (kSmemLimit - kXBytes) / kWarpBytes < kMaxWarps ? (kSmemLimit - kXBytes) / kWarpBytes : kMaxWarps;
};

template <int NT, int MT, int MODE>
__global__ void __launch_bounds__(kMaxWarps * 32, 1) nvfp4_gemv_kernel(const GemvParams p) {
    using C = Config<NT, MT, MODE>;
    constexpr bool SWIGLU = C::SWIGLU;
    constexpr bool FP8 = C::FP8;
    constexpr int V = C::kVec;
    constexpr int R = C::kRows;
    constexpr int WC = C::kStageChunks;
    constexpr int XC = C::kXChunks;

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t full[kMaxWarps][kWeightStages];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int threads = blockDim.x;

    pdl_launch_dependents();
    const int row_group = blockIdx.x / p.splits;
    const int split = blockIdx.x - row_group * p.splits;
    const int tile = row_group * p.tiles_per_cta + warp;
    const bool active = warp < p.tiles_per_cta && tile < p.num_tiles && !status_is_set(p.status);

    const int K = p.in_features;
    const int chunks = K / kChunk;
    const int c_begin = static_cast<int>(static_cast<long long>(chunks) * split / p.splits);
    const int c_end = static_cast<int>(static_cast<long long>(chunks) * (split + 1) / p.splits);
    const int group_blocks = K / 64;
    const int row_bytes = FP8 ? K : K / 2;

    unsigned char* x_base = smem;
    unsigned char* ring = smem + C::kXBytes + warp * C::kWarpBytes;

    // Row of staged slot `i` (0..R-1) for fragment row group `gg`, and the word of the
    // 16-byte scale unit that belongs to it.
    const int row_block = (SWIGLU || MT == 1) ? (tile >> 3) : (tile >> 2);
    const int quad = (SWIGLU || MT == 1) ? (tile & 3) : (tile & 3);
    const int hi = (SWIGLU || MT == 1) ? ((tile & 7) >> 2) : 0;
    auto row_of = [&](int i, int gg) {
        const int j = (SWIGLU || MT == 1) ? (2 * hi + (i & 1)) : i;
        return 128 * row_block + 8 * quad + gg + 32 * j;
    };
    int rows[R];
    bool row_ok[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        rows[i] = row_of(i, g);
        row_ok[i] = active && rows[i] < p.out_features;
    }

    // ---- weight staging: one bulk copy per row and stage, one mbarrier per stage -------
    if (lane == 0) {
        for (int s = 0; s < kWeightStages; ++s) {
            mbar_init(&full[warp][s], 1);
        }
        mbar_fence_init();
    }
    __syncwarp();

    const int my_copy_row = row_of(lane >> 3, lane & 7);
    const bool my_copy_ok = active && lane < C::kWarpRows && my_copy_row < p.out_features;
    const int valid_rows = __popc(__ballot_sync(0xffffffffu, my_copy_ok));
    const uint8_t* my_copy_src =
        p.packed[SWIGLU ? (lane >> 4) : 0] + static_cast<size_t>(my_copy_ok ? my_copy_row : 0) * row_bytes;
    // lanes 0..(kUnits * 2 WC - 1) copy the 128-byte scale pieces: unit = lane / (2 WC), piece = lane % (2 WC)
    const bool my_scale_lane = !FP8 && active && lane < C::kUnits * 2 * WC;
    const uint8_t* my_scale_src =
        FP8 ? nullptr
            : p.scales[SWIGLU ? (lane / (2 * WC)) : 0] +
                  (static_cast<size_t>(active ? row_block : 0) * group_blocks + (lane % (2 * WC))) * 512 + quad * 128;

    auto issue_weights = [&](int stage) {
        const int slot = stage % kWeightStages;
        const int first = c_begin + stage * WC;
        const int n = min(WC, c_end - first);
        unsigned char* dst = ring + slot * C::kWarpStageBytes;
        if (lane == 0) {
            const uint32_t bytes = valid_rows * n * C::kChunkBytes + (FP8 ? 0 : C::kUnits * n * 2 * 128);
            mbar_arrive_expect_tx(&full[warp][slot], bytes);
        }
        __syncwarp();
        if (my_copy_ok) {
            bulk_g2s(dst + lane * kRowPitch, my_copy_src + static_cast<size_t>(first) * C::kChunkBytes,
                     n * C::kChunkBytes, &full[warp][slot]);
        }
        if (my_scale_lane && (lane % (2 * WC)) < 2 * n) {
            bulk_g2s(dst + C::kWarpRows * kRowPitch + lane * 128,
                     my_scale_src + static_cast<size_t>(first) * 1024, 128, &full[warp][slot]);
        }
    };

    // ---- activation staging: bf16 global -> f16 shared, B-fragment order ----------
    // A staging unit is 32 bytes of one token row: 16 elements = two 16-byte pieces.
    // Shared layout per stage: [chunk][n tile][piece 0..3][lane][16 B], so that the
    // B fragments of lane (g, t) for steps 2*piece and 2*piece+1 are one 16-byte read.
    constexpr int kHeld = 2;
    uint4 held[kHeld][2];
    auto stage_units = [&](int stage) {
        const int first = c_begin + stage * XC;
        const int n = min(XC, c_end - first);
        return n * NT * 64;
    };
    auto unit_source = [&](int stage, int u, bool& valid) {
        const int jj = u & 1;
        const int tt = (u >> 1) & 3;
        const int gg = (u >> 3) & 7;
        const int rest = u >> 6;
        const int n = rest % NT;
        const int cc = rest / NT;
        const int token = 8 * n + gg;
        valid = token < p.batch;
        // Element e of lane (g, t) is k = 32 t + e for nibbles (one 16-byte read per row);
        // for bytes the two reads sit 64 bytes apart: k = 16 t + e, then 64 + 16 t + (e - 16).
        const int k = (c_begin + stage * XC + cc) * kChunk + (FP8 ? 64 * jj + 16 * tt : 32 * tt + 16 * jj);
        return p.x + static_cast<size_t>(valid ? token : 0) * K + k;
    };
    auto unit_store = [&](unsigned char* buffer, int u, const uint4& lo, const uint4& hi4) {
        const int jj = u & 1;
        const int tt = (u >> 1) & 3;
        const int gg = (u >> 3) & 7;
        const int rest = u >> 6;  // cc * NT + n
        const uint32_t in[8] = {lo.x, lo.y, lo.z, lo.w, hi4.x, hi4.y, hi4.z, hi4.w};
        uint32_t out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            out[i] = bf16x2_to_f16x2(in[i]);
        }
        unsigned char* base = buffer + ((rest * 4 + 2 * jj) * 32 + 4 * gg + tt) * 16;
        *reinterpret_cast<uint4*>(base) = make_uint4(out[0], out[1], out[2], out[3]);
        *reinterpret_cast<uint4*>(base + 512) = make_uint4(out[4], out[5], out[6], out[7]);
    };
    auto stage_issue = [&](int stage) {
        const int total = stage_units(stage);
#pragma unroll
        for (int h = 0; h < kHeld; ++h) {
            const int u = threadIdx.x + h * threads;
            if (u < total) {
                bool valid;
                const __nv_bfloat16* src = unit_source(stage, u, valid);
                if (valid) {
                    held[h][0] = *reinterpret_cast<const uint4*>(src);
                    held[h][1] = *reinterpret_cast<const uint4*>(src + 8);
                } else {
                    held[h][0] = make_uint4(0, 0, 0, 0);
                    held[h][1] = make_uint4(0, 0, 0, 0);
                }
            }
        }
    };
    auto stage_commit = [&](int stage) {
        unsigned char* buffer = x_base + (stage & 1) * C::kXStageBytes;
        const int total = stage_units(stage);
#pragma unroll
        for (int h = 0; h < kHeld; ++h) {
            const int u = threadIdx.x + h * threads;
            if (u < total) {
                unit_store(buffer, u, held[h][0], held[h][1]);
            }
        }
        // Small CTAs have more units than two per thread: the rest go through directly.
        for (int u = threadIdx.x + kHeld * threads; u < total; u += threads) {
            bool valid;
            const __nv_bfloat16* src = unit_source(stage, u, valid);
            uint4 lo = make_uint4(0, 0, 0, 0), hi4 = lo;
            if (valid) {
                lo = *reinterpret_cast<const uint4*>(src);
                hi4 = *reinterpret_cast<const uint4*>(src + 8);
            }
            unit_store(buffer, u, lo, hi4);
        }
    };

    float acc[C::kMTiles][NT][4];
#pragma unroll
    for (int m = 0; m < C::kMTiles; ++m) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[m][n][j] = 0.0f;
            }
        }
    }

    // One chunk: `ws` is the warp's weight stage, `q` the chunk inside it, `xs` the chunk's
    // activation block.
    auto compute_chunk = [&](const unsigned char* xs, const unsigned char* ws, int q) {
        uint4 w[R][V];
#pragma unroll
        for (int i = 0; i < R; ++i) {
#pragma unroll
            for (int v = 0; v < V; ++v) {
                w[i][v] = *reinterpret_cast<const uint4*>(ws + (8 * i + g) * kRowPitch + q * C::kChunkBytes + 64 * v +
                                                          16 * t);
            }
        }
        // Block scales of this thread's two 16-element groups, per row, broadcast to f16x2.
        uint32_t scale_lo[R], scale_hi[R];
        if (!FP8) {
#pragma unroll
            for (int m = 0; m < C::kUnits; ++m) {
                const uint4 unit = *reinterpret_cast<const uint4*>(ws + C::kWarpRows * kRowPitch +
                                                                   (m * 2 * WC + 2 * q + (t >> 1)) * 128 + g * 16);
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    if ((SWIGLU ? (i >> 1) : 0) != m) {
                        continue;
                    }
                    const int sel = (SWIGLU || MT == 1) ? (2 * hi + (i & 1)) : i;
                    const uint32_t word = sel == 0 ? unit.x : (sel == 1 ? unit.y : (sel == 2 ? unit.z : unit.w));
                    const uint32_t pair = cvt_e4m3x2_to_f16x2(word >> (16 * (t & 1)));
                    scale_lo[i] = __byte_perm(pair, 0, 0x1010);
                    scale_hi[i] = __byte_perm(pair, 0, 0x3232);
                }
            }
        }
#pragma unroll
        for (int sp = 0; sp < 4; ++sp) {
            uint4 b[NT];
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                b[n] = *reinterpret_cast<const uint4*>(xs + ((n * 4 + sp) * 32 + lane) * 16);
            }
#pragma unroll
            for (int m = 0; m < C::kMTiles; ++m) {
                uint32_t h0[4], h1[4];
                if (FP8) {
                    // Elements 8 sp .. 8 sp + 7 are bytes 8 sp .. of the thread's 32: two words.
                    const uint4& v0 = w[2 * m][sp >> 1];
                    const uint4& v1 = w[2 * m + 1][sp >> 1];
                    const uint32_t a0 = (sp & 1) ? v0.z : v0.x, a1 = (sp & 1) ? v0.w : v0.y;
                    const uint32_t b0 = (sp & 1) ? v1.z : v1.x, b1 = (sp & 1) ? v1.w : v1.y;
                    cvt_e4m3x4_to_f16x2(a0, h0[0], h0[1]);
                    cvt_e4m3x4_to_f16x2(a1, h0[2], h0[3]);
                    cvt_e4m3x4_to_f16x2(b0, h1[0], h1[1]);
                    cvt_e4m3x4_to_f16x2(b1, h1[2], h1[3]);
                } else {
                    const uint32_t w0[4] = {w[2 * m][0].x, w[2 * m][0].y, w[2 * m][0].z, w[2 * m][0].w};
                    const uint32_t w1[4] = {w[2 * m + 1][0].x, w[2 * m + 1][0].y, w[2 * m + 1][0].z,
                                            w[2 * m + 1][0].w};
                    cvt_e2m1x8_to_f16x2(w0[sp], h0);
                    cvt_e2m1x8_to_f16x2(w1[sp], h1);
                    const uint32_t s0 = sp < 2 ? scale_lo[2 * m] : scale_hi[2 * m];
                    const uint32_t s1 = sp < 2 ? scale_lo[2 * m + 1] : scale_hi[2 * m + 1];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        h0[j] = hmul2_bits(h0[j], s0);
                        h1[j] = hmul2_bits(h1[j], s1);
                    }
                }
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    mma_f16_16816(acc[m][n], h0[0], h1[0], h0[1], h1[1], b[n].x, b[n].y);
                    mma_f16_16816(acc[m][n], h0[2], h1[2], h0[3], h1[3], b[n].z, b[n].w);
                }
            }
        }
    };

    // ---- main loop ------------------------------------------------------------------
    const int total_chunks = c_end - c_begin;
    const int num_wstages = (total_chunks + WC - 1) / WC;
    const int num_xstages = (total_chunks + XC - 1) / XC;
    bool alive = active;
    if (alive) {
#pragma unroll
        for (int s = 0; s < kWeightStages; ++s) {
            if (s < num_wstages) {
                issue_weights(s);
            }
        }
    }
    // The weight copies above start before the kernel that produces the activations has finished.
    pdl_wait();
    if (num_xstages > 0) {
        stage_issue(0);
        stage_commit(0);
    }
    for (int wstage = 0; wstage < num_wstages; ++wstage) {
        const int slot = wstage % kWeightStages;
        if (alive) {
            const bool arrived =
                mbar_wait_bounded(&full[warp][slot], (wstage / kWeightStages) & 1, kStatusGemvWait, p.status);
            alive = __all_sync(0xffffffffu, arrived);
        }
        const unsigned char* ws = ring + slot * C::kWarpStageBytes;
#pragma unroll
        for (int q = 0; q < WC; ++q) {
            const int rel = wstage * WC + q;
            if (rel < total_chunks) {
                const int xstage = rel / XC;
                const bool more = xstage + 1 < num_xstages;
                if (rel % XC == 0) {
                    __syncthreads();  // activation stage visible; the other buffer is free again
                    if (more) {
                        stage_issue(xstage + 1);
                    }
                }
                if (alive) {
                    compute_chunk(x_base + (xstage & 1) * C::kXStageBytes + (rel % XC) * (NT * 4 * 512), ws, q);
                }
                if (more && (rel % XC == XC - 1)) {
                    stage_commit(xstage + 1);
                }
            }
        }
        __syncwarp();
        if (alive && wstage + kWeightStages < num_wstages) {
            issue_weights(wstage + kWeightStages);
        }
    }

    // ---- split-K reduction through distributed shared memory ------------------------
    if (p.splits > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        float* reduce = reinterpret_cast<float*>(smem);
        __syncthreads();
        if (split != 0) {
#pragma unroll
            for (int m = 0; m < C::kMTiles; ++m) {
#pragma unroll
                for (int n = 0; n < NT; ++n) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        reduce[((m * NT + n) * 4 + j) * threads + threadIdx.x] = acc[m][n][j];
                    }
                }
            }
        }
        cluster.sync();
        if (split == 0) {
            for (int r = 1; r < p.splits; ++r) {
                const float* peer = cluster.map_shared_rank(reduce, r);
#pragma unroll
                for (int m = 0; m < C::kMTiles; ++m) {
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            acc[m][n][j] += peer[((m * NT + n) * 4 + j) * threads + threadIdx.x];
                        }
                    }
                }
            }
        }
        cluster.sync();
        if (split != 0) {
            return;
        }
    }

    // ---- epilogue ---------------------------------------------------------------------
    if (!alive) {
        return;
    }
    const int N = p.out_features;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int token = 8 * n + 2 * t + (j & 1);
            if (token >= p.batch) {
                continue;
            }
            if (SWIGLU) {
                const int i = j >> 1;  // rows[0], rows[1] (gate) pair with rows[2], rows[3] (up)
                if (!row_ok[i]) {
                    continue;
                }
                const float gate = acc[0][n][j] * p.inverse_scale[0];
                const float up = acc[1][n][j] * p.inverse_scale[1];
                const float silu = gate / (1.0f + __expf(-gate));
                p.y[static_cast<size_t>(token) * N + rows[i]] = __float2bfloat16(silu * up);
            } else {
#pragma unroll
                for (int m = 0; m < C::kMTiles; ++m) {
                    const int i = 2 * m + (j >> 1);
                    if (!row_ok[i]) {
                        continue;
                    }
                    if (FP8) {
                        p.y_f32[static_cast<size_t>(token) * N + rows[i]] = acc[m][n][j] * p.row_scales[rows[i]];
                    } else {
                        p.y[static_cast<size_t>(token) * N + rows[i]] =
                            __float2bfloat16(acc[m][n][j] * p.inverse_scale[0]);
                    }
                }
            }
        }
    }
}

// ---- host side ----------------------------------------------------------------------

int sm_count() {
    static int cached[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64) {
        return 148;
    }
    if (cached[device] == 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
            sms = 148;
        }
        cached[device] = sms;
    }
    return cached[device];
}

struct Plan {
    int tiles_per_cta;
    int splits;
    int ctas;
};

// Picks warps per CTA and the K split so that one wave of CTAs covers the SMs evenly.
// `resident_clusters[i]` is how many clusters of 1 << i CTAs the device holds at once: a cluster
// must sit inside one GPC, so this is less than sms / size for sizes that do not divide a GPC.
Plan choose_plan(int num_tiles, int chunks, int sms, int max_tiles, const int (&resident_clusters)[4]) {
    Plan best = {1, 1, num_tiles};
    double best_score = -1.0;
    for (int splits = 1, index = 0; splits <= 8; splits *= 2, ++index) {
        if (chunks / splits < 4 && splits > 1) {
            break;
        }
        const int clusters = splits == 1 ? sms : resident_clusters[index];
        if (clusters <= 0) {
            continue;
        }
        int tiles_per_cta = (num_tiles + clusters - 1) / clusters;
        tiles_per_cta = tiles_per_cta < 1 ? 1 : (tiles_per_cta > max_tiles ? max_tiles : tiles_per_cta);
        const int row_groups = (num_tiles + tiles_per_cta - 1) / tiles_per_cta;
        const int ctas = row_groups * splits;
        const int waves = (row_groups + clusters - 1) / clusters;
        const int slice = (chunks + splits - 1) / splits;
        const double useful = static_cast<double>(num_tiles) * chunks;
        const double spent = static_cast<double>(waves) * sms * tiles_per_cta * slice;
        double score = useful / spent;
        // Few warps per SM cannot keep enough loads in flight; a wider split costs a
        // cluster reduction.
        const double depth = tiles_per_cta >= max_tiles / 2 ? 1.0 : (0.5 + tiles_per_cta / (1.0 * max_tiles));
        score *= depth;
        score *= 1.0 - 0.015 * (splits == 1 ? 0 : (splits == 2 ? 1 : (splits == 4 ? 2 : 3)));
        if (score > best_score) {
            best_score = score;
            best = {tiles_per_cta, splits, ctas};
        }
    }
    return best;
}

template <int NT, int MT, int MODE>
cudaError_t launch(const GemvParams& base, cudaStream_t stream) {
    using C = Config<NT, MT, MODE>;
    constexpr bool SWIGLU = C::SWIGLU;
    GemvParams p = base;
    const int row_blocks = (p.out_features + 127) / 128;
    p.num_tiles = row_blocks * ((SWIGLU || MT == 1) ? 8 : 4);
    static PerDevice<cudaError_t> opted_per_device;
    const cudaError_t* opted = opted_per_device.get([]() {
        return cudaFuncSetAttribute(nvfp4_gemv_kernel<NT, MT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemLimit);
    });
    if (opted == nullptr) {
        return cudaErrorInvalidDevice;
    }
    if (*opted != cudaSuccess) {
        return *opted;
    }
    // Resident clusters of 1, 2, 4 and 8 full-size CTAs, asked of the driver once.
    struct Residency {
        int clusters[4];
    };
    static PerDevice<Residency> residency_per_device;
    const Residency* residency_found = residency_per_device.get([]() {
        Residency r = {};
        for (int index = 0; index < 4; ++index) {
            cudaLaunchConfig_t probe = {};
            probe.gridDim = dim3((1 << index) * 64);
            probe.blockDim = dim3(C::kMaxTiles * 32);
            probe.dynamicSmemBytes = C::kXBytes + C::kMaxTiles * C::kWarpBytes;
            cudaLaunchAttribute attribute[1];
            attribute[0].id = cudaLaunchAttributeClusterDimension;
            attribute[0].val.clusterDim.x = 1 << index;
            attribute[0].val.clusterDim.y = 1;
            attribute[0].val.clusterDim.z = 1;
            probe.attrs = attribute;
            probe.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, nvfp4_gemv_kernel<NT, MT, MODE>, &probe) != cudaSuccess) {
                clusters = 0;
                (void)cudaGetLastError();
            }
            r.clusters[index] = clusters;
        }
        return r;
    });
    if (residency_found == nullptr) {
        return cudaErrorInvalidDevice;
    }
    const Residency& residency = *residency_found;
    const Plan plan =
        choose_plan(p.num_tiles, p.in_features / kChunk, sm_count(), C::kMaxTiles, residency.clusters);
    p.tiles_per_cta = plan.tiles_per_cta;
    p.splits = plan.splits;
    p.status = status_ptr();
    if (p.status == nullptr) {
        return cudaErrorInvalidValue;
    }

    // The split-K reduction reuses the front of the buffer: kAcc floats per thread.
    const int reduce_bytes = plan.splits > 1 ? C::kMTiles * NT * 16 * plan.tiles_per_cta * 32 : 0;
    int smem_bytes = C::kXBytes + plan.tiles_per_cta * C::kWarpBytes;
    smem_bytes = smem_bytes < reduce_bytes ? reduce_bytes : smem_bytes;

    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(plan.ctas);
    config.blockDim = dim3(plan.tiles_per_cta * 32);
    config.dynamicSmemBytes = smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = plan.splits;
    attribute[1].val.clusterDim.y = 1;
    attribute[1].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = plan.splits > 1 ? 2 : 1;
    return cudaLaunchKernelEx(&config, nvfp4_gemv_kernel<NT, MT, MODE>, p);
}

thread_local NextProjection g_next_projection = {};

}  // namespace

void set_next_projection(const NextProjection& next) { g_next_projection = next; }

NextProjection take_next_projection() {
    const NextProjection taken = g_next_projection;
    g_next_projection = NextProjection{};
    return taken;
}

namespace {

template <int MODE>
cudaError_t dispatch(const GemvParams& p, cudaStream_t stream) {
    const int wide_tiles = ((p.out_features + 127) / 128) * 4;
    const bool wide = MODE == kNvfp4 && wide_tiles >= 2 * sm_count();
    // The tcgen05 kernel streams weights faster than the mma.sync one at every batch size but has a
    // longer start-up (TMEM allocation, first TMA round trip, cluster reduction): it takes over
    // above eight rows, and below that for matrices of 30 MB and more.
    const bool large = static_cast<long long>(p.out_features) * p.in_features >= 60ll * 1000 * 1000;
    // its stores are 16 bytes wide and its activation fetch is a tiled TMA copy
    const bool aligned = p.out_features % 8 == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 &&
                         ((reinterpret_cast<uintptr_t>(p.packed[0]) | reinterpret_cast<uintptr_t>(p.packed[1]) |
                           reinterpret_cast<uintptr_t>(p.scales[0]) | reinterpret_cast<uintptr_t>(p.scales[1])) & 15) == 0 &&
                         (MODE != kFp8Rows || ((reinterpret_cast<uintptr_t>(p.y_f32) & 15) == 0 &&
                                               (reinterpret_cast<uintptr_t>(p.row_scales) & 15) == 0));
    if (p.batch <= 8 && !(large && aligned)) {
        (void)take_next_projection();  // only the tcgen05 kernel acts on the hint; it is good for one launch
        return launch<1, 1, MODE>(p, stream);
    }
    if (MODE == kFp8Rows && aligned) {
        return launch_fp8_umma(p.packed[0], p.row_scales, p.x, p.y_f32, p.out_features, p.in_features, p.batch,
                               stream);
    }
    if (MODE != kFp8Rows && aligned) {
        // Above eight rows the legacy tensor path cannot keep up with the weight stream.
        return launch_nvfp4_umma(p.packed[0], p.scales[0], p.packed[1], p.scales[1], p.x, p.y, p.out_features,
                                 p.in_features, p.batch, p.inverse_scale[0], p.inverse_scale[1],
                                 MODE == kNvfp4Swiglu, stream);
    }
    (void)take_next_projection();
    if (p.batch <= 16) {
        return wide ? launch<2, 2, MODE>(p, stream) : launch<2, 1, MODE>(p, stream);
    }
    return wide ? launch<4, 2, MODE>(p, stream) : launch<4, 1, MODE>(p, stream);
}

}  // namespace

// Entry for the FP8 vocabulary head (vocab_head.cu): same streaming kernel, byte weights.
cudaError_t launch_fp8_rows(const void* weights, const float* row_scales, const void* hidden, float* logits,
                            int batch, int hidden_size, int vocab, cudaStream_t stream) {
    GemvParams p = {};
    p.packed[0] = p.packed[1] = static_cast<const uint8_t*>(weights);
    p.scales[0] = p.scales[1] = static_cast<const uint8_t*>(weights);
    p.x = static_cast<const __nv_bfloat16*>(hidden);
    p.row_scales = row_scales;
    p.y_f32 = logits;
    p.inverse_scale[0] = p.inverse_scale[1] = 1.0f;
    p.out_features = vocab;
    p.in_features = hidden_size;
    p.batch = batch;
    return dispatch<kFp8Rows>(p, stream);
}

namespace {

}  // namespace
}  // namespace qwc

extern "C" int qwc_nvfp4_prefetch_next(const void* packed0, const void* scales0, const void* packed1,
                                       const void* scales1, int out_features, int in_features, int kind) {
    const bool pair = kind == 1 || kind == 4;
    const bool rows = kind == 2;
    if (kind < 0 || kind > 4 || packed0 == nullptr || (!rows && scales0 == nullptr) ||
        (pair && (packed1 == nullptr || scales1 == nullptr)) || out_features <= 0 || in_features <= 0 ||
        in_features % 256 != 0 ||
        ((reinterpret_cast<uintptr_t>(packed0) | reinterpret_cast<uintptr_t>(scales0) |
          reinterpret_cast<uintptr_t>(packed1) | reinterpret_cast<uintptr_t>(scales1)) & 15) != 0) {
        return cudaErrorInvalidValue;
    }
    qwc::NextProjection next = {};
    next.packed[0] = packed0;
    next.packed[1] = pair ? packed1 : packed0;
    next.scales[0] = rows ? packed0 : scales0;
    next.scales[1] = pair ? scales1 : next.scales[0];
    next.out_features = out_features;
    next.in_features = in_features;
    next.kind = kind;
    qwc::set_next_projection(next);
    return cudaSuccess;
}

extern "C" int qwc_nvfp4_w4a16(const void* packed, const void* scales, const void* input, void* output,
                               int out_features, int in_features, int batch, float weight_global_scale,
                               cudaStream_t stream) {
    if (packed == nullptr || scales == nullptr || input == nullptr || output == nullptr || out_features <= 0 ||
        in_features <= 0 || in_features % 256 != 0 || batch <= 0 || batch > qwc::kMaxBatch ||
        !(weight_global_scale > 0.0f)) {
        (void)qwc::take_next_projection();  // a hint is good for one call, also for one that is refused
        return cudaErrorInvalidValue;
    }
    qwc::GemvParams p = {};
    p.packed[0] = static_cast<const uint8_t*>(packed);
    p.scales[0] = static_cast<const uint8_t*>(scales);
    p.packed[1] = p.packed[0];
    p.scales[1] = p.scales[0];
    p.x = static_cast<const __nv_bfloat16*>(input);
    p.y = static_cast<__nv_bfloat16*>(output);
    p.inverse_scale[0] = 1.0f / weight_global_scale;
    p.inverse_scale[1] = p.inverse_scale[0];
    p.out_features = out_features;
    p.in_features = in_features;
    p.batch = batch;
    return qwc::dispatch<qwc::kNvfp4>(p, stream);
}

extern "C" int qwc_nvfp4_swiglu_w4a16(const void* gate_packed, const void* gate_scales, const void* up_packed,
                                      const void* up_scales, const void* input, void* output, int out_features,
                                      int in_features, int batch, float gate_global_scale, float up_global_scale,
                                      cudaStream_t stream) {
    if (gate_packed == nullptr || gate_scales == nullptr || up_packed == nullptr || up_scales == nullptr ||
        input == nullptr || output == nullptr || out_features <= 0 || in_features <= 0 ||
        in_features % 256 != 0 || batch <= 0 || batch > qwc::kMaxBatch || !(gate_global_scale > 0.0f) ||
        !(up_global_scale > 0.0f)) {
        (void)qwc::take_next_projection();
        return cudaErrorInvalidValue;
    }
    qwc::GemvParams p = {};
    p.packed[0] = static_cast<const uint8_t*>(gate_packed);
    p.scales[0] = static_cast<const uint8_t*>(gate_scales);
    p.packed[1] = static_cast<const uint8_t*>(up_packed);
    p.scales[1] = static_cast<const uint8_t*>(up_scales);
    p.x = static_cast<const __nv_bfloat16*>(input);
    p.y = static_cast<__nv_bfloat16*>(output);
    p.inverse_scale[0] = 1.0f / gate_global_scale;
    p.inverse_scale[1] = 1.0f / up_global_scale;
    p.out_features = out_features;
    p.in_features = in_features;
    p.batch = batch;
    return qwc::dispatch<qwc::kNvfp4Swiglu>(p, stream);
}
