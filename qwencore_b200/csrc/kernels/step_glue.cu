// Small per-row kernels between the streaming ops of the decode step: embedding gather,
// residual RMSNorm, DeltaNet pre- and post-processing, QK-norm + RoPE + FP8 page write,
// vocabulary head entry points and greedy argmax.  Each is a few hundred KB of traffic
// per layer, so the aim is few launches and wide accesses, not roofline.
//
// Rounding points follow the reference kernels exactly (file:line at each launcher).

#include <cooperative_groups.h>

#include "common.cuh"
#include "exchange.cuh"

namespace qwc {

cudaError_t launch_fp8_rows(const void* weights, const float* row_scales, const void* hidden, float* logits,
                            int batch, int hidden_size, int vocab, cudaStream_t stream);

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float fp8_to_float(uint8_t raw) {
    __nv_fp8_e4m3 value;
    value.__x = raw;
    return static_cast<float>(value);
}

__device__ __forceinline__ uint8_t to_fp8(float value) {
    __nv_fp8_e4m3 converted(value);
    return converted.__x;
}

__device__ __forceinline__ float sigmoidf_fast(float x) { return 1.0f / (1.0f + __expf(-x)); }

// Sum over the CTA; every thread receives the total.  `scratch` holds one float per warp.
__device__ __forceinline__ float block_sum(float value, float* scratch) {  // scratch: blockDim.x / 32 floats
    value = warp_sum(value);
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) {
        scratch[warp] = value;
    }
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) {
        total += scratch[w];
    }
    return total;
}

// ---- embedding gather (cuda/vocab_fp8.cu:113-136) ---------------------------------
__global__ void embedding_gather_kernel(const uint8_t* __restrict__ table, const float* __restrict__ row_scales,
                                        const uint32_t* __restrict__ token_ids, __nv_bfloat16* __restrict__ output,
                                        int cols, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t token = token_ids[blockIdx.x];
    const size_t output_base = static_cast<size_t>(blockIdx.x) * cols;
    const bool valid = token < static_cast<uint32_t>(vocab);
    const float scale = valid ? row_scales[token] : 0.0f;
    const size_t table_base = static_cast<size_t>(valid ? token : 0) * cols;
    for (int column = threadIdx.x; column < cols; column += blockDim.x) {
        const float value = valid ? fp8_to_float(table[table_base + column]) * scale : 0.0f;
        output[output_base + column] = __float2bfloat16(value);
    }
}

// ---- bf16 rows -> e4m3 rows with one fp32 scale per row (cuda/vocab_fp8.cu:70-111) -----
// The weight loader's step for the vocabulary tables: scale = max|x| / 448 (1 for an all-zero row),
// code = e4m3(x / scale), round to nearest even, saturating.  A warp per row, eight rows per CTA: 16
// bytes per lane and load, the second pass over the row (10 KB at 5120 columns) comes from L1, and the
// codes leave eight bytes per lane.

__global__ void __launch_bounds__(kThreads) quantize_rows_kernel(const __nv_bfloat16* __restrict__ input,
                                                                 uint8_t* __restrict__ output,
                                                                 float* __restrict__ row_scales, int rows, int cols,
                                                                 int first_row) {
    const int lane = threadIdx.x & 31;
    const int local_row = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (local_row >= rows) {
        return;
    }
    const __nv_bfloat16* in = input + static_cast<size_t>(local_row) * cols;
    uint8_t* out = output + static_cast<size_t>(first_row + local_row) * cols;
    const int vectors = cols / 8;  // the launcher sends other widths to the scalar form below
    float peak = 0.0f;
    for (int v = lane; v < vectors; v += 32) {
        const uint4 raw = *reinterpret_cast<const uint4*>(in + 8 * v);
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            peak = fmaxf(peak, fmaxf(fabsf(__uint_as_float(words[j] << 16)), fabsf(__uint_as_float(words[j] & 0xffff0000u))));
        }
    }
    peak = warp_max(peak);
    const float scale = peak > 0.0f ? peak / 448.0f : 1.0f;
    if (lane == 0) {
        row_scales[first_row + local_row] = scale;
    }
    const float inverse = 1.0f / scale;
    for (int v = lane; v < vectors; v += 32) {
        const uint4 raw = *reinterpret_cast<const uint4*>(in + 8 * v);
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t packed[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 pair = make_float2(__uint_as_float(words[j] << 16) * inverse,
                                            __uint_as_float(words[j] & 0xffff0000u) * inverse);
            const uint32_t codes = __nv_cvt_float2_to_fp8x2(pair, __NV_SATFINITE, __NV_E4M3);
            packed[j >> 1] |= codes << (16 * (j & 1));
        }
        *reinterpret_cast<uint2*>(out + 8 * v) = make_uint2(packed[0], packed[1]);
    }
}

// ... any width, one column per thread step (rows whose width is not a multiple of eight)
__global__ void __launch_bounds__(kThreads) quantize_rows_scalar_kernel(const __nv_bfloat16* __restrict__ input,
                                                                        uint8_t* __restrict__ output,
                                                                        float* __restrict__ row_scales, int cols,
                                                                        int first_row) {
    __shared__ float scratch[kThreads / 32];
    const __nv_bfloat16* in = input + static_cast<size_t>(blockIdx.x) * cols;
    uint8_t* out = output + static_cast<size_t>(first_row + blockIdx.x) * cols;
    float peak = 0.0f;
    for (int c = threadIdx.x; c < cols; c += kThreads) {
        peak = fmaxf(peak, fabsf(__bfloat162float(in[c])));
    }
    peak = warp_max(peak);
    if ((threadIdx.x & 31) == 0) {
        scratch[threadIdx.x >> 5] = peak;
    }
    __syncthreads();
    peak = 0.0f;
    for (int w = 0; w < kThreads / 32; ++w) {
        peak = fmaxf(peak, scratch[w]);
    }
    const float scale = peak > 0.0f ? peak / 448.0f : 1.0f;
    if (threadIdx.x == 0) {
        row_scales[first_row + blockIdx.x] = scale;
    }
    const float inverse = 1.0f / scale;
    for (int c = threadIdx.x; c < cols; c += kThreads) {
        out[c] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(__bfloat162float(in[c]) * inverse, __NV_SATFINITE, __NV_E4M3));
    }
}

// ---- residual RMSNorm (cuda/rmsnorm.cu:85-149) --------------------------------------
// One CTA per row; the rounded bf16 row stays in registers between the two passes.
constexpr int kNormMaxPerThread = 10;  // 8 * 256 * 10 = 20480 columns at most

__global__ void __launch_bounds__(kThreads) rmsnorm_bf16_kernel(const __nv_bfloat16* __restrict__ input,
                                                                __nv_bfloat16* __restrict__ residual,
                                                                const __nv_bfloat16* __restrict__ weight,
                                                                __nv_bfloat16* __restrict__ output,
                                                                __half* __restrict__ staged, int padded_rows,
                                                                int hidden, float epsilon) {
    pdl_launch_dependents();  // the projection that follows may start streaming its weights
    __shared__ float scratch[kThreads / 32];
    const size_t base = static_cast<size_t>(blockIdx.x) * hidden;
    const int vectors = hidden / 8;
    // The norm weights are never written during a step: they are fetched while the kernel that
    // produces the input is still running.
    uint4 gains[kNormMaxPerThread];
#pragma unroll
    for (int i = 0; i < kNormMaxPerThread; ++i) {
        const int vec = threadIdx.x + i * kThreads;
        if (vec < vectors) {
            gains[i] = *reinterpret_cast<const uint4*>(weight + 8 * vec);
        }
    }
    pdl_wait();
    uint4 held[kNormMaxPerThread];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormMaxPerThread; ++i) {
        const int vec = threadIdx.x + i * kThreads;
        if (vec < vectors) {
            uint4 raw = *reinterpret_cast<const uint4*>(input + base + 8 * vec);
            uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
            if (residual != nullptr) {
                const uint4 res = *reinterpret_cast<const uint4*>(residual + base + 8 * vec);
                const uint32_t rw[4] = {res.x, res.y, res.z, res.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float lo = __uint_as_float(words[j] << 16) + __uint_as_float(rw[j] << 16);
                    const float hi = __uint_as_float(words[j] & 0xffff0000u) + __uint_as_float(rw[j] & 0xffff0000u);
                    __nv_bfloat162 rounded = __floats2bfloat162_rn(lo, hi);
                    words[j] = *reinterpret_cast<uint32_t*>(&rounded);
                }
                raw = make_uint4(words[0], words[1], words[2], words[3]);
                *reinterpret_cast<uint4*>(residual + base + 8 * vec) = raw;
            }
            held[i] = raw;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float lo = __uint_as_float(words[j] << 16);
                const float hi = __uint_as_float(words[j] & 0xffff0000u);
                sum = fmaf(lo, lo, sum);
                sum = fmaf(hi, hi, sum);
            }
        }
    }
    const float total = block_sum(sum, scratch);
    const float inverse = rsqrtf(total / static_cast<float>(hidden) + epsilon);
#pragma unroll
    for (int i = 0; i < kNormMaxPerThread; ++i) {
        const int vec = threadIdx.x + i * kThreads;
        if (vec < vectors) {
            const uint32_t ww[4] = {gains[i].x, gains[i].y, gains[i].z, gains[i].w};
            const uint32_t xw[4] = {held[i].x, held[i].y, held[i].z, held[i].w};
            uint32_t out[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float lo = __uint_as_float(xw[j] << 16) * inverse * (1.0f + __uint_as_float(ww[j] << 16));
                const float hi = __uint_as_float(xw[j] & 0xffff0000u) * inverse *
                                 (1.0f + __uint_as_float(ww[j] & 0xffff0000u));
                __nv_bfloat162 rounded = __floats2bfloat162_rn(lo, hi);
                out[j] = *reinterpret_cast<uint32_t*>(&rounded);
            }
            if (output != nullptr) {
                *reinterpret_cast<uint4*>(output + base + 8 * vec) = make_uint4(out[0], out[1], out[2], out[3]);
            }
            if (staged != nullptr) {
                // the same bf16 values as f16, where the projection that follows reads its operand:
                // [hidden / 8][padded rows][8]
                *reinterpret_cast<uint4*>(staged + (static_cast<size_t>(vec) * padded_rows + blockIdx.x) * 8) =
                    make_uint4(bf16x2_to_f16x2(out[0]), bf16x2_to_f16x2(out[1]), bf16x2_to_f16x2(out[2]),
                               bf16x2_to_f16x2(out[3]));
            }
        }
    }
}

// One output of a projection that ran as a regular K split (qwc_nvfp4_w4a16_split): the slices summed in
// slice order, scaled and rounded to bf16 as the projection's own epilogue would have done.  In latency
// mode the slices are tagged words that the ranks stored into one another's memory (exchange.cuh): one
// activation row, and a read that may have to wait for a peer.
struct SplitSource {
    const float* sums;  // [slices][batch][width] fp32, or null: the consumer reads bf16 rows instead
    int slices;
    int batch;
    int width;
    float scale;
    TaggedRow tagged;  // words != null: the exchanged form (sums is null then)
};

__device__ __forceinline__ bool has_slices(const SplitSource& source) {
    return source.sums != nullptr || source.tagged.words != nullptr;
}

// The tag that this step's words of an exchanged row carry (read once, after the wait for the preceding kernel).
__device__ __forceinline__ uint32_t split_tag(const SplitSource& source) {
    return source.tagged.words != nullptr ? exchange_tag(source.tagged.epoch, source.tagged.instance) : 0u;
}

// (The loads of up to four slices are issued together: one round trip, not one per slice.  A slice
// past the last one reads the last one again and adds nothing.)
template <bool kExchanged>
__device__ __forceinline__ float split_value(const SplitSource& source, uint32_t tag, int row, int column) {
    if (kExchanged) {
        return __bfloat162float(__float2bfloat16(tagged_sum(source.tagged, tag, column) * source.scale));
    }
    const size_t stride = static_cast<size_t>(source.batch) * source.width;
    const float* at = source.sums + static_cast<size_t>(row) * source.width + column;
    float total = 0.0f;
    for (int first = 0; first < source.slices; first += 4) {
        float part[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            part[j] = __ldcg(at + min(first + j, source.slices - 1) * stride);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            total += first + j < source.slices ? part[j] : 0.0f;
        }
    }
    return __bfloat162float(__float2bfloat16(total * source.scale));
}

// ---- residual RMSNorm that also finishes a K-split projection ------------------------
// The projection before a residual RMSNorm (mixer output, MLP down: 5120 outputs, too few row tiles
// for the SMs) runs as a regular K split and leaves fp32 partial rows [slice][batch][hidden]; summing
// them here costs this kernel nothing it would not wait for anyway (one round trip for its input),
// and the projection ends with plain stores instead of a reduction between CTAs.  The arithmetic is
// the unsplit one: x = bf16(sum * scale) is the projection's bf16 output (cuda/nvfp4.cu:209-220),
// then cuda/rmsnorm.cu:85-149 on x.  Slices are summed in slice order: bit-reproducible.
constexpr int kSplitNormThreads = 640;
constexpr int kSplitNormMaxItems = 4;  // float4 items per thread: hidden <= 4 * 4 * 640

template <bool kExchanged>  // the slices are another rank's tagged words (latency mode, one row)
__global__ void __launch_bounds__(kSplitNormThreads) rmsnorm_split_kernel(
    const float* __restrict__ partial_sums, int splits, float scale, __nv_bfloat16* __restrict__ projection,
    __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ weight,
    __nv_bfloat16* __restrict__ output, __half* __restrict__ staged, int padded_rows, int hidden, int batch,
    float epsilon, const TaggedRow exchanged) {
    pdl_launch_dependents();
    __shared__ float scratch[kSplitNormThreads / 32];
    const int token = blockIdx.x;
    const int items = hidden / 4;
    uint2 gains[kSplitNormMaxItems];
#pragma unroll
    for (int i = 0; i < kSplitNormMaxItems; ++i) {
        const int item = threadIdx.x + i * kSplitNormThreads;
        if (item < items) {
            gains[i] = *reinterpret_cast<const uint2*>(weight + 4 * item);  // static: fetched before the wait
        }
    }
    pdl_wait();
    const uint32_t tag = kExchanged ? exchange_tag(exchanged.epoch, exchanged.instance) : 0u;
    const size_t slice_stride = static_cast<size_t>(batch) * hidden;
    const float* mine = partial_sums + static_cast<size_t>(token) * hidden;
    float held[kSplitNormMaxItems][4];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kSplitNormMaxItems; ++i) {
        const int item = threadIdx.x + i * kSplitNormThreads;
        if (item < items) {
            uint2 res = make_uint2(0u, 0u);
            if (residual != nullptr) {
                res = *reinterpret_cast<const uint2*>(residual + static_cast<size_t>(token) * hidden + 4 * item);
            }
            // eight slices in flight at a time: the sum costs one round trip, not one per slice
            float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (kExchanged) {  // latency mode: the ranks' tagged slices of the one row
                total = tagged_sum4(exchanged, tag, 4 * item);
            }
            for (int first = 0; !kExchanged && first < splits; first += 8) {
                float4 part[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    part[j] = __ldcg(reinterpret_cast<const float4*>(mine + min(first + j, splits - 1) * slice_stride +
                                                                     4 * item));
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (first + j < splits) {
                        total.x += part[j].x;
                        total.y += part[j].y;
                        total.z += part[j].z;
                        total.w += part[j].w;
                    }
                }
            }
            // the projection's own output rounding, then the residual sum's
            float x[4] = {__bfloat162float(__float2bfloat16(total.x * scale)),
                          __bfloat162float(__float2bfloat16(total.y * scale)),
                          __bfloat162float(__float2bfloat16(total.z * scale)),
                          __bfloat162float(__float2bfloat16(total.w * scale))};
            if (projection != nullptr) {  // a caller that also wants the projection's own bf16 rows
                __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]);
                __nv_bfloat162 hi = __floats2bfloat162_rn(x[2], x[3]);
                *reinterpret_cast<uint2*>(projection + static_cast<size_t>(token) * hidden + 4 * item) =
                    make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            }
            if (residual != nullptr) {
                const float r[4] = {__uint_as_float(res.x << 16), __uint_as_float(res.x & 0xffff0000u),
                                    __uint_as_float(res.y << 16), __uint_as_float(res.y & 0xffff0000u)};
                __nv_bfloat162 lo = __floats2bfloat162_rn(x[0] + r[0], x[1] + r[1]);
                __nv_bfloat162 hi = __floats2bfloat162_rn(x[2] + r[2], x[3] + r[3]);
                const uint2 stored = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                *reinterpret_cast<uint2*>(residual + static_cast<size_t>(token) * hidden + 4 * item) = stored;
                x[0] = __uint_as_float(stored.x << 16);
                x[1] = __uint_as_float(stored.x & 0xffff0000u);
                x[2] = __uint_as_float(stored.y << 16);
                x[3] = __uint_as_float(stored.y & 0xffff0000u);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                held[i][j] = x[j];
                sum = fmaf(x[j], x[j], sum);
            }
        }
    }
    const float total = block_sum(sum, scratch);
    const float inverse = rsqrtf(total / static_cast<float>(hidden) + epsilon);
#pragma unroll
    for (int i = 0; i < kSplitNormMaxItems; ++i) {
        const int item = threadIdx.x + i * kSplitNormThreads;
        if (item < items) {
            const float g[4] = {__uint_as_float(gains[i].x << 16), __uint_as_float(gains[i].x & 0xffff0000u),
                                __uint_as_float(gains[i].y << 16), __uint_as_float(gains[i].y & 0xffff0000u)};
            __nv_bfloat162 lo = __floats2bfloat162_rn(held[i][0] * inverse * (1.0f + g[0]),
                                                      held[i][1] * inverse * (1.0f + g[1]));
            __nv_bfloat162 hi = __floats2bfloat162_rn(held[i][2] * inverse * (1.0f + g[2]),
                                                      held[i][3] * inverse * (1.0f + g[3]));
            const uint2 out = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            if (output != nullptr) {
                *reinterpret_cast<uint2*>(output + static_cast<size_t>(token) * hidden + 4 * item) = out;
            }
            if (staged != nullptr) {
                // half of a K core: [hidden / 8][padded rows][8]
                *reinterpret_cast<uint2*>(staged + (static_cast<size_t>(item >> 1) * padded_rows + token) * 8 +
                                          (item & 1) * 4) = make_uint2(bf16x2_to_f16x2(out.x), bf16x2_to_f16x2(out.y));
            }
        }
    }
}

// ---- the same with every row spread over a cluster -------------------------------------
// The kernel above is one CTA per row pulling every slice of the row through one SM (in latency mode
// 8 slices x 5120 x 8 bytes: several microseconds of one SM's L2 bandwidth, several times what the
// arithmetic takes), and its 640-thread CTAs do not fit on an SM beside a CTA of the projection
// kernel, so the projection that follows cannot start (and fetch its weights) on those SMs until the
// norm is over.  Here a row is divided over a cluster of eight CTAs, each summing and normalising
// hidden / 8 columns (one item of four columns per thread, every slice of it in flight at once, about
// 5 K registers per CTA: resident beside a projection CTA); the only thing they share is the sum of
// squares: each CTA stores its partial into every CTA's shared memory, one cluster barrier, and all
// add the eight partials in rank order.  Same arithmetic as above except for the order in which the
// squares are added.
constexpr int kRowNormCtas = 8;

template <bool kExchanged>
__global__ void __cluster_dims__(kRowNormCtas, 1, 1) __launch_bounds__(256)
    rmsnorm_row_cluster_kernel(const float* __restrict__ partial_sums, int splits, float scale,
                               __nv_bfloat16* __restrict__ projection, __nv_bfloat16* __restrict__ residual,
                               const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ output,
                               __half* __restrict__ staged, int padded_rows, int hidden, int batch, float epsilon,
                               const TaggedRow exchanged) {
    pdl_launch_dependents();
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float scratch[256 / 32];
    __shared__ float partials[kRowNormCtas];
    const int rank = static_cast<int>(cluster.block_rank());
    const int token = blockIdx.y;
    const size_t row_base = static_cast<size_t>(token) * hidden;
    const int items_per_cta = hidden / (4 * kRowNormCtas);
    const bool active = static_cast<int>(threadIdx.x) < items_per_cta;
    const int item = rank * items_per_cta + threadIdx.x;
    uint2 gains = make_uint2(0u, 0u);
    if (active) {
        gains = *reinterpret_cast<const uint2*>(weight + 4 * item);  // static: fetched before the wait
    }
    pdl_wait();
    float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float sum = 0.0f;
    if (active) {
        uint2 res = make_uint2(0u, 0u);
        if (residual != nullptr) {
            res = *reinterpret_cast<const uint2*>(residual + row_base + 4 * item);
        }
        float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (kExchanged) {
            total = tagged_sum4(exchanged, exchange_tag(exchanged.epoch, exchanged.instance), 4 * item);
        } else {
            for (int first = 0; first < splits; first += 8) {
                float4 part[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    part[j] = __ldcg(reinterpret_cast<const float4*>(
                        partial_sums + (static_cast<size_t>(min(first + j, splits - 1)) * batch + token) * hidden +
                        4 * item));
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (first + j < splits) {
                        total.x += part[j].x;
                        total.y += part[j].y;
                        total.z += part[j].z;
                        total.w += part[j].w;
                    }
                }
            }
        }
        x[0] = __bfloat162float(__float2bfloat16(total.x * scale));
        x[1] = __bfloat162float(__float2bfloat16(total.y * scale));
        x[2] = __bfloat162float(__float2bfloat16(total.z * scale));
        x[3] = __bfloat162float(__float2bfloat16(total.w * scale));
        if (projection != nullptr) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]);
            __nv_bfloat162 hi = __floats2bfloat162_rn(x[2], x[3]);
            *reinterpret_cast<uint2*>(projection + row_base + 4 * item) =
                make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
        if (residual != nullptr) {
            const float r[4] = {__uint_as_float(res.x << 16), __uint_as_float(res.x & 0xffff0000u),
                                __uint_as_float(res.y << 16), __uint_as_float(res.y & 0xffff0000u)};
            __nv_bfloat162 lo = __floats2bfloat162_rn(x[0] + r[0], x[1] + r[1]);
            __nv_bfloat162 hi = __floats2bfloat162_rn(x[2] + r[2], x[3] + r[3]);
            const uint2 stored = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            *reinterpret_cast<uint2*>(residual + row_base + 4 * item) = stored;
            x[0] = __uint_as_float(stored.x << 16);
            x[1] = __uint_as_float(stored.x & 0xffff0000u);
            x[2] = __uint_as_float(stored.y << 16);
            x[3] = __uint_as_float(stored.y & 0xffff0000u);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            sum = fmaf(x[j], x[j], sum);
        }
    }
    const float mine = block_sum(sum, scratch);
    if (threadIdx.x < kRowNormCtas) {
        *cluster.map_shared_rank(&partials[rank], threadIdx.x) = mine;  // into CTA threadIdx.x's copy
    }
    cluster.sync();
    float total = 0.0f;
#pragma unroll
    for (int r = 0; r < kRowNormCtas; ++r) {
        total += partials[r];
    }
    const float inverse = rsqrtf(total / static_cast<float>(hidden) + epsilon);
    if (active) {
        const float g[4] = {__uint_as_float(gains.x << 16), __uint_as_float(gains.x & 0xffff0000u),
                            __uint_as_float(gains.y << 16), __uint_as_float(gains.y & 0xffff0000u)};
        __nv_bfloat162 lo = __floats2bfloat162_rn(x[0] * inverse * (1.0f + g[0]), x[1] * inverse * (1.0f + g[1]));
        __nv_bfloat162 hi = __floats2bfloat162_rn(x[2] * inverse * (1.0f + g[2]), x[3] * inverse * (1.0f + g[3]));
        const uint2 out = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        if (output != nullptr) {
            *reinterpret_cast<uint2*>(output + row_base + 4 * item) = out;
        }
        if (staged != nullptr) {  // half of a K core: [hidden / 8][padded rows][8]
            *reinterpret_cast<uint2*>(staged + (static_cast<size_t>(item >> 1) * padded_rows + token) * 8 +
                                      (item & 1) * 4) =
                make_uint2(bf16x2_to_f16x2(out.x), bf16x2_to_f16x2(out.y));
        }
    }
}

// hidden a multiple of 256 and at most 8192: hidden / 32 threads per CTA (rounded up to warps)
template <bool kExchanged>
cudaError_t launch_row_norm(const float* partial_sums, int splits, float scale, void* projection, void* residual,
                            const void* weight, void* output, void* staged, int batch, int hidden, float epsilon,
                            const TaggedRow& exchanged, cudaStream_t stream) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(kRowNormCtas, batch);
    config.blockDim = dim3(((hidden / (4 * kRowNormCtas)) + 31) / 32 * 32);
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[0].val.programmaticStreamSerializationAllowed = 1;
    attributes[1].id = cudaLaunchAttributeClusterDimension;
    attributes[1].val.clusterDim.x = kRowNormCtas;
    attributes[1].val.clusterDim.y = 1;
    attributes[1].val.clusterDim.z = 1;
    config.attrs = attributes;
    config.numAttrs = 2;
    return cudaLaunchKernelEx(&config, rmsnorm_row_cluster_kernel<kExchanged>, partial_sums, splits, scale,
                              static_cast<__nv_bfloat16*>(projection), static_cast<__nv_bfloat16*>(residual),
                              static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(output),
                              static_cast<__half*>(staged), batch <= 16 ? 16 : 32, hidden, batch, epsilon, exchanged);
}

bool row_norm_fits(int hidden) { return hidden % 256 == 0 && hidden <= 8192; }

// fp32 slices -> the projection's bf16 rows, for consumers that read rows: four outputs per thread.
template <bool kExchanged>
__global__ void __launch_bounds__(kThreads) sum_slices_kernel(const SplitSource source, __nv_bfloat16* __restrict__ rows) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t tag = split_tag(source);
    const size_t quads = static_cast<size_t>(source.batch) * source.width / 4;
    const size_t stride = static_cast<size_t>(source.batch) * source.width;
    for (size_t quad = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; quad < quads;
         quad += static_cast<size_t>(gridDim.x) * kThreads) {
        float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (kExchanged) {
            total = tagged_sum4(source.tagged, tag, static_cast<int>(4 * quad));
        }
        for (int first = 0; !kExchanged && first < source.slices; first += 4) {
            float4 part[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                part[j] = __ldcg(reinterpret_cast<const float4*>(source.sums + min(first + j, source.slices - 1) * stride +
                                                                 4 * quad));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool keep = first + j < source.slices;
                total.x += keep ? part[j].x : 0.0f;
                total.y += keep ? part[j].y : 0.0f;
                total.z += keep ? part[j].z : 0.0f;
                total.w += keep ? part[j].w : 0.0f;
            }
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(total.x * source.scale, total.y * source.scale);
        __nv_bfloat162 hi = __floats2bfloat162_rn(total.z * source.scale, total.w * source.scale);
        *reinterpret_cast<uint2*>(rows + 4 * quad) =
            make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
}

// ---- latency mode: the SwiGLU pair finished on the consumer side ----------------------
// The gate and up projections of a rank's columns ran as one K-split launch whose slices every rank
// received ([slice][gate | up] tagged words); this sums them and applies the epilogue of the fused
// one-GPU kernel (gate and up scaled in fp32, silu(gate) * up rounded once to bf16,
// cuda/nvfp4.cu:292-318), two outputs per thread, into the staged operand of the down projection.
__global__ void __launch_bounds__(kThreads) swiglu_combine_kernel(const TaggedRow row, float gate_scale, float up_scale,
                                                                  __nv_bfloat16* __restrict__ output,
                                                                  __half* __restrict__ staged, int intermediate) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t tag = exchange_tag(row.epoch, row.instance);
    // two outputs per thread: their gate and up words of every slice are one batch of 16-byte loads
    const int pair = blockIdx.x * kThreads + threadIdx.x;
    if (2 * pair >= intermediate) {
        return;
    }
    const uint2* gate_at = row.words + 2 * pair;
    const uint2* up_at = row.words + intermediate + 2 * pair;
    float gate[2] = {0.0f, 0.0f}, up[2] = {0.0f, 0.0f};
    for (int first = 0; first < row.slices; first += 8) {
        uint4 g[8], u[8];
        for (int attempt = 0;; ++attempt) {
            bool complete = true;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const size_t slice = static_cast<size_t>(min(first + j, row.slices - 1)) * row.width;
                g[j] = load_tagged_pair(gate_at + slice);
                u[j] = load_tagged_pair(up_at + slice);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                complete = complete &&
                           (((g[j].y ^ tag) | (g[j].w ^ tag) | (u[j].y ^ tag) | (u[j].w ^ tag)) & row.tag_mask) == 0;
            }
            if (complete || !keep_retrying(attempt, row.status)) {
                break;
            }
            __nanosleep(100);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (first + j < row.slices) {
                const size_t slice = static_cast<size_t>(first + j) * row.width;
                const auto take = [&](uint32_t bits, uint32_t word_tag, const uint2* at) {
                    return ((word_tag ^ tag) & row.tag_mask) == 0 ? __uint_as_float(bits)
                                                                  : await_tagged(at, tag, row.status, row.wait_profile);
                };
                gate[0] += take(g[j].x, g[j].y, gate_at + slice);
                gate[1] += take(g[j].z, g[j].w, gate_at + slice + 1);
                up[0] += take(u[j].x, u[j].y, up_at + slice);
                up[1] += take(u[j].z, u[j].w, up_at + slice + 1);
            }
        }
    }
    __nv_bfloat16 rounded[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float gated = gate[i] * gate_scale;
        rounded[i] = __float2bfloat16(__fdividef(gated, 1.0f + __expf(-gated)) * (up[i] * up_scale));
    }
    __nv_bfloat162 both = __halves2bfloat162(rounded[0], rounded[1]);
    const uint32_t out = *reinterpret_cast<uint32_t*>(&both);
    if (output != nullptr) {
        *reinterpret_cast<uint32_t*>(output + 2 * pair) = out;
    }
    if (staged != nullptr) {  // one row of [intermediate / 8][16][8]
        *reinterpret_cast<uint32_t*>(staged + static_cast<size_t>(pair >> 2) * 16 * 8 + (pair & 3) * 2) =
            bf16x2_to_f16x2(out);
    }
}

// The first kernel of a latency-mode step: a new epoch, hence new tags for every exchange of the step.
__global__ void exchange_advance_kernel(uint32_t* epoch) {
    pdl_launch_dependents();
    pdl_wait();
    *epoch = *epoch + 1u;
}

// ---- DeltaNet prepare (cuda/delta_prepare.cu:44-86,168-245), one launch -------------
// One CTA per (key head, row): 128 threads = the 128 dims of the head.  The CTA updates
// the conv history of its q and k channels and of the value heads that share this key
// head, applies SiLU, L2-normalises q and k, and writes k.q, alpha and beta.
__device__ __forceinline__ float softplusf_ref(float value) {
    if (value > 20.0f) {
        return value;
    }
    if (value < -20.0f) {
        return __expf(value);
    }
    return log1pf(__expf(value));
}

// One channel of the causal conv: the operands are fetched by load_* (all channels of a thread
// first, so that their latencies overlap), then finished here.
struct ConvOperands {
    float history[3];
    float current;
    uint2 weight;  // four bf16 taps
};

__device__ __forceinline__ float conv_finish(const ConvOperands& in, float* __restrict__ history) {
    const float w0 = __uint_as_float(in.weight.x << 16);
    const float w1 = __uint_as_float(in.weight.x & 0xffff0000u);
    const float w2 = __uint_as_float(in.weight.y << 16);
    const float w3 = __uint_as_float(in.weight.y & 0xffff0000u);
    float convolved = w0 * in.history[0];
    convolved = fmaf(w1, in.history[1], convolved);
    convolved = fmaf(w2, in.history[2], convolved);
    convolved = fmaf(w3, in.current, convolved);
    history[0] = in.history[1];
    history[1] = in.history[2];
    history[2] = in.current;
    return __bfloat162float(__float2bfloat16(convolved * sigmoidf_fast(convolved)));
}

constexpr int kMaxValueRatio = 3;  // value heads per key head: 32 / 16 or 48 / 16

template <bool kExchanged>  // the split source is an exchanged row of tagged words (latency mode)
__global__ void __launch_bounds__(kDeltaHeadDim) delta_prepare_kernel(
    const __nv_bfloat16* __restrict__ mixed_qkv, const __nv_bfloat16* __restrict__ a_projection,
    const __nv_bfloat16* __restrict__ b_projection, const __nv_bfloat16* __restrict__ conv_weight,
    const __nv_bfloat16* __restrict__ a_log, const __nv_bfloat16* __restrict__ dt_bias,
    float* __restrict__ conv_state, const uint32_t* __restrict__ state_slots, float* __restrict__ query,
    float* __restrict__ key, float* __restrict__ value, float* __restrict__ alpha, float* __restrict__ beta,
    float* __restrict__ kq, int mixed_stride, int gate_stride, int v_heads, int state_capacity, int* status,
    const SplitSource split, int a_column, int b_column, bool early) {
    pdl_launch_dependents();
    __shared__ float scratch[kDeltaHeadDim / 32];
    const int head = blockIdx.x;
    const int batch = blockIdx.y;
    const int dimension = threadIdx.x;
    const int ratio = v_heads / kDeltaKeyHeads;
    const int qk_elements = kDeltaKeyHeads * kDeltaHeadDim;
    const int channels = 2 * qk_elements + v_heads * kDeltaHeadDim;

    // This thread's channels: q, k and one per value head that shares the key head.
    int channel[2 + kMaxValueRatio];
    channel[0] = head * kDeltaHeadDim + dimension;
    channel[1] = qk_elements + head * kDeltaHeadDim + dimension;
#pragma unroll
    for (int r = 0; r < kMaxValueRatio; ++r) {
        channel[2 + r] = 2 * qk_elements + (head * ratio + r) * kDeltaHeadDim + dimension;
    }
    // Conv taps and the gate constants are never written during a step: fetched before the wait.
    ConvOperands operands[2 + kMaxValueRatio];
#pragma unroll
    for (int i = 0; i < 2 + kMaxValueRatio; ++i) {
        if (i < 2 + ratio) {
            operands[i].weight = *reinterpret_cast<const uint2*>(conv_weight + static_cast<size_t>(channel[i]) * 4);
        }
    }
    float log_a = 0.0f, bias = 0.0f;
    if (dimension < ratio) {
        log_a = __bfloat162float(a_log[head * ratio + dimension]);
        bias = __bfloat162float(dt_bias[head * ratio + dimension]);
    }
    // `early` (the step's own form): the rows' slots were fixed when the step was packed and a layer's conv
    // history is written by nobody but this kernel, so both are fetched while the in-projection still runs.
    if (!early) {
        pdl_wait();
    }
    const uint32_t slot = state_slots[batch];
    if (slot >= static_cast<uint32_t>(state_capacity)) {
        // a slot beyond the pool: the row's conv history is neither read nor written; the host
        // learns of it through the status word (uniform over the CTA: the slot is per row)
        if (threadIdx.x == 0) {
            atomicCAS(status, 0, kStatusStateSlotRange);
        }
        return;
    }
    const size_t slot_base = static_cast<size_t>(slot) * channels;
    const __nv_bfloat16* mixed_row = mixed_qkv + static_cast<size_t>(batch) * mixed_stride;
    // every load of the step's data is issued before the first use
#pragma unroll
    for (int i = 0; i < 2 + kMaxValueRatio; ++i) {
        if (i < 2 + ratio) {
            const float* history = conv_state + (slot_base + channel[i]) * 3;
            operands[i].history[0] = history[0];
            operands[i].history[1] = history[1];
            operands[i].history[2] = history[2];
        }
    }
    if (early) {
        pdl_wait();  // the in-projection's outputs
    }
    const uint32_t tag = split_tag(split);
    float projected_a = 0.0f, projected_b = 0.0f;
    if (kExchanged) {
        // latency mode: every word this thread needs is asked for at once (channels, a and b; a thread
        // without an a / b of its own asks for column 0 and drops it)
        constexpr int kValues = 2 + kMaxValueRatio + 2;
        int columns[kValues];
        float sums[kValues];
#pragma unroll
        for (int i = 0; i < 2 + kMaxValueRatio; ++i) {
            columns[i] = i < 2 + ratio ? channel[i] : 0;
        }
        columns[kValues - 2] = dimension < ratio ? a_column + head * ratio + dimension : 0;
        columns[kValues - 1] = dimension < ratio ? b_column + head * ratio + dimension : 0;
        tagged_sums<kValues>(split.tagged, tag, columns, sums);
#pragma unroll
        for (int i = 0; i < 2 + kMaxValueRatio; ++i) {
            operands[i].current = __bfloat162float(__float2bfloat16(sums[i] * split.scale));
        }
        projected_a = __bfloat162float(__float2bfloat16(sums[kValues - 2] * split.scale));
        projected_b = __bfloat162float(__float2bfloat16(sums[kValues - 1] * split.scale));
    }
#pragma unroll
    for (int i = 0; i < 2 + kMaxValueRatio; ++i) {
        if (i < 2 + ratio && !kExchanged) {
            operands[i].current = split.sums != nullptr ? split_value<false>(split, tag, batch, channel[i])
                                                    : __bfloat162float(mixed_row[channel[i]]);
        }
    }
    if (dimension < ratio && !kExchanged) {
        const size_t gate_read = static_cast<size_t>(batch) * gate_stride + head * ratio + dimension;
        if (split.sums != nullptr) {
            projected_a = split_value<false>(split, tag, batch, a_column + head * ratio + dimension);
            projected_b = split_value<false>(split, tag, batch, b_column + head * ratio + dimension);
        } else {
            projected_a = __bfloat162float(a_projection[gate_read]);
            projected_b = __bfloat162float(b_projection[gate_read]);
        }
    }

    const float q = conv_finish(operands[0], conv_state + (slot_base + channel[0]) * 3);
    const float k = conv_finish(operands[1], conv_state + (slot_base + channel[1]) * 3);
#pragma unroll
    for (int r = 0; r < kMaxValueRatio; ++r) {
        if (r < ratio) {
            const int value_head = head * ratio + r;
            const float v = conv_finish(operands[2 + r], conv_state + (slot_base + channel[2 + r]) * 3);
            value[(static_cast<size_t>(batch) * v_heads + value_head) * kDeltaHeadDim + dimension] = v;
        }
    }

    const float q_sum = block_sum(q * q, scratch);
    const float k_sum = block_sum(k * k, scratch);
    const float q_inverse = rsqrtf(q_sum + 1e-6f) * (1.0f / sqrtf(128.0f));
    const float k_inverse = rsqrtf(k_sum + 1e-6f);
    const float normalized_q = q * q_inverse;
    const float normalized_k = k * k_inverse;
    const size_t base = (static_cast<size_t>(batch) * kDeltaKeyHeads + head) * kDeltaHeadDim;
    query[base + dimension] = normalized_q;
    key[base + dimension] = normalized_k;
    const float kq_sum = block_sum(normalized_q * normalized_k, scratch);
    if (dimension == 0) {
        kq[static_cast<size_t>(batch) * kDeltaKeyHeads + head] = kq_sum;
    }
    if (dimension < ratio) {
        const int value_head = head * ratio + dimension;
        const size_t gate_offset = static_cast<size_t>(batch) * v_heads + value_head;
        const float log_decay = -__expf(log_a) * softplusf_ref(projected_a + bias);
        alpha[gate_offset] = __expf(log_decay);
        beta[gate_offset] = sigmoidf_fast(projected_b);
    }
}

// ---- gated RMSNorm over value heads (cuda/delta_output.cu:20-64) --------------------
template <bool kExchanged>
__global__ void __launch_bounds__(kDeltaHeadDim) gated_rmsnorm_kernel(const float* __restrict__ input,
                                                                      const __nv_bfloat16* __restrict__ gate,
                                                                      const __nv_bfloat16* __restrict__ weight,
                                                                      __nv_bfloat16* __restrict__ output,
                                                                      __half* __restrict__ staged, int padded_rows,
                                                                      float epsilon, int gate_stride, int heads,
                                                                      const SplitSource split, int gate_column) {
    pdl_launch_dependents();  // the projection that follows may start streaming its weights
    __shared__ float scratch[kDeltaHeadDim / 32];
    const int head = blockIdx.x;
    const int batch = blockIdx.y;
    const int dimension = threadIdx.x;
    const float gain = __bfloat162float(weight[dimension]);  // static: fetched before the wait
    pdl_wait();
    const size_t offset = (static_cast<size_t>(batch) * heads + head) * kDeltaHeadDim + dimension;
    const size_t gate_offset = static_cast<size_t>(batch) * gate_stride + head * kDeltaHeadDim + dimension;
    // issued with the input load, used last
    const float gate_value = has_slices(split) ? split_value<kExchanged>(split, split_tag(split), batch,
                                                             gate_column + head * kDeltaHeadDim + dimension)
                                               : __bfloat162float(gate[gate_offset]);
    const float value = __bfloat162float(__float2bfloat16(input[offset]));
    const float sum = block_sum(value * value, scratch);
    const float inverse = rsqrtf(sum / static_cast<float>(kDeltaHeadDim) + epsilon);
    const __nv_bfloat16 normalized = __float2bfloat16(value * inverse);
    const __nv_bfloat16 weighted = __float2bfloat16(gain * __bfloat162float(normalized));
    const float silu = gate_value / (1.0f + __expf(-gate_value));
    const __nv_bfloat16 result = __float2bfloat16(__bfloat162float(weighted) * silu);
    if (output != nullptr) {
        output[offset] = result;
    }
    if (staged != nullptr) {
        const int feature = head * kDeltaHeadDim + dimension;
        staged[(static_cast<size_t>(feature >> 3) * padded_rows + batch) * 8 + (feature & 7)] =
            __float2half_rn(fminf(fmaxf(__bfloat162float(result), -65504.0f), 65504.0f));
    }
}

// ---- QK-norm + partial RoPE + FP8 page write (cuda/attention_prepare.cu:52-143) -----
// One launch: blockIdx.x < 24 are query heads, the next 4 are KV heads.
__global__ void __launch_bounds__(kHeadDim) prepare_attention_kernel(
    const __nv_bfloat16* __restrict__ query_gate_projection, const __nv_bfloat16* __restrict__ key_projection,
    const __nv_bfloat16* __restrict__ value_projection, const __nv_bfloat16* __restrict__ query_norm_weight,
    const __nv_bfloat16* __restrict__ key_norm_weight, const __nv_bfloat16* __restrict__ cosine,
    const __nv_bfloat16* __restrict__ sine, const uint32_t* __restrict__ physical_blocks,
    const uint32_t* __restrict__ block_offsets, const float* __restrict__ key_scales,
    const float* __restrict__ value_scales, __nv_bfloat16* __restrict__ query, uint8_t* __restrict__ key_cache,
    uint8_t* __restrict__ value_cache, int page_size, int query_stride, int key_stride, int value_stride,
    float epsilon) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[kHeadDim / 32];
    __shared__ __nv_bfloat16 normalized[kHeadDim];
    const int batch = blockIdx.y;
    const int dimension = threadIdx.x;
    const bool is_query = blockIdx.x < kQueryHeads;
    const int head = is_query ? blockIdx.x : blockIdx.x - kQueryHeads;
    const __nv_bfloat16* raw_row =
        is_query ? query_gate_projection + static_cast<size_t>(batch) * query_stride + head * (2 * kHeadDim)
                 : key_projection + static_cast<size_t>(batch) * key_stride + head * kHeadDim;
    const __nv_bfloat16* norm_weight = is_query ? query_norm_weight : key_norm_weight;
    const float raw = __bfloat162float(raw_row[dimension]);
    const float sum = block_sum(raw * raw, scratch);
    const float inverse = rsqrtf(sum / static_cast<float>(kHeadDim) + epsilon);
    normalized[dimension] = __float2bfloat16(raw * inverse * (1.0f + __bfloat162float(norm_weight[dimension])));
    __syncthreads();
    float rotated_value = __bfloat162float(normalized[dimension]);
    if (dimension < kRopeDim) {
        const int half = kRopeDim / 2;
        const int paired = dimension < half ? dimension + half : dimension - half;
        const float rotated = __bfloat162float(normalized[paired]) * (dimension < half ? -1.0f : 1.0f);
        const float c = __bfloat162float(cosine[static_cast<size_t>(batch) * kRopeDim + dimension]);
        const float s = __bfloat162float(sine[static_cast<size_t>(batch) * kRopeDim + dimension]);
        rotated_value = rotated_value * c + rotated * s;
    }
    if (is_query) {
        query[(static_cast<size_t>(batch) * kQueryHeads + head) * kHeadDim + dimension] =
            __float2bfloat16(rotated_value);
        return;
    }
    const size_t cache_base =
        ((static_cast<size_t>(physical_blocks[batch]) * kKvHeads + head) * page_size + block_offsets[batch]) *
        kHeadDim;
    const float k_inverse = key_scales ? 1.0f / key_scales[head] : 1.0f;
    const float v_inverse = value_scales ? 1.0f / value_scales[head] : 1.0f;
    const float v = __bfloat162float(
        value_projection[static_cast<size_t>(batch) * value_stride + head * kHeadDim + dimension]);
    key_cache[cache_base + dimension] = to_fp8(rotated_value * k_inverse);
    value_cache[cache_base + dimension] = to_fp8(v * v_inverse);
}

// ---- greedy argmax over fp32 logits -------------------------------------------------------
// Behind the ABI of cuda/sampling.cu:39-92 (largest logit, ties to the smaller index, NaN never wins,
// UINT32_MAX for a row without a comparable value), in one launch: a cluster of eight CTAs per row,
// each scanning an eighth of the row with 16-byte loads; a candidate is one 64-bit key - the logit's
// bits made monotonic in the high word, the complemented index in the low word - so that "better" is an
// integer maximum; the eight CTA winners meet in the first CTA's shared memory (one cluster barrier).
// The caller's partial arrays of the two-launch form are not needed.
constexpr int kArgmaxCtas = 8;

__device__ __forceinline__ unsigned long long argmax_key(float value, uint32_t index) {
    const uint32_t raw = __float_as_uint(value);
    const uint32_t bits = raw == 0x80000000u ? 0u : raw;  // -0 equals +0: the index decides between them
    const uint32_t ordered = (bits & 0x80000000u) != 0 ? ~bits : bits | 0x80000000u;  // ascending with the value
    return value != value ? 0ull : (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - index);
}

__global__ void __cluster_dims__(kArgmaxCtas, 1, 1) __launch_bounds__(kThreads)
    argmax_cluster_kernel(const float* __restrict__ logits, uint32_t* __restrict__ output, int vocab) {
    pdl_launch_dependents();
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ unsigned long long warp_keys[kThreads / 32];
    __shared__ unsigned long long cta_keys[kArgmaxCtas];
    pdl_wait();
    const int row_index = blockIdx.y;
    const int rank = static_cast<int>(cluster.block_rank());
    const float* row = logits + static_cast<size_t>(row_index) * vocab;
    const int span = ((vocab + kArgmaxCtas - 1) / kArgmaxCtas + 3) & ~3;
    const int begin = rank * span;
    const int end = min(vocab, begin + span);
    unsigned long long best = 0ull;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        for (int column = begin + 4 * threadIdx.x; column < end; column += 4 * kThreads) {
            if (column + 4 <= end) {
                const float4 v = __ldcs(reinterpret_cast<const float4*>(row + column));
                best = max(best, max(max(argmax_key(v.x, column), argmax_key(v.y, column + 1)),
                                     max(argmax_key(v.z, column + 2), argmax_key(v.w, column + 3))));
            } else {
                for (int c = column; c < end; ++c) {
                    best = max(best, argmax_key(row[c], c));
                }
            }
        }
    } else {
        for (int column = begin + threadIdx.x; column < end; column += kThreads) {
            best = max(best, argmax_key(row[column], column));
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        best = max(best, __shfl_xor_sync(0xffffffffu, best, offset));
    }
    if ((threadIdx.x & 31) == 0) {
        warp_keys[threadIdx.x >> 5] = best;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kThreads / 32; ++w) {
            best = max(best, warp_keys[w]);
        }
        *cluster.map_shared_rank(&cta_keys[rank], 0) = best;
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        unsigned long long winner = 0ull;
        for (int r = 0; r < kArgmaxCtas; ++r) {
            winner = max(winner, cta_keys[r]);
        }
        output[row_index] = 0xffffffffu - static_cast<uint32_t>(winner & 0xffffffffull);
    }
}

constexpr int kMaxLogitsRows = 32;

}  // namespace
}  // namespace qwc

using namespace qwc;

extern "C" int qwc_fp8_quantize_rows(const void* input, void* output, void* row_scales, int rows, int cols,
                                     int first_row, cudaStream_t stream) {
    if (input == nullptr || output == nullptr || row_scales == nullptr || rows <= 0 || cols <= 0 || first_row < 0) {
        return cudaErrorInvalidValue;
    }
    const bool vector = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(input) & 15) == 0 &&
                        (reinterpret_cast<uintptr_t>(output) & 7) == 0;
    if (vector) {
        quantize_rows_kernel<<<(rows + kThreads / 32 - 1) / (kThreads / 32), kThreads, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(input), static_cast<uint8_t*>(output), static_cast<float*>(row_scales),
            rows, cols, first_row);
    } else {
        quantize_rows_scalar_kernel<<<rows, kThreads, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(input), static_cast<uint8_t*>(output), static_cast<float*>(row_scales),
            cols, first_row);
    }
    return cudaGetLastError();
}

extern "C" int qwc_fp8_embedding_gather(const void* table, const void* row_scales, const void* token_ids,
                                        void* output, int batch, int cols, int vocab, cudaStream_t stream) {
    if (table == nullptr || row_scales == nullptr || token_ids == nullptr || output == nullptr || batch <= 0 ||
        cols <= 0 || vocab <= 0) {
        return cudaErrorInvalidValue;
    }
    return qwc::launch_chained(embedding_gather_kernel, dim3(batch), dim3(kThreads), 0, stream, 
        static_cast<const uint8_t*>(table), static_cast<const float*>(row_scales),
        static_cast<const uint32_t*>(token_ids), static_cast<__nv_bfloat16*>(output), cols, vocab);
}

extern "C" int qwc_rmsnorm_bf16_staged(const void* input, void* residual, const void* weight, void* output,
                                       void* staged_output, int batch, int hidden, float epsilon,
                                       cudaStream_t stream) {
    if (input == nullptr || weight == nullptr || (output == nullptr && staged_output == nullptr) || batch <= 0 ||
        batch > kMaxStepRows || (staged_output != nullptr && batch > 32) || hidden <= 0 || hidden % 256 != 0 ||
        hidden > 8 * kThreads * kNormMaxPerThread || !isfinite(epsilon) || epsilon <= 0.0f) {
        return cudaErrorInvalidValue;
    }
    return qwc::launch_chained(rmsnorm_bf16_kernel, dim3(batch), dim3(kThreads), 0, stream,
        static_cast<const __nv_bfloat16*>(input), static_cast<__nv_bfloat16*>(residual),
        static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(output),
        static_cast<__half*>(staged_output), batch <= 16 ? 16 : 32, hidden, epsilon);
}

extern "C" int qwc_rmsnorm_bf16_split_staged(const float* partial_sums, int splits, float weight_global_scale,
                                             void* projection_output, void* residual, const void* weight,
                                             void* output, void* staged_output, int batch, int hidden,
                                             float epsilon, cudaStream_t stream) {
    if (partial_sums == nullptr || splits <= 0 || splits > 64 || !(weight_global_scale > 0.0f) || weight == nullptr ||
        (output == nullptr && staged_output == nullptr) || batch <= 0 || batch > 32 || hidden <= 0 ||
        hidden % 256 != 0 || hidden > 4 * kSplitNormThreads * kSplitNormMaxItems || !isfinite(epsilon) ||
        epsilon <= 0.0f || (reinterpret_cast<uintptr_t>(partial_sums) & 15) != 0) {
        return cudaErrorInvalidValue;
    }
    if (batch == 1 && row_norm_fits(hidden)) {  // one row: spread over a cluster (several rows fill the SMs as they are)
        return launch_row_norm<false>(partial_sums, splits, 1.0f / weight_global_scale, projection_output, residual,
                                      weight, output, staged_output, batch, hidden, epsilon, TaggedRow{}, stream);
    }
    return qwc::launch_chained(rmsnorm_split_kernel<false>, dim3(batch), dim3(kSplitNormThreads), 0, stream, partial_sums,
                               splits, 1.0f / weight_global_scale, static_cast<__nv_bfloat16*>(projection_output),
                               static_cast<__nv_bfloat16*>(residual),
                               static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(output),
                               static_cast<__half*>(staged_output), batch <= 16 ? 16 : 32, hidden, batch, epsilon,
                               TaggedRow{});
}

extern "C" int qwc_rmsnorm_bf16(const void* input, void* residual, const void* weight, void* output, int batch,
                                int hidden, float epsilon, cudaStream_t stream) {
    if (output == nullptr) {
        return cudaErrorInvalidValue;
    }
    return qwc_rmsnorm_bf16_staged(input, residual, weight, output, nullptr, batch, hidden, epsilon, stream);
}

namespace {
int launch_delta_prepare(const void* mixed_qkv, const void* a_projection, const void* b_projection,
                         const void* conv_weight, const void* a_log, const void* dt_bias, void* conv_state,
                         const void* state_slots, void* query, void* key, void* value, void* alpha, void* beta,
                         void* kq, int state_capacity, int batch, int mixed_stride, int gate_stride,
                         const qwc::SplitSource& split, int a_column, int b_column, bool early, cudaStream_t stream);
}

extern "C" int qwc_delta_prepare_decode(const void* mixed_qkv, const void* a_projection, const void* b_projection,
                                        const void* conv_weight, const void* a_log, const void* dt_bias,
                                        void* conv_state, const void* state_slots, void* query, void* key,
                                        void* value, void* alpha, void* beta, void* kq, int state_capacity,
                                        int batch, int mixed_stride, int gate_stride, cudaStream_t stream) {
    if (mixed_qkv == nullptr || a_projection == nullptr || b_projection == nullptr) {
        return cudaErrorInvalidValue;
    }
    return launch_delta_prepare(mixed_qkv, a_projection, b_projection, conv_weight, a_log, dt_bias, conv_state,
                                state_slots, query, key, value, alpha, beta, kq, state_capacity, batch, mixed_stride,
                                gate_stride, qwc::SplitSource{}, 0, 0, false, stream);
}

// The same on a mixer in-projection that ran as a regular K split: fp32 slices
// [slices][batch][width] instead of bf16 rows; a and b are columns of the same rows.  This is the
// step's own form: it reads state_slots and conv_state before it waits for the preceding kernel, so
// neither may be written by the kernels that run just before it on the stream (in a decode step the
// slots are packed at the start and a layer's conv history belongs to this kernel).
extern "C" int qwc_delta_prepare_decode_split(const float* partial_sums, int slices, int width,
                                              float weight_global_scale, int a_column, int b_column,
                                              const void* conv_weight, const void* a_log, const void* dt_bias,
                                              void* conv_state, const void* state_slots, void* query, void* key,
                                              void* value, void* alpha, void* beta, void* kq, int state_capacity,
                                              int batch, cudaStream_t stream) {
    const int v_heads = current_shape().delta_value_heads;
    const int channels = 2 * kDeltaKeyHeads * kDeltaHeadDim + v_heads * kDeltaHeadDim;
    if (partial_sums == nullptr || slices <= 0 || slices > 64 || width < channels || a_column < channels ||
        b_column < channels || a_column + v_heads > width || b_column + v_heads > width ||
        !(weight_global_scale > 0.0f)) {
        return cudaErrorInvalidValue;
    }
    const qwc::SplitSource split = {partial_sums, slices, batch, width, 1.0f / weight_global_scale};
    return launch_delta_prepare(partial_sums, partial_sums, partial_sums, conv_weight, a_log, dt_bias, conv_state,
                                state_slots, query, key, value, alpha, beta, kq, state_capacity, batch, width, width,
                                split, a_column, b_column, true, stream);
}

namespace {
int launch_delta_prepare(const void* mixed_qkv, const void* a_projection, const void* b_projection,
                         const void* conv_weight, const void* a_log, const void* dt_bias, void* conv_state,
                         const void* state_slots, void* query, void* key, void* value, void* alpha, void* beta,
                         void* kq, int state_capacity, int batch, int mixed_stride, int gate_stride,
                         const qwc::SplitSource& split, int a_column, int b_column, bool early, cudaStream_t stream) {
    const int v_heads = current_shape().delta_value_heads;
    const int channels = 2 * kDeltaKeyHeads * kDeltaHeadDim + v_heads * kDeltaHeadDim;
    if (mixed_qkv == nullptr || a_projection == nullptr || b_projection == nullptr || conv_weight == nullptr ||
        a_log == nullptr || dt_bias == nullptr || conv_state == nullptr || state_slots == nullptr ||
        query == nullptr || key == nullptr || value == nullptr || alpha == nullptr || beta == nullptr ||
        kq == nullptr || state_capacity < batch || batch <= 0 || batch > kMaxDecodeBatch ||
        mixed_stride < channels || gate_stride < v_heads) {
        return cudaErrorInvalidValue;
    }
    int* status = qwc::status_ptr();
    if (status == nullptr) {
        return cudaErrorInvalidValue;
    }
    const dim3 grid(kDeltaKeyHeads, batch);
    return qwc::launch_chained(split.tagged.words != nullptr ? delta_prepare_kernel<true> : delta_prepare_kernel<false>,
                               dim3(grid), dim3(kDeltaHeadDim), 0, stream,
        static_cast<const __nv_bfloat16*>(mixed_qkv), static_cast<const __nv_bfloat16*>(a_projection),
        static_cast<const __nv_bfloat16*>(b_projection), static_cast<const __nv_bfloat16*>(conv_weight),
        static_cast<const __nv_bfloat16*>(a_log), static_cast<const __nv_bfloat16*>(dt_bias),
        static_cast<float*>(conv_state), static_cast<const uint32_t*>(state_slots), static_cast<float*>(query),
        static_cast<float*>(key), static_cast<float*>(value), static_cast<float*>(alpha),
        static_cast<float*>(beta), static_cast<float*>(kq), mixed_stride, gate_stride, v_heads, state_capacity,
        status, split, a_column, b_column, early);
}
}  // namespace

extern "C" int qwc_delta_gated_rmsnorm_staged(const float* input, const void* gate, const void* weight, void* output,
                                              void* staged_output, int batch, float epsilon, int gate_stride,
                                              cudaStream_t stream) {
    const int heads = current_shape().delta_value_heads;
    if (input == nullptr || gate == nullptr || weight == nullptr || (output == nullptr && staged_output == nullptr) ||
        batch <= 0 || batch > kMaxStepRows || (staged_output != nullptr && batch > 32) || !isfinite(epsilon) ||
        epsilon <= 0.0f || gate_stride < heads * kDeltaHeadDim) {
        return cudaErrorInvalidValue;
    }
    const dim3 grid(heads, batch);
    return qwc::launch_chained(gated_rmsnorm_kernel<false>, dim3(grid), dim3(kDeltaHeadDim), 0, stream,
        input, static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(weight),
        static_cast<__nv_bfloat16*>(output), static_cast<__half*>(staged_output), batch <= 16 ? 16 : 32, epsilon,
        gate_stride, heads, SplitSource{}, 0);
}

// The same with the gate rows taken from a K-split in-projection (column `gate_column` of its rows).
extern "C" int qwc_delta_gated_rmsnorm_split(const float* input, const float* partial_sums, int slices, int width,
                                             float weight_global_scale, int gate_column, const void* weight,
                                             void* output, void* staged_output, int batch, float epsilon,
                                             cudaStream_t stream) {
    const int heads = current_shape().delta_value_heads;
    if (input == nullptr || partial_sums == nullptr || slices <= 0 || slices > 64 || gate_column < 0 ||
        gate_column + heads * kDeltaHeadDim > width || !(weight_global_scale > 0.0f) || weight == nullptr ||
        (output == nullptr && staged_output == nullptr) || batch <= 0 || batch > 32 || !isfinite(epsilon) ||
        epsilon <= 0.0f) {
        return cudaErrorInvalidValue;
    }
    const SplitSource split = {partial_sums, slices, batch, width, 1.0f / weight_global_scale};
    const dim3 grid(heads, batch);
    return qwc::launch_chained(gated_rmsnorm_kernel<false>, dim3(grid), dim3(kDeltaHeadDim), 0, stream,
        input, static_cast<const __nv_bfloat16*>(nullptr), static_cast<const __nv_bfloat16*>(weight),
        static_cast<__nv_bfloat16*>(output), static_cast<__half*>(staged_output), batch <= 16 ? 16 : 32, epsilon,
        width, heads, split, gate_column);
}

// fp32 slices of a K-split projection -> its bf16 rows [batch][width] (for consumers that read rows).
extern "C" int qwc_nvfp4_sum_slices(const float* partial_sums, int slices, float weight_global_scale, void* rows,
                                    int batch, int width, cudaStream_t stream) {
    if (partial_sums == nullptr || slices <= 0 || slices > 64 || !(weight_global_scale > 0.0f) || rows == nullptr ||
        batch <= 0 || batch > 32 || width <= 0 || width % 4 != 0 ||
        (reinterpret_cast<uintptr_t>(partial_sums) & 15) != 0 || (reinterpret_cast<uintptr_t>(rows) & 7) != 0) {
        return cudaErrorInvalidValue;
    }
    const SplitSource split = {partial_sums, slices, batch, width, 1.0f / weight_global_scale};
    const int blocks = static_cast<int>((static_cast<size_t>(batch) * width / 4 + kThreads - 1) / kThreads);
    return qwc::launch_chained(sum_slices_kernel<false>, dim3(blocks < 592 ? blocks : 592), dim3(kThreads), 0, stream, split,
                               static_cast<__nv_bfloat16*>(rows));
}

// ---- latency mode: consumers of exchanged rows (exchange.cuh) --------------------------
extern "C" int qwc_exchange_advance(void* epoch, cudaStream_t stream) {
    if (epoch == nullptr || (reinterpret_cast<uintptr_t>(epoch) & 3) != 0) {
        return cudaErrorInvalidValue;
    }
    return qwc::launch_chained(exchange_advance_kernel, dim3(1), dim3(1), 0, stream, static_cast<uint32_t*>(epoch));
}

extern "C" size_t qwc_exchange_row_bytes(int width) {
    if (width <= 0 || width % 4 != 0) {
        return 0;
    }
    return static_cast<size_t>(kExchangeMaxSlices) * width * sizeof(uint2);
}

namespace {
bool valid_slices(int slices) { return slices > 0 && slices <= kExchangeMaxSlices; }
}  // namespace

extern "C" int qwc_rmsnorm_bf16_exchanged(const qwc_exchange_row* row, int slices, float weight_global_scale,
                                          void* projection_output, void* residual, const void* weight,
                                          void* output, void* staged_output, int hidden, float epsilon,
                                          cudaStream_t stream) {
    int* status = qwc::status_ptr();
    if (!valid_exchange_row(row) || !valid_slices(slices) || row->width != hidden || !(weight_global_scale > 0.0f) ||
        weight == nullptr || (output == nullptr && staged_output == nullptr) || hidden <= 0 || hidden % 256 != 0 ||
        hidden > 4 * kSplitNormThreads * kSplitNormMaxItems || !isfinite(epsilon) || epsilon <= 0.0f ||
        status == nullptr) {
        return cudaErrorInvalidValue;
    }
    const TaggedRow tagged = tagged_row(*row, slices, status);
    if (row_norm_fits(hidden)) {
        return launch_row_norm<true>(nullptr, slices, 1.0f / weight_global_scale, projection_output, residual, weight,
                                     output, staged_output, 1, hidden, epsilon, tagged, stream);
    }
    return qwc::launch_chained(rmsnorm_split_kernel<true>, dim3(1), dim3(kSplitNormThreads), 0, stream,
                               static_cast<const float*>(nullptr), slices, 1.0f / weight_global_scale,
                               static_cast<__nv_bfloat16*>(projection_output), static_cast<__nv_bfloat16*>(residual),
                               static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(output),
                               static_cast<__half*>(staged_output), 16, hidden, 1, epsilon,
                               tagged);
}

extern "C" int qwc_delta_prepare_decode_exchanged(const qwc_exchange_row* row, int slices, float weight_global_scale,
                                                  int a_column, int b_column, const void* conv_weight,
                                                  const void* a_log, const void* dt_bias, void* conv_state,
                                                  const void* state_slots, void* query, void* key, void* value,
                                                  void* alpha, void* beta, void* kq, int state_capacity,
                                                  cudaStream_t stream) {
    const int v_heads = current_shape().delta_value_heads;
    const int channels = 2 * kDeltaKeyHeads * kDeltaHeadDim + v_heads * kDeltaHeadDim;
    int* status = qwc::status_ptr();
    if (!valid_exchange_row(row) || !valid_slices(slices) || row->width < channels || a_column < channels ||
        b_column < channels || a_column + v_heads > row->width || b_column + v_heads > row->width ||
        !(weight_global_scale > 0.0f) || status == nullptr) {
        return cudaErrorInvalidValue;
    }
    qwc::SplitSource split = {nullptr, slices, 1, row->width, 1.0f / weight_global_scale};
    split.tagged = tagged_row(*row, slices, status);
    return launch_delta_prepare(row, row, row, conv_weight, a_log, dt_bias, conv_state, state_slots, query, key,
                                value, alpha, beta, kq, state_capacity, 1, row->width, row->width, split, a_column,
                                b_column, true, stream);
}

extern "C" int qwc_delta_gated_rmsnorm_exchanged(const float* input, const qwc_exchange_row* row, int slices,
                                                 float weight_global_scale, int gate_column, const void* weight,
                                                 void* output, void* staged_output, float epsilon,
                                                 cudaStream_t stream) {
    const int heads = current_shape().delta_value_heads;
    int* status = qwc::status_ptr();
    if (input == nullptr || !valid_exchange_row(row) || !valid_slices(slices) || gate_column < 0 ||
        gate_column + heads * kDeltaHeadDim > row->width || !(weight_global_scale > 0.0f) || weight == nullptr ||
        (output == nullptr && staged_output == nullptr) || !isfinite(epsilon) || epsilon <= 0.0f ||
        status == nullptr) {
        return cudaErrorInvalidValue;
    }
    SplitSource split = {nullptr, slices, 1, row->width, 1.0f / weight_global_scale};
    split.tagged = tagged_row(*row, slices, status);
    const dim3 grid(heads, 1);
    return qwc::launch_chained(gated_rmsnorm_kernel<true>, dim3(grid), dim3(kDeltaHeadDim), 0, stream, input,
                               static_cast<const __nv_bfloat16*>(nullptr), static_cast<const __nv_bfloat16*>(weight),
                               static_cast<__nv_bfloat16*>(output), static_cast<__half*>(staged_output), 16, epsilon,
                               row->width, heads, split, gate_column);
}

extern "C" int qwc_nvfp4_sum_exchanged(const qwc_exchange_row* row, int slices, float weight_global_scale,
                                       void* rows, cudaStream_t stream) {
    int* status = qwc::status_ptr();
    if (!valid_exchange_row(row) || !valid_slices(slices) || !(weight_global_scale > 0.0f) || rows == nullptr ||
        (reinterpret_cast<uintptr_t>(rows) & 7) != 0 || status == nullptr) {
        return cudaErrorInvalidValue;
    }
    SplitSource split = {nullptr, slices, 1, row->width, 1.0f / weight_global_scale};
    split.tagged = tagged_row(*row, slices, status);
    const int blocks = (row->width / 4 + kThreads - 1) / kThreads;
    return qwc::launch_chained(sum_slices_kernel<true>, dim3(blocks), dim3(kThreads), 0, stream, split,
                               static_cast<__nv_bfloat16*>(rows));
}

extern "C" int qwc_swiglu_combine_exchanged(const qwc_exchange_row* row, int slices, float gate_global_scale,
                                            float up_global_scale, void* output, void* staged_output,
                                            int intermediate, cudaStream_t stream) {
    int* status = qwc::status_ptr();
    if (!valid_exchange_row(row) || !valid_slices(slices) || intermediate <= 0 || intermediate % 8 != 0 ||
        row->width != 2 * intermediate || !(gate_global_scale > 0.0f) || !(up_global_scale > 0.0f) ||
        (output == nullptr && staged_output == nullptr) || (reinterpret_cast<uintptr_t>(output) & 7) != 0 ||
        (reinterpret_cast<uintptr_t>(staged_output) & 15) != 0 || status == nullptr) {
        return cudaErrorInvalidValue;
    }
    const TaggedRow tagged = tagged_row(*row, slices, status);
    const int blocks = (intermediate / 2 + kThreads - 1) / kThreads;
    return qwc::launch_chained(swiglu_combine_kernel, dim3(blocks), dim3(kThreads), 0, stream, tagged,
                               1.0f / gate_global_scale, 1.0f / up_global_scale,
                               static_cast<__nv_bfloat16*>(output), static_cast<__half*>(staged_output), intermediate);
}

extern "C" int qwc_delta_gated_rmsnorm(const float* input, const void* gate, const void* weight, void* output,
                                       int batch, float epsilon, int gate_stride, cudaStream_t stream) {
    if (output == nullptr) {
        return cudaErrorInvalidValue;
    }
    return qwc_delta_gated_rmsnorm_staged(input, gate, weight, output, nullptr, batch, epsilon, gate_stride, stream);
}

extern "C" int qwc_prepare_attention_decode_fp8_scaled(
    const void* query_gate_projection, const void* key_projection, const void* value_projection,
    const void* query_norm_weight, const void* key_norm_weight, const void* cosine, const void* sine,
    const void* physical_blocks, const void* block_offsets, const float* key_scales, const float* value_scales,
    void* query, void* key_cache, void* value_cache, int batch, int page_size, int query_stride, int key_stride,
    int value_stride, float epsilon, cudaStream_t stream) {
    if (query_gate_projection == nullptr || key_projection == nullptr || value_projection == nullptr ||
        query_norm_weight == nullptr || key_norm_weight == nullptr || cosine == nullptr || sine == nullptr ||
        physical_blocks == nullptr || block_offsets == nullptr || query == nullptr || key_cache == nullptr ||
        value_cache == nullptr || batch <= 0 || batch > kMaxStepRows || !isfinite(epsilon) || epsilon <= 0.0f ||
        (page_size != 16 && page_size != 64) || query_stride < kQueryHeads * 2 * kHeadDim ||
        key_stride < kKvHeads * kHeadDim || value_stride < kKvHeads * kHeadDim) {
        return cudaErrorInvalidValue;
    }
    const dim3 grid(kQueryHeads + kKvHeads, batch);
    return qwc::launch_chained(prepare_attention_kernel, dim3(grid), dim3(kHeadDim), 0, stream, 
        static_cast<const __nv_bfloat16*>(query_gate_projection), static_cast<const __nv_bfloat16*>(key_projection),
        static_cast<const __nv_bfloat16*>(value_projection), static_cast<const __nv_bfloat16*>(query_norm_weight),
        static_cast<const __nv_bfloat16*>(key_norm_weight), static_cast<const __nv_bfloat16*>(cosine),
        static_cast<const __nv_bfloat16*>(sine), static_cast<const uint32_t*>(physical_blocks),
        static_cast<const uint32_t*>(block_offsets), key_scales, value_scales, static_cast<__nv_bfloat16*>(query),
        static_cast<uint8_t*>(key_cache), static_cast<uint8_t*>(value_cache), page_size, query_stride, key_stride,
        value_stride, epsilon);
}

extern "C" int qwc_prepare_attention_decode_fp8(const void* query_gate_projection, const void* key_projection,
                                                const void* value_projection, const void* query_norm_weight,
                                                const void* key_norm_weight, const void* cosine, const void* sine,
                                                const void* physical_blocks, const void* block_offsets, void* query,
                                                void* key_cache, void* value_cache, int batch, float epsilon,
                                                cudaStream_t stream) {
    return qwc_prepare_attention_decode_fp8_scaled(
        query_gate_projection, key_projection, value_projection, query_norm_weight, key_norm_weight, cosine, sine,
        physical_blocks, block_offsets, nullptr, nullptr, query, key_cache, value_cache, batch,
        current_shape().kv_page_size, kQueryHeads * 2 * kHeadDim, kKvHeads * kHeadDim, kKvHeads * kHeadDim, epsilon,
        stream);
}

extern "C" int qwc_fp8_max_logits_batch(void) { return kMaxLogitsRows; }
extern "C" int qwc_fp8_max_batched_logits(void) { return kMaxLogitsRows; }

extern "C" int qwc_fp8_lm_head_batched(const void* weights, const void* row_scales, const void* hidden,
                                       void* logits, int batch, int hidden_size, int vocab, cudaStream_t stream) {
    if (weights == nullptr || row_scales == nullptr || hidden == nullptr || logits == nullptr || batch <= 0 ||
        batch > kMaxLogitsRows || hidden_size <= 0 || hidden_size % 256 != 0 || vocab <= 0) {
        (void)take_next_projection();  // a hint is good for one call, also for one that is refused
        return cudaErrorInvalidValue;
    }
    return launch_fp8_rows(weights, static_cast<const float*>(row_scales), hidden, static_cast<float*>(logits),
                           batch, hidden_size, vocab, stream);
}

extern "C" int qwc_fp8_lm_head(const void* weights, const void* row_scales, const void* hidden, void* logits,
                               int batch, int hidden_size, int vocab, cudaStream_t stream) {
    return qwc_fp8_lm_head_batched(weights, row_scales, hidden, logits, batch, hidden_size, vocab, stream);
}

extern "C" int qwc_argmax(const float* logits, float* partial_values, uint32_t* partial_indices, uint32_t* output,
                          int vocab, int batch, int parts, cudaStream_t stream) {
    // partial_values / partial_indices / parts belong to the two-launch form of the reference's signature:
    // checked as that form would, not used.
    if (logits == nullptr || partial_values == nullptr || partial_indices == nullptr || output == nullptr ||
        vocab <= 0 || batch <= 0 || batch > kMaxDecodeBatch || parts <= 0 || parts > kThreads) {
        return cudaErrorInvalidValue;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(kArgmaxCtas, batch);
    config.blockDim = dim3(kThreads);
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[0].val.programmaticStreamSerializationAllowed = 1;
    attributes[1].id = cudaLaunchAttributeClusterDimension;
    attributes[1].val.clusterDim.x = kArgmaxCtas;
    attributes[1].val.clusterDim.y = 1;
    attributes[1].val.clusterDim.z = 1;
    config.attrs = attributes;
    config.numAttrs = 2;
    return cudaLaunchKernelEx(&config, argmax_cluster_kernel, logits, output, vocab);
}
