// Gated DeltaNet recurrent decode step on int8 state with a per-row fp32 scale.
//
// Replaces crates/qwc-cuda/cuda/delta_net.cu:1220-1237 (qwc_delta_decode_int8) behind the
// same C signature.  Arithmetic per state row (cuda/delta_net.cu:99-119,137-175):
//   s = float(code) * scale;  u = s.k;  w = s.q;  c = beta (v - alpha u)
//   s <- alpha s + c k;  out = alpha w + c (k.q)
//   peak = max|s|; inverse = 127 / peak; code = rint(s * inverse); scale = peak * (1/127)
//
// The op reads and rewrites 16 KiB + 512 B per (slot, value head) and nothing else of
// size, so it is bound by HBM read+write bandwidth.  Layout for sm_100a:
//   * one CTA per (value head, slot, row split); the state tile is brought into shared
//     memory by bulk-async copies (TMA 1-D) in 4 KiB quarters, each signalling its own
//     mbarrier, so the first rows are processed while the rest are in flight, and the
//     requantised tile leaves by one bulk store;
//   * eight lanes share a row (16 codes each: one 16-byte shared-memory access per lane and
//     row), so the three per-row reductions cost three shuffle steps; the lane's 16 elements
//     of k and q stay in registers for all rows of the tile.  That keeps the kernel at 72
//     registers, so seven CTAs are resident per SM (112 KiB of state in flight per SM): the
//     kernel is bound by dependent-instruction latency, and the warps of more resident CTAs
//     are what hides it (four lanes per row, 121 registers and four CTAs per SM ran 9 %
//     slower);
//   * the elementwise fp32 work uses the packed f32x2 pipe, and both int8 <-> fp32
//     conversions are bit tricks on the 2^23 binade (exact, round-to-nearest-even),
//     which keeps the instruction count under what the memory stream allows.
//
// The requantiser rounds exactly as the reference's: multiply by `127 / peak` in fp32,
// round to nearest even, scale = peak * (1/127); a zero row stores codes 0 and scale 0.

#include "common.cuh"

namespace qwc {
namespace {

constexpr int kDim = kDeltaHeadDim;  // 128 x 128 state per head
constexpr int kThreads = 128;
constexpr int kPartRows = 32;        // rows per bulk copy / per CTA iteration
constexpr int kMaxParts = kDim / kPartRows;

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// What the fused output stage needs (the gated RMSNorm of cuda/delta_output.cu:20-64 on this CTA's head,
// staged for the output projection); `staged == nullptr`: no fusion, `out` is written instead.
struct GatedNorm {
    const __nv_bfloat16* weight;  // [128]
    const float* gate_sums;       // the in-projection's K-split slices [slices][batch][width], or null
    const __nv_bfloat16* gate_rows;  // ... or its bf16 rows with `gate_stride` elements per row
    int slices;
    int batch;
    int width;
    int gate_column;  // of z within a row
    float gate_scale;
    float epsilon;
    __half* staged;   // [heads * 128 / 8][padded rows][8]
    int padded_rows;
};

// `kEarly`: the rows' state slots were fixed when the step was packed and a layer's state is written by
// nobody but this kernel, so the slot lookup and the copies of the state tile are issued before the
// wait for the preceding kernel (which produces q, k, v and the gates).  Callers outside a step, who
// may have written slots or state just before on the same stream, get the conservative order.
template <bool kEarly>
__global__ void __launch_bounds__(kThreads, 7) delta_decode_int8_kernel(
    int8_t* __restrict__ state, float* __restrict__ state_scales, const uint32_t* __restrict__ state_slots,
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ alpha, const float* __restrict__ beta, const float* __restrict__ kq,
    float* __restrict__ out, int v_heads, int state_capacity, int* status, const GatedNorm norm) {
    pdl_launch_dependents();
    if (!kEarly) {
        pdl_wait();
    }
    __shared__ __align__(128) uint8_t tile[kDim * kDim];
    __shared__ __align__(16) float row_scale[kDim];
    __shared__ float out_rows[kDim];
    __shared__ __align__(16) float v_rows[kDim];
    __shared__ uint64_t bars[kMaxParts];
    __shared__ int failed;

    if (status_is_set(status)) {
        return;
    }
    const int h = blockIdx.x;
    const int b = blockIdx.y;
    const int rows_here = kDim / gridDim.z;
    const int row_begin = blockIdx.z * rows_here;
    const int slot = state_slots == nullptr ? b : static_cast<int>(state_slots[b]);
    if (static_cast<uint32_t>(slot) >= static_cast<uint32_t>(state_capacity)) {
        // a slot beyond the pool: nothing of this row is read or written, the host learns of it
        // through the status word (the whole CTA takes this branch: the slot is per row)
        if (threadIdx.x == 0) {
            atomicCAS(status, 0, kStatusStateSlotRange);
        }
        return;
    }
    const int hk = h / (v_heads / kDeltaKeyHeads);
    const int parts = (rows_here + kPartRows - 1) / kPartRows;
    const int part_rows = rows_here < kPartRows ? rows_here : kPartRows;

    int8_t* S = state + (static_cast<size_t>(slot) * v_heads + h) * (kDim * kDim) + row_begin * kDim;
    float* scales = state_scales + (static_cast<size_t>(slot) * v_heads + h) * kDim + row_begin;

    if (threadIdx.x == 0) {
        failed = 0;
        for (int part = 0; part < parts; ++part) {
            mbar_init(&bars[part], 1);
        }
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int part = 0; part < parts; ++part) {
            const uint32_t bytes = part_rows * kDim;
            mbar_arrive_expect_tx(&bars[part], bytes + (part == 0 ? rows_here * 4 : 0));
            bulk_g2s(tile + part * kPartRows * kDim, S + part * kPartRows * kDim, bytes, &bars[part]);
            if (part == 0) {
                bulk_g2s(row_scale, scales, rows_here * 4, &bars[0]);
            }
        }
    }
    if (kEarly) {
        pdl_wait();  // q, k, v and the gates come from the preceding kernel
    }
    for (int i = threadIdx.x; i < rows_here; i += kThreads) {
        v_rows[i] = v[(static_cast<size_t>(b) * v_heads + h) * kDim + row_begin + i];
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int sub = lane & 7;        // which eighth of the row this lane owns: columns [16 sub, 16 sub + 16)
    const int row_in_warp = lane >> 3;

    float2 kk[8], qq[8];
    {
        const float* kp = k + (static_cast<size_t>(b) * kDeltaKeyHeads + hk) * kDim + 16 * sub;
        const float* qp = q + (static_cast<size_t>(b) * kDeltaKeyHeads + hk) * kDim + 16 * sub;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 kv = *reinterpret_cast<const float4*>(kp + 4 * i);
            const float4 qv = *reinterpret_cast<const float4*>(qp + 4 * i);
            kk[2 * i] = f2(kv.x, kv.y);
            kk[2 * i + 1] = f2(kv.z, kv.w);
            qq[2 * i] = f2(qv.x, qv.y);
            qq[2 * i + 1] = f2(qv.z, qv.w);
        }
    }
    const float a = alpha[static_cast<size_t>(b) * v_heads + h];
    const float bt = beta[static_cast<size_t>(b) * v_heads + h];
    const float kq_token = kq[static_cast<size_t>(b) * kDeltaKeyHeads + hk];

    constexpr float kMagic = 12582912.0f;        // 1.5 * 2^23
    constexpr float kMagicBiased = 12583040.0f;  // kMagic + 128

    for (int part = 0; part < parts; ++part) {
        // a warp leaves as a whole: the row reductions below are full-warp shuffles
        const bool arrived =
            __all_sync(0xffffffffu, mbar_wait_bounded(&bars[part], 0, kStatusDeltaTileWait, status));
        if (!arrived) {
            failed = 1;
            break;
        }
        if (warp * 8 >= part_rows) {
            continue;  // whole warp beyond the split's rows
        }
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
            const int local = part * kPartRows + warp * 8 + pass * 4 + row_in_warp;
            uint8_t* row_ptr = tile + local * kDim + 16 * sub;
            const uint4 codes = *reinterpret_cast<const uint4*>(row_ptr);
            const float scale = row_scale[local];
            const float v_row = v_rows[local];

            const uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
            float2 s[8];
            const float2 bias = f2(-kMagicBiased, -kMagicBiased);
            const float2 scale2 = f2(scale, scale);
            float2 u2 = f2(0.0f, 0.0f), w2 = f2(0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t x = words[i] ^ 0x80808080u;
                const float2 lo = f2(__uint_as_float(__byte_perm(x, 0x4B400000u, 0x7650)),
                                     __uint_as_float(__byte_perm(x, 0x4B400000u, 0x7651)));
                const float2 hi = f2(__uint_as_float(__byte_perm(x, 0x4B400000u, 0x7652)),
                                     __uint_as_float(__byte_perm(x, 0x4B400000u, 0x7653)));
                s[2 * i] = __fmul2_rn(__fadd2_rn(lo, bias), scale2);
                s[2 * i + 1] = __fmul2_rn(__fadd2_rn(hi, bias), scale2);
                u2 = __ffma2_rn(s[2 * i], kk[2 * i], u2);
                w2 = __ffma2_rn(s[2 * i], qq[2 * i], w2);
                u2 = __ffma2_rn(s[2 * i + 1], kk[2 * i + 1], u2);
                w2 = __ffma2_rn(s[2 * i + 1], qq[2 * i + 1], w2);
            }
            float u = u2.x + u2.y;
            float w = w2.x + w2.y;
#pragma unroll
            for (int offset = 1; offset < 8; offset <<= 1) {
                u += __shfl_xor_sync(0xffffffffu, u, offset);
                w += __shfl_xor_sync(0xffffffffu, w, offset);
            }

            const float c = bt * (v_row - a * u);
            const float contribution = a * w + c * kq_token;

            const float2 a2 = f2(a, a);
            const float2 cc = f2(c, c);
            float peak = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                s[i] = __ffma2_rn(cc, kk[i], __fmul2_rn(a2, s[i]));
                peak = fmaxf(peak, fmaxf(fabsf(s[i].x), fabsf(s[i].y)));
            }
#pragma unroll
            for (int offset = 1; offset < 8; offset <<= 1) {
                peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, offset));
            }

            const float inverse = peak == 0.0f ? 0.0f : __fdiv_rn(127.0f, peak);
            const float2 inverse2 = f2(inverse, inverse);
            const float2 magic2 = f2(kMagic, kMagic);
            uint32_t packed[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 y0 = __fadd2_rn(__fmul2_rn(s[2 * i], inverse2), magic2);
                const float2 y1 = __fadd2_rn(__fmul2_rn(s[2 * i + 1], inverse2), magic2);
                const uint32_t lo = __byte_perm(__float_as_uint(y0.x), __float_as_uint(y0.y), 0x0040);
                const uint32_t hi = __byte_perm(__float_as_uint(y1.x), __float_as_uint(y1.y), 0x0040);
                packed[i] = __byte_perm(lo, hi, 0x5410);
            }
            *reinterpret_cast<uint4*>(row_ptr) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            if (sub == 0) {
                row_scale[local] = __fmul_rn(peak, 1.0f / 127.0f);
                out_rows[local] = contribution;
            }
        }
    }

    fence_proxy_async();
    __syncthreads();
    if (failed) {
        // The copies that were asked for may still be landing in this CTA's shared memory: their
        // thread waits for each of them (bounded) before the CTA gives the memory back.
        if (threadIdx.x == 0) {
            for (int part = 0; part < parts; ++part) {
                mbar_wait_bounded(&bars[part], 0, kStatusDeltaTileWait, status);
            }
        }
        return;
    }
    if (threadIdx.x == 0) {
        bulk_s2g(S, tile, rows_here * kDim);
        bulk_s2g(scales, row_scale, rows_here * 4);
        bulk_commit();
    }
    if (norm.staged != nullptr) {
        // The whole head is here (the launcher fuses only unsplit heads): gated RMSNorm and the staged
        // store, thread = dimension.  Rounding points as cuda/delta_output.cu:38-64.
        __shared__ float warp_sums[kThreads / 32];
        const int dimension = threadIdx.x;
        const int column = norm.gate_column + h * kDim + dimension;
        float gate_value;
        if (norm.gate_sums != nullptr) {
            const size_t stride = static_cast<size_t>(norm.batch) * norm.width;
            const float* at = norm.gate_sums + static_cast<size_t>(b) * norm.width + column;
            float total = 0.0f;
            for (int first = 0; first < norm.slices; first += 4) {
                float part[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    part[j] = __ldcg(at + min(first + j, norm.slices - 1) * stride);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    total += first + j < norm.slices ? part[j] : 0.0f;
                }
            }
            gate_value = __bfloat162float(__float2bfloat16(total * norm.gate_scale));
        } else {
            gate_value = __bfloat162float(norm.gate_rows[static_cast<size_t>(b) * norm.width + column]);
        }
        const float gain = __bfloat162float(norm.weight[dimension]);
        const float value = __bfloat162float(__float2bfloat16(out_rows[dimension]));
        float sum = warp_sum(value * value);
        if ((threadIdx.x & 31) == 0) {
            warp_sums[threadIdx.x >> 5] = sum;
        }
        __syncthreads();
        sum = 0.0f;
        for (int w = 0; w < kThreads / 32; ++w) {
            sum += warp_sums[w];
        }
        const float inverse = rsqrtf(sum / static_cast<float>(kDim) + norm.epsilon);
        const __nv_bfloat16 normalized = __float2bfloat16(value * inverse);
        const __nv_bfloat16 weighted = __float2bfloat16(gain * __bfloat162float(normalized));
        const float silu = gate_value / (1.0f + __expf(-gate_value));
        const __nv_bfloat16 result = __float2bfloat16(__bfloat162float(weighted) * silu);
        const int feature = h * kDim + dimension;
        norm.staged[(static_cast<size_t>(feature >> 3) * norm.padded_rows + b) * 8 + (feature & 7)] =
            __float2half_rn(fminf(fmaxf(__bfloat162float(result), -65504.0f), 65504.0f));
    } else {
        float* op = out + (static_cast<size_t>(b) * v_heads + h) * kDim + row_begin;
        for (int i = threadIdx.x; i < rows_here; i += kThreads) {
            op[i] = out_rows[i];
        }
    }
    if (threadIdx.x == 0) {
        bulk_wait_all_read();
    }
}

// Row splits so that the grid has at least two CTAs per SM
// (same purpose as splits_for, cuda/delta_net.cu:1184-1200).
int splits_for(int batch, int v_heads) {
    int sms = 148;
    int device = 0;
    if (cudaGetDevice(&device) == cudaSuccess) {
        int value = 0;
        if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && value > 0) {
            sms = value;
        }
    }
    const int base = v_heads * batch;
    int split = 1;
    while (split < 16 && base * split < 2 * sms) {
        split *= 2;
    }
    return split;
}

}  // namespace
}  // namespace qwc

extern "C" int qwc_delta_decode_int8(void* state, float* state_scales, const void* state_slots, const void* q,
                                     const void* k, const void* v, const void* alpha, const void* beta,
                                     const void* kq, void* out, int state_capacity, int batch,
                                     cudaStream_t stream) {
    if (state == nullptr || state_scales == nullptr || q == nullptr || k == nullptr || v == nullptr ||
        alpha == nullptr || beta == nullptr || kq == nullptr || out == nullptr || state_capacity < batch ||
        batch <= 0 || batch > qwc::kMaxDecodeBatch) {
        return cudaErrorInvalidValue;
    }
    const int v_heads = qwc::current_shape().delta_value_heads;
    int* status = qwc::status_ptr();
    if (status == nullptr) {
        return cudaErrorInvalidValue;
    }
    const dim3 grid(v_heads, batch, qwc::splits_for(batch, v_heads));
    return qwc::launch_chained(qwc::delta_decode_int8_kernel<false>, dim3(grid), dim3(qwc::kThreads), 0, stream,
        static_cast<int8_t*>(state), state_scales, static_cast<const uint32_t*>(state_slots),
        static_cast<const float*>(q), static_cast<const float*>(k), static_cast<const float*>(v),
        static_cast<const float*>(alpha), static_cast<const float*>(beta), static_cast<const float*>(kq),
        static_cast<float*>(out), v_heads, state_capacity, status, qwc::GatedNorm{});
}

// The step's form of the same update (additive; the decode executor's own): the state slots and the
// state tiles are fetched while the preceding kernel still runs (see kEarly above), and when every head
// is one CTA (qwc_delta_decode_fuses_norm) the gated RMSNorm of qwc_delta_gated_rmsnorm_split /
// _staged runs in the same CTA and the result is stored staged for the output projection; `out` is
// then not written.  gate: either the in-projection's K-split slices (gate_sums, slices, scale) or its
// bf16 rows (gate_rows), `width` elements per row, z at column `gate_column`.
extern "C" int qwc_delta_decode_fuses_norm(int batch) {
    const int v_heads = qwc::current_shape().delta_value_heads;
    return batch > 0 && batch <= 32 && qwc::splits_for(batch, v_heads) == 1 ? 1 : 0;
}

extern "C" int qwc_delta_decode_int8_step(void* state, float* state_scales, const void* state_slots, const void* q,
                                          const void* k, const void* v, const void* alpha, const void* beta,
                                          const void* kq, void* out, int state_capacity, int batch,
                                          const float* gate_sums, int slices, float gate_global_scale,
                                          const void* gate_rows, int width, int gate_column,
                                          const void* norm_weight, float epsilon, void* staged_output,
                                          cudaStream_t stream) {
    if (state == nullptr || state_scales == nullptr || state_slots == nullptr || q == nullptr || k == nullptr ||
        v == nullptr || alpha == nullptr || beta == nullptr || kq == nullptr || out == nullptr ||
        state_capacity < batch || batch <= 0 || batch > qwc::kMaxDecodeBatch) {
        return cudaErrorInvalidValue;
    }
    const int v_heads = qwc::current_shape().delta_value_heads;
    int* status = qwc::status_ptr();
    if (status == nullptr) {
        return cudaErrorInvalidValue;
    }
    const int splits = qwc::splits_for(batch, v_heads);
    qwc::GatedNorm norm = {};
    if (staged_output != nullptr) {
        if (splits != 1 || batch > 32 || norm_weight == nullptr || (gate_sums == nullptr && gate_rows == nullptr) ||
            (gate_sums != nullptr && (slices <= 0 || slices > 64 || !(gate_global_scale > 0.0f))) ||
            gate_column < 0 || gate_column + v_heads * qwc::kDim > width || !isfinite(epsilon) || epsilon <= 0.0f) {
            return cudaErrorInvalidValue;
        }
        norm.weight = static_cast<const __nv_bfloat16*>(norm_weight);
        norm.gate_sums = gate_sums;
        norm.gate_rows = static_cast<const __nv_bfloat16*>(gate_rows);
        norm.slices = slices;
        norm.batch = batch;
        norm.width = width;
        norm.gate_column = gate_column;
        norm.gate_scale = gate_sums != nullptr ? 1.0f / gate_global_scale : 1.0f;
        norm.epsilon = epsilon;
        norm.staged = static_cast<__half*>(staged_output);
        norm.padded_rows = batch <= 16 ? 16 : 32;
    }
    const dim3 grid(v_heads, batch, splits);
    return qwc::launch_chained(qwc::delta_decode_int8_kernel<true>, dim3(grid), dim3(qwc::kThreads), 0, stream,
        static_cast<int8_t*>(state), state_scales, static_cast<const uint32_t*>(state_slots),
        static_cast<const float*>(q), static_cast<const float*>(k), static_cast<const float*>(v),
        static_cast<const float*>(alpha), static_cast<const float*>(beta), static_cast<const float*>(kq),
        static_cast<float*>(out), v_heads, state_capacity, status, norm);
}
