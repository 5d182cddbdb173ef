/*
 * CPU oracle for the decode-step hot path. TEST INFRASTRUCTURE ONLY.
 *
 * Scalar fp32 restatement of the reference's own CPU `reference` modules and of
 * the arithmetic its CUDA launchers define, generalised over the shape
 * parameters the reference bakes in as constants (value heads, page size,
 * vocabulary).  Only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg may link or call this file; nothing in the shipped library
 * depends on it.
 *
 * Parity pin: every function is checked against the reference's known-answer
 * tests (number formats, swizzle probes, the CSR layout example, the int8 grid
 * statement) in tests/test_oracle_golden.py.
 *
 * Built with -O2 -ffp-contract=off so that every fp32 operation rounds once,
 * in source order.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define QO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* Number formats                                                      */
/* ------------------------------------------------------------------ */

/* crates/qwc-cuda/src/bf16.rs:5-12 : round to nearest even, NaN -> 0x7fc0. */
QO_API uint16_t qo_bf16_from_f32(float x) {
    uint32_t bits;
    memcpy(&bits, &x, 4);
    if (x != x) {
        return 0x7fc0;
    }
    const uint32_t lsb = (bits >> 16) & 1u;
    return (uint16_t)((bits + 0x7fffu + lsb) >> 16);
}

/* crates/qwc-cuda/src/bf16.rs:14-16 */
QO_API float qo_bf16_to_f32(uint16_t x) {
    const uint32_t bits = (uint32_t)x << 16;
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

static inline float bf16_round(float x) { return qo_bf16_to_f32(qo_bf16_from_f32(x)); }

/* crates/qwc-cuda/src/nvfp4.rs:574-580 */
static const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

QO_API float qo_e2m1(uint8_t raw) { return kE2M1[raw & 0x0f]; }

/* crates/qwc-cuda/src/nvfp4.rs:583-594 : E4M3 finite, 0x7f / 0xff are NaN. */
QO_API float qo_e4m3(uint8_t raw) {
    const float sign = (raw & 0x80) ? -1.0f : 1.0f;
    const int exponent = (raw >> 3) & 0x0f;
    const int mantissa = raw & 0x07;
    if (exponent == 0) {
        return sign * (float)mantissa * ldexpf(1.0f, -9);
    }
    if (exponent == 0x0f && mantissa == 0x07) {
        return NAN;
    }
    return sign * (1.0f + (float)mantissa / 8.0f) * ldexpf(1.0f, exponent - 7);
}

/*
 * Encode as the CUDA `__nv_fp8_e4m3(float)` constructor does (used by
 * crates/qwc-cuda/cuda/attention_prepare.cu:69-72 and vocab_fp8.cu:33-36):
 * round to nearest even on the E4M3 grid, saturate finite values to +-448,
 * NaN -> 0x7f.
 */
QO_API uint8_t qo_e4m3_encode(float value) {
    if (value != value) {
        return 0x7f;
    }
    const uint8_t sign = signbit(value) ? 0x80 : 0x00;
    float x = fabsf(value);
    if (x >= 448.0f) {
        return sign | 0x7e; /* includes +-inf */
    }
    /* Subnormal grid: multiples of 2^-9 below 2^-6. */
    if (x < ldexpf(1.0f, -6)) {
        const float steps = rintf(x * 512.0f); /* exact scaling, RNE */
        return sign | (uint8_t)steps;         /* 8 -> 0x08 == 2^-6, the first normal */
    }
    int exponent;
    const float fraction = frexpf(x, &exponent); /* x = fraction * 2^exponent, fraction in [0.5,1) */
    /* mantissa steps of 1/8 over [1,2): m = x / 2^(exponent-1) */
    float scaled = fraction * 16.0f;            /* in [8,16) */
    float rounded = rintf(scaled);              /* RNE, may reach 16 */
    int e = exponent - 1;                       /* unbiased exponent */
    if (rounded >= 16.0f) {
        rounded = 8.0f;
        e += 1;
    }
    const int biased = e + 7;
    if (biased > 15 || (biased == 15 && rounded - 8.0f > 6.0f)) {
        return sign | 0x7e;
    }
    return sign | (uint8_t)((biased << 3) | (int)(rounded - 8.0f));
}

/* ------------------------------------------------------------------ */
/* NVFP4 W4A16                                                         */
/* ------------------------------------------------------------------ */

static size_t round_up(size_t value, size_t multiple) {
    return (value + multiple - 1) / multiple * multiple;
}

/* crates/qwc-cuda/src/nvfp4.rs:475-477 */
QO_API size_t qo_block_scale_storage_len(int rows, int in_features) {
    return round_up((size_t)rows, 128) * round_up((size_t)in_features / 16, 4);
}

/* crates/qwc-cuda/src/nvfp4.rs:480-502 and cuda/nvfp4.cu:33-39 */
QO_API size_t qo_block_scale_offset(int row, int group, int in_features) {
    const size_t groups = (size_t)in_features / 16;
    const size_t group_blocks = round_up(groups, 4) / 4;
    const size_t row_block = (size_t)row / 128;
    const size_t row_in_block = (size_t)row % 128;
    const size_t row_quad = row_in_block / 32;
    const size_t row_in_quad = row_in_block % 32;
    const size_t group_block = (size_t)group / 4;
    const size_t group_in_block = (size_t)group % 4;
    return ((((row_block * group_blocks + group_block) * 32 + row_in_quad) * 4 + row_quad) * 4) +
           group_in_block;
}

QO_API void qo_swizzle_block_scales(const uint8_t* scales, uint8_t* out, int rows, int in_features) {
    const int groups = in_features / 16;
    memset(out, 0, qo_block_scale_storage_len(rows, in_features));
    for (int row = 0; row < rows; ++row) {
        for (int group = 0; group < groups; ++group) {
            out[qo_block_scale_offset(row, group, in_features)] = scales[(size_t)row * groups + group];
        }
    }
}

/* crates/qwc-cuda/src/nvfp4.rs:504-522 */
QO_API void qo_unswizzle_block_scales(const uint8_t* swizzled, uint8_t* out, int rows, int in_features) {
    const int groups = in_features / 16;
    for (int row = 0; row < rows; ++row) {
        for (int group = 0; group < groups; ++group) {
            out[(size_t)row * groups + group] = swizzled[qo_block_scale_offset(row, group, in_features)];
        }
    }
}

/*
 * crates/qwc-cuda/src/nvfp4.rs:597-635 (reference::gemv_w4a16).  `scales` is
 * the logical row-major [out, in/16] matrix; low nibble holds the even k.
 * Rows are independent, so the outer loop is parallel; each row keeps the
 * reference's summation order.
 */
QO_API void qo_gemv_w4a16(const uint8_t* packed, const uint8_t* scales, float weight_global_scale,
                          const uint16_t* input, float* output, int out_features, int in_features,
                          int batch) {
    const int groups = in_features / 16;
    float* x = (float*)malloc(sizeof(float) * (size_t)batch * in_features);
    for (size_t i = 0; i < (size_t)batch * in_features; ++i) {
        x[i] = qo_bf16_to_f32(input[i]);
    }
#pragma omp parallel for schedule(static)
    for (int row = 0; row < out_features; ++row) {
        for (int b = 0; b < batch; ++b) {
            float acc = 0.0f;
            for (int group = 0; group < groups; ++group) {
                const float scale = qo_e4m3(scales[(size_t)row * groups + group]) / weight_global_scale;
                float partial = 0.0f;
                for (int j = 0; j < 16; ++j) {
                    const int k = group * 16 + j;
                    const uint8_t byte = packed[(size_t)row * (in_features / 2) + k / 2];
                    const uint8_t nibble = (k & 1) == 0 ? (byte & 0x0f) : (byte >> 4);
                    partial += kE2M1[nibble] * x[(size_t)b * in_features + k];
                }
                acc += partial * scale;
            }
            output[(size_t)b * out_features + row] = acc;
        }
    }
    free(x);
}

/*
 * Fused SwiGLU as the reference test states it
 * (crates/qwc-cuda/tests/nvfp4.rs:87-89): silu(gate) * up on the fp32 sums.
 */
QO_API void qo_swiglu_combine(const float* gate, const float* up, float* output, size_t count) {
    for (size_t i = 0; i < count; ++i) {
        output[i] = gate[i] / (1.0f + expf(-gate[i])) * up[i];
    }
}

/* ------------------------------------------------------------------ */
/* Packed paged FP8 attention                                          */
/* ------------------------------------------------------------------ */

/*
 * crates/qwc-cuda/src/paged_attention.rs:783-831 (reference::decode_fp8),
 * token-sequential online softmax in fp32.  Generalised: page size, head
 * counts, optional per-kv-head dequantisation scales (1.0 reproduces the
 * reference, whose cache is unscaled: cuda/paged_attention.cu:34-38) and the
 * optional sigmoid output gate read from the second half of each head of the
 * [q;gate] projection (cuda/paged_attention.cu:92-106,
 * tests/paged_attention.rs:880-885).
 */
QO_API void qo_paged_attention_fp8(const uint16_t* query, const uint16_t* query_gate_projection,
                                   const uint8_t* key_cache, const uint8_t* value_cache,
                                   const uint32_t* block_tables, const uint32_t* context_lengths,
                                   int max_blocks, float* output, int batch, int q_heads,
                                   int kv_heads, int head_dim, int page_size, const float* k_scale,
                                   const float* v_scale, float softmax_scale) {
    const int group = q_heads / kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < batch; ++b) {
        for (int query_head = 0; query_head < q_heads; ++query_head) {
            const int context = (int)context_lengths[b];
            const int kv_head = query_head / group;
            const size_t query_base = ((size_t)b * q_heads + query_head) * head_dim;
            const float ks = k_scale ? k_scale[kv_head] : 1.0f;
            const float vs = v_scale ? v_scale[kv_head] : 1.0f;
            float maximum = -INFINITY;
            float denominator = 0.0f;
            float* accumulator = (float*)calloc((size_t)head_dim, sizeof(float));
            for (int token = 0; token < context; ++token) {
                const uint32_t physical = block_tables[(size_t)b * max_blocks + token / page_size];
                const size_t cache_base =
                    (((size_t)physical * kv_heads + kv_head) * page_size + token % page_size) *
                    head_dim;
                float score = 0.0f;
                for (int d = 0; d < head_dim; ++d) {
                    score += qo_bf16_to_f32(query[query_base + d]) * (qo_e4m3(key_cache[cache_base + d]) * ks);
                }
                score *= softmax_scale;
                const float next_maximum = fmaxf(maximum, score);
                const float old_weight = expf(maximum - next_maximum);
                const float token_weight = expf(score - next_maximum);
                denominator = denominator * old_weight + token_weight;
                for (int d = 0; d < head_dim; ++d) {
                    accumulator[d] = accumulator[d] * old_weight +
                                     token_weight * (qo_e4m3(value_cache[cache_base + d]) * vs);
                }
                maximum = next_maximum;
            }
            for (int d = 0; d < head_dim; ++d) {
                float value = accumulator[d] / denominator;
                if (query_gate_projection != NULL) {
                    const size_t gate_offset =
                        ((size_t)b * q_heads + query_head) * (2 * (size_t)head_dim) + head_dim + d;
                    const float gate = qo_bf16_to_f32(query_gate_projection[gate_offset]);
                    value *= 1.0f / (1.0f + expf(-gate));
                }
                output[query_base + d] = value;
            }
            free(accumulator);
        }
    }
}

/* ------------------------------------------------------------------ */
/* Gated DeltaNet, int8 state                                          */
/* ------------------------------------------------------------------ */

/*
 * One state row -> int8 codes + scale, operation by operation as
 * crates/qwc-cuda/cuda/delta_net.cu:149-175 (state_store_int8):
 * peak = max|s|; zero row -> codes 0, scale 0; inverse = 127/peak;
 * code = clamp(rintf(s*inverse), +-127); scale = peak * (1/127).
 */
QO_API float qo_delta_quantize_row(const float* row, int8_t* codes, int width) {
    float peak = 0.0f;
    for (int j = 0; j < width; ++j) {
        peak = fmaxf(peak, fabsf(row[j]));
    }
    if (peak == 0.0f) {
        memset(codes, 0, (size_t)width);
    } else {
        const float inverse = 127.0f / peak;
        for (int j = 0; j < width; ++j) {
            codes[j] = (int8_t)(int)fminf(fmaxf(rintf(row[j] * inverse), -127.0f), 127.0f);
        }
    }
    return peak * (1.0f / 127.0f);
}

/*
 * Recurrence of crates/qwc-cuda/src/delta_net.rs:815-861 (reference::decode)
 * on the int8 storage of cuda/delta_net.cu:137-147,177-256: dequantise
 * `(float)code * scale`, u = S k, w = S q, c = beta (v - alpha u),
 * S <- alpha S + c k, out = alpha w + c (k.q), requantise the row.
 * `kq` is an input, as for the kernel (cuda/delta_prepare.cu:214-226 computes it).
 * `state_slots == NULL` means slot b (cuda/delta_net.cu:191).
 * v-head h reads k/q head h / (v_heads / k_heads) (cuda/delta_net.cu:192).
 */
QO_API void qo_delta_decode_int8(int8_t* state, float* state_scales, const uint32_t* state_slots,
                                 const float* q, const float* k, const float* v,
                                 const float* alpha, const float* beta, const float* kq, float* out,
                                 int batch, int v_heads, int k_heads, int dv, int dk) {
    const int ratio = v_heads / k_heads;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
        for (int h = 0; h < v_heads; ++h) {
            const int slot = state_slots ? (int)state_slots[b] : b;
            const int hk = h / ratio;
            const float* kv = k + ((size_t)b * k_heads + hk) * dk;
            const float* qv = q + ((size_t)b * k_heads + hk) * dk;
            const float a = alpha[(size_t)b * v_heads + h];
            const float bt = beta[(size_t)b * v_heads + h];
            const float kq_token = kq[(size_t)b * k_heads + hk];
            int8_t* S = state + ((size_t)slot * v_heads + h) * dv * dk;
            float* scales = state_scales + ((size_t)slot * v_heads + h) * dv;
            float row_values[1024];
            for (int row = 0; row < dv; ++row) {
                int8_t* sr = S + (size_t)row * dk;
                const float scale = scales[row];
                float u = 0.0f, w = 0.0f;
                for (int j = 0; j < dk; ++j) {
                    const float x = (float)sr[j] * scale;
                    row_values[j] = x;
                    u += x * kv[j];
                    w += x * qv[j];
                }
                const float c = bt * (v[((size_t)b * v_heads + h) * dv + row] - a * u);
                out[((size_t)b * v_heads + h) * dv + row] = a * w + c * kq_token;
                for (int j = 0; j < dk; ++j) {
                    row_values[j] = a * row_values[j] + c * kv[j];
                }
                scales[row] = qo_delta_quantize_row(row_values, sr, dk);
            }
        }
    }
}

/* ------------------------------------------------------------------ */
/* Step glue                                                           */
/* ------------------------------------------------------------------ */

/*
 * crates/qwc-cuda/src/rmsnorm.rs:99-140 with the bf16 output rounding of
 * cuda/rmsnorm.cu:143-148.  residual (nullable) is updated in place with
 * bf16(input + residual) and the statistics use the rounded value.
 */
QO_API void qo_rmsnorm_bf16(const uint16_t* input, uint16_t* residual, const uint16_t* weight,
                            uint16_t* output, int batch, int hidden, float epsilon) {
    float* staged = (float*)malloc(sizeof(float) * (size_t)hidden);
    for (int row = 0; row < batch; ++row) {
        const size_t base = (size_t)row * hidden;
        float sum = 0.0f;
        for (int column = 0; column < hidden; ++column) {
            float value = qo_bf16_to_f32(input[base + column]);
            if (residual != NULL) {
                value += qo_bf16_to_f32(residual[base + column]);
                residual[base + column] = qo_bf16_from_f32(value);
                value = qo_bf16_to_f32(residual[base + column]);
            }
            staged[column] = value;
            sum += value * value;
        }
        const float inverse = 1.0f / sqrtf(sum / (float)hidden + epsilon);
        for (int column = 0; column < hidden; ++column) {
            output[base + column] = qo_bf16_from_f32(staged[column] * inverse *
                                                     (1.0f + qo_bf16_to_f32(weight[column])));
        }
    }
    free(staged);
}

static float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

/* crates/qwc-cuda/cuda/delta_prepare.cu:34-42 */
static float softplusf_(float x) {
    if (x > 20.0f) return x;
    if (x < -20.0f) return expf(x);
    return log1pf(expf(x));
}

/*
 * crates/qwc-cuda/cuda/delta_prepare.cu:44-86 (conv1d update + SiLU + split)
 * and :168-245 (L2 normalisation, k.q, alpha, beta).  Channels are
 * [q (k_heads*128), k (k_heads*128), v (v_heads*128)]; conv_state is
 * f32[capacity][channels][3]; conv_weight bf16[channels][4].
 */
QO_API void qo_delta_prepare_decode(const uint16_t* mixed_qkv, const uint16_t* a_projection,
                                    const uint16_t* b_projection, const uint16_t* conv_weight,
                                    const uint16_t* a_log, const uint16_t* dt_bias,
                                    float* conv_state, const uint32_t* state_slots, float* query,
                                    float* key, float* value, float* alpha, float* beta, float* kq,
                                    int batch, int mixed_stride, int gate_stride, int k_heads,
                                    int v_heads, int head_dim) {
    const int qk = k_heads * head_dim;
    const int vel = v_heads * head_dim;
    const int channels = 2 * qk + vel;
    const int ratio = v_heads / k_heads;
    for (int b = 0; b < batch; ++b) {
        const uint32_t slot = state_slots[b];
        for (int channel = 0; channel < channels; ++channel) {
            float* history = conv_state + ((size_t)slot * channels + channel) * 3;
            const float current = qo_bf16_to_f32(mixed_qkv[(size_t)b * mixed_stride + channel]);
            const uint16_t* w = conv_weight + (size_t)channel * 4;
            float convolved = qo_bf16_to_f32(w[0]) * history[0];
            convolved = fmaf(qo_bf16_to_f32(w[1]), history[1], convolved);
            convolved = fmaf(qo_bf16_to_f32(w[2]), history[2], convolved);
            convolved = fmaf(qo_bf16_to_f32(w[3]), current, convolved);
            history[0] = history[1];
            history[1] = history[2];
            history[2] = current;
            const float activated = bf16_round(convolved * sigmoidf_(convolved));
            if (channel < qk) {
                query[(size_t)b * qk + channel] = activated;
            } else if (channel < 2 * qk) {
                key[(size_t)b * qk + channel - qk] = activated;
            } else {
                value[(size_t)b * vel + channel - 2 * qk] = activated;
            }
        }
        for (int head = 0; head < k_heads; ++head) {
            float* qh = query + ((size_t)b * k_heads + head) * head_dim;
            float* kh = key + ((size_t)b * k_heads + head) * head_dim;
            float q_sum = 0.0f, k_sum = 0.0f;
            for (int d = 0; d < head_dim; ++d) {
                q_sum += qh[d] * qh[d];
                k_sum += kh[d] * kh[d];
            }
            const float q_inverse = (1.0f / sqrtf(q_sum + 1e-6f)) * (1.0f / sqrtf((float)head_dim));
            const float k_inverse = 1.0f / sqrtf(k_sum + 1e-6f);
            float kq_sum = 0.0f;
            for (int d = 0; d < head_dim; ++d) {
                qh[d] = qh[d] * q_inverse;
                kh[d] = kh[d] * k_inverse;
                kq_sum += qh[d] * kh[d];
            }
            kq[(size_t)b * k_heads + head] = kq_sum;
            for (int r = 0; r < ratio; ++r) {
                const int value_head = head * ratio + r;
                const size_t gate_read = (size_t)b * gate_stride + value_head;
                const size_t gate_offset = (size_t)b * v_heads + value_head;
                const float projected_a = qo_bf16_to_f32(a_projection[gate_read]);
                const float projected_b = qo_bf16_to_f32(b_projection[gate_read]);
                const float log_a = qo_bf16_to_f32(a_log[value_head]);
                const float bias = qo_bf16_to_f32(dt_bias[value_head]);
                const float log_decay = -expf(log_a) * softplusf_(projected_a + bias);
                alpha[gate_offset] = expf(log_decay);
                beta[gate_offset] = sigmoidf_(projected_b);
            }
        }
    }
}

/* crates/qwc-cuda/cuda/delta_output.cu:20-64 : four bf16 roundings, direct weight. */
QO_API void qo_delta_gated_rmsnorm(const float* input, const uint16_t* gate, const uint16_t* weight,
                                   uint16_t* output, int batch, int heads, int head_dim,
                                   float epsilon, int gate_stride) {
    for (int b = 0; b < batch; ++b) {
        for (int head = 0; head < heads; ++head) {
            const size_t offset = ((size_t)b * heads + head) * head_dim;
            const size_t gate_offset = (size_t)b * gate_stride + (size_t)head * head_dim;
            float sum = 0.0f;
            for (int d = 0; d < head_dim; ++d) {
                const float value = bf16_round(input[offset + d]);
                sum += value * value;
            }
            const float inverse = 1.0f / sqrtf(sum / (float)head_dim + epsilon);
            for (int d = 0; d < head_dim; ++d) {
                const float value = bf16_round(input[offset + d]);
                const float normalized = bf16_round(value * inverse);
                const float weighted = bf16_round(qo_bf16_to_f32(weight[d]) * normalized);
                const float g = qo_bf16_to_f32(gate[gate_offset + d]);
                const float silu = g / (1.0f + expf(-g));
                output[offset + d] = qo_bf16_from_f32(weighted * silu);
            }
        }
    }
}

/*
 * crates/qwc-cuda/cuda/attention_prepare.cu:52-143 with the CPU statement of
 * crates/qwc-cuda/tests/attention_prepare.rs:9-33: per-head zero-centred RMSNorm
 * (1 + w), rotate-half RoPE on the first rope_dim dims, query -> bf16, key and
 * value -> e4m3 written at (physical_blocks[b], block_offsets[b]).
 * k_inv_scale / v_inv_scale (nullable, per kv head) divide before the fp8
 * store; NULL is the reference's unscaled cache.
 */
QO_API void qo_prepare_attention_decode_fp8(
    const uint16_t* query_gate_projection, const uint16_t* key_projection,
    const uint16_t* value_projection, const uint16_t* query_norm_weight,
    const uint16_t* key_norm_weight, const uint16_t* cosine, const uint16_t* sine,
    const uint32_t* physical_blocks, const uint32_t* block_offsets, uint16_t* query,
    uint8_t* key_cache, uint8_t* value_cache, int batch, float epsilon, int q_heads, int kv_heads,
    int head_dim, int rope_dim, int page_size, const float* k_inv_scale, const float* v_inv_scale) {
    float* normalized = (float*)malloc(sizeof(float) * (size_t)head_dim);
    const int half = rope_dim / 2;
    for (int b = 0; b < batch; ++b) {
        const uint16_t* row_cos = cosine + (size_t)b * rope_dim;
        const uint16_t* row_sin = sine + (size_t)b * rope_dim;
        for (int pass = 0; pass < 2; ++pass) {
            const int heads = pass == 0 ? q_heads : kv_heads;
            for (int head = 0; head < heads; ++head) {
                const uint16_t* raw =
                    pass == 0
                        ? query_gate_projection + ((size_t)b * q_heads + head) * (2 * (size_t)head_dim)
                        : key_projection + ((size_t)b * kv_heads + head) * head_dim;
                const uint16_t* weight = pass == 0 ? query_norm_weight : key_norm_weight;
                float sum = 0.0f;
                for (int d = 0; d < head_dim; ++d) {
                    const float x = qo_bf16_to_f32(raw[d]);
                    sum += x * x;
                }
                const float inverse = 1.0f / sqrtf(sum / (float)head_dim + epsilon);
                for (int d = 0; d < head_dim; ++d) {
                    normalized[d] = bf16_round(qo_bf16_to_f32(raw[d]) * inverse *
                                               (1.0f + qo_bf16_to_f32(weight[d])));
                }
                size_t cache_base = 0;
                if (pass == 1) {
                    cache_base = (((size_t)physical_blocks[b] * kv_heads + head) * page_size +
                                  block_offsets[b]) * head_dim;
                }
                for (int d = 0; d < head_dim; ++d) {
                    float value = normalized[d];
                    if (d < rope_dim) {
                        const int paired = d < half ? d + half : d - half;
                        const float rotated = normalized[paired] * (d < half ? -1.0f : 1.0f);
                        value = value * qo_bf16_to_f32(row_cos[d]) + rotated * qo_bf16_to_f32(row_sin[d]);
                    }
                    if (pass == 0) {
                        query[((size_t)b * q_heads + head) * head_dim + d] = qo_bf16_from_f32(value);
                    } else {
                        const float ks = k_inv_scale ? k_inv_scale[head] : 1.0f;
                        const float vs = v_inv_scale ? v_inv_scale[head] : 1.0f;
                        key_cache[cache_base + d] = qo_e4m3_encode(value * ks);
                        const float vv = qo_bf16_to_f32(
                            value_projection[((size_t)b * kv_heads + head) * head_dim + d]);
                        value_cache[cache_base + d] = qo_e4m3_encode(vv * vs);
                    }
                }
            }
        }
    }
    free(normalized);
}

/* crates/qwc-cuda/cuda/vocab_fp8.cu:113-136 ; out-of-vocabulary id -> zero row. */
QO_API void qo_fp8_embedding_gather(const uint8_t* table, const float* row_scales,
                                    const uint32_t* token_ids, uint16_t* output, int batch, int cols,
                                    int vocab) {
    for (int b = 0; b < batch; ++b) {
        const uint32_t token = token_ids[b];
        for (int c = 0; c < cols; ++c) {
            float value = 0.0f;
            if (token < (uint32_t)vocab) {
                value = qo_e4m3(table[(size_t)token * cols + c]) * row_scales[token];
            }
            output[(size_t)b * cols + c] = qo_bf16_from_f32(value);
        }
    }
}

/* crates/qwc-cuda/src/vocab.rs:454-474 : logit = (sum e4m3(w) * hidden) * row_scale, fp32. */
QO_API void qo_fp8_lm_head(const uint8_t* weights, const float* row_scales, const uint16_t* hidden,
                           float* logits, int batch, int hidden_size, int vocab) {
    float* x = (float*)malloc(sizeof(float) * (size_t)batch * hidden_size);
    for (size_t i = 0; i < (size_t)batch * hidden_size; ++i) {
        x[i] = qo_bf16_to_f32(hidden[i]);
    }
#pragma omp parallel for schedule(static)
    for (int row = 0; row < vocab; ++row) {
        for (int b = 0; b < batch; ++b) {
            float acc = 0.0f;
            for (int c = 0; c < hidden_size; ++c) {
                acc += qo_e4m3(weights[(size_t)row * hidden_size + c]) * x[(size_t)b * hidden_size + c];
            }
            logits[(size_t)b * vocab + row] = acc * row_scales[row];
        }
    }
    free(x);
}

/* crates/qwc-cuda/cuda/vocab_fp8.cu:70-110 : per-row amax / 448 scale, empty row -> scale 1. */
QO_API void qo_fp8_quantize_rows(const uint16_t* input, uint8_t* output, float* row_scales, int rows,
                                 int cols) {
    for (int row = 0; row < rows; ++row) {
        float row_max = 0.0f;
        for (int c = 0; c < cols; ++c) {
            row_max = fmaxf(row_max, fabsf(qo_bf16_to_f32(input[(size_t)row * cols + c])));
        }
        const float scale = row_max > 0.0f ? row_max / 448.0f : 1.0f;
        row_scales[row] = scale;
        const float inverse = 1.0f / scale;
        for (int c = 0; c < cols; ++c) {
            output[(size_t)row * cols + c] =
                qo_e4m3_encode(qo_bf16_to_f32(input[(size_t)row * cols + c]) * inverse);
        }
    }
}

/* crates/qwc-cuda/cuda/sampling.cu:11-14 : maximum value, ties -> lower index. */
QO_API void qo_argmax(const float* logits, uint32_t* output, int vocab, int batch) {
    for (int b = 0; b < batch; ++b) {
        float best = -INFINITY;
        uint32_t best_index = UINT32_MAX;
        for (int c = 0; c < vocab; ++c) {
            const float value = logits[(size_t)b * vocab + c];
            if (value > best || (value == best && (uint32_t)c < best_index)) {
                best = value;
                best_index = (uint32_t)c;
            }
        }
        output[b] = best_index;
    }
}

/* ------------------------------------------------------------------ */
/* Ragged-batch layout (integer path)                                  */
/* ------------------------------------------------------------------ */

/*
 * crates/qwc-runtime/src/layout.rs:54-152 (BatchLayout::build, decode rows) followed by
 * crates/qwc-engine/src/executor.rs:1939-1990 (upload_layout_decode).
 *
 * Inputs describe the cache per state slot: seq_tokens[slot] (tokens including the
 * one this step appends) and seq_blocks[slot][0..max_blocks) (page ids in logical
 * order).  row_slots[row] lists the decode rows in batch order.
 * Outputs are the device arrays the step reads, plus the CSR intermediates.
 * Returns 0, or a negative code mirroring LayoutError
 * (-1 missing/empty sequence, -2 duplicate, -4 missing KV blocks).
 */
QO_API int qo_layout_decode(const uint32_t* row_slots, int rows, const uint32_t* seq_tokens,
                            const uint32_t* seq_blocks, const uint32_t* seq_block_counts,
                            int capacity, int max_blocks, int page_size, uint32_t* state_slots,
                            uint32_t* positions, uint32_t* context_lengths,
                            uint32_t* block_table_offsets, uint32_t* block_ids,
                            uint32_t* physical_blocks, uint32_t* block_offsets,
                            uint32_t* block_tables) {
    uint8_t* seen = (uint8_t*)calloc((size_t)capacity, 1);
    memset(block_tables, 0, sizeof(uint32_t) * (size_t)rows * max_blocks);
    block_table_offsets[0] = 0;
    int status = 0;
    for (int row = 0; row < rows && status == 0; ++row) {
        const uint32_t slot = row_slots[row];
        if (slot >= (uint32_t)capacity || seq_tokens[slot] == 0) {
            status = -1;
            break;
        }
        if (seen[slot]) {
            status = -2;
            break;
        }
        seen[slot] = 1;
        const uint32_t tokens = seq_tokens[slot];
        const uint32_t position = tokens - 1;
        const uint32_t blocks = (tokens + (uint32_t)page_size - 1) / (uint32_t)page_size;
        if (blocks > seq_block_counts[slot] || blocks > (uint32_t)max_blocks) {
            status = -4;
            break;
        }
        state_slots[row] = slot;
        positions[row] = position;
        context_lengths[row] = tokens;
        const uint32_t begin = block_table_offsets[row];
        for (uint32_t i = 0; i < blocks; ++i) {
            const uint32_t id = seq_blocks[(size_t)slot * max_blocks + i];
            block_ids[begin + i] = id;
            block_tables[(size_t)row * max_blocks + i] = id;
        }
        block_table_offsets[row + 1] = begin + blocks;
        physical_blocks[row] = seq_blocks[(size_t)slot * max_blocks + position / (uint32_t)page_size];
        block_offsets[row] = position % (uint32_t)page_size;
    }
    free(seen);
    return status;
}

/*
 * RoPE rows as crates/qwc-engine/src/executor.rs:1953-1958 builds them on the
 * host: inverse = theta^(-2 (d mod rope_dim/2) / rope_dim) in f32 powf,
 * angle = f32(position) * inverse, cos/sin rounded to bf16.
 */
QO_API void qo_rope_rows(const uint32_t* positions, int rows, int rope_dim, float theta,
                         uint16_t* cosine, uint16_t* sine) {
    for (int row = 0; row < rows; ++row) {
        for (int d = 0; d < rope_dim; ++d) {
            const int pair = d % (rope_dim / 2);
            const float inverse = powf(theta, -(2.0f * (float)pair) / (float)rope_dim);
            const float angle = (float)positions[row] * inverse;
            cosine[(size_t)row * rope_dim + d] = qo_bf16_from_f32(cosf(angle));
            sine[(size_t)row * rope_dim + d] = qo_bf16_from_f32(sinf(angle));
        }
    }
}

QO_API int qo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

QO_API void qo_set_num_threads(int threads) {
#ifdef _OPENMP
    omp_set_num_threads(threads);
#else
    (void)threads;
#endif
}
