// Decode executor: resident buffers, synthetic model, the captured 64-layer step.
//
// C++ counterpart of the decode path of crates/qwc-engine/src/executor.rs
// (new_with_pool_options :395-546, execute_layout :878-952, launch_decode :954-995,
// decode_forward :997-1112, linear_attention :1774-1831, full_attention :1833-1937).
// Differences that come from the device-side batch packing: the page table and token
// counts are resident on the device, a step uploads row slots, tokens and table edits in one
// copy, and the packing kernels run inside the captured graph.  q, k and v projections of a
// full-attention layer are one fused matrix (they share the input), as the mixer in-proj
// already is in the reference (crates/qwc-engine/src/weights.rs:50-60).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../../include/qwc_engine.h"
#include "runtime.h"
#include "runtime_handles.h"

namespace {

using qwc::runtime::Batch;
using qwc::runtime::BatchLayout;

constexpr int kQueryHeads = 24;
constexpr int kKvHeads = 4;
constexpr int kHeadDim = 256;
constexpr int kRopeDim = 64;
constexpr int kDeltaKeyHeads = 16;
constexpr int kDeltaDim = 128;
constexpr float kRopeTheta = 1.0e7f;  // crates/qwc-core/src/arch.rs:76
constexpr float kEps = 1.0e-6f;       // crates/qwc-core/src/arch.rs:14
constexpr int kArgmaxParts = 64;

#define QWC_TRY(expr)                     \
    do {                                  \
        const int qwc_try_code = (expr);  \
        if (qwc_try_code != 0) {          \
            return qwc_try_code;          \
        }                                 \
    } while (0)

// ---- synthetic data ------------------------------------------------------------------

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// kind 0: uniform bytes; 1: e4m3 block-scale codes (0.0078 .. 0.22, the bulk of |N(0,1)| * 0.05);
// 2: e4m3 cache codes, both signs, magnitude codes below 0x70; 3: int8 state codes in [-127, 127]
__global__ void fill_bytes_kernel(uint8_t* out, size_t n, uint64_t seed, int kind) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x * 8;
    for (size_t base = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; base < n; base += stride) {
        uint64_t r = mix64(seed * 0x100000001B3ull + base);
        for (int j = 0; j < 8 && base + j < n; ++j) {
            const uint32_t byte = static_cast<uint32_t>(r >> (8 * j)) & 0xff;
            uint8_t value;
            if (kind == 0) {
                value = static_cast<uint8_t>(byte);
            } else if (kind == 1) {
                value = static_cast<uint8_t>(0x08 + (byte % 0x28));
            } else if (kind == 2) {
                value = static_cast<uint8_t>((byte & 0x80) | ((byte & 0x7f) % 0x70));
            } else {
                value = static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(byte % 255) - 127));
            }
            out[base + j] = value;
        }
    }
}

// Normal(mean, std) rounded to bf16 (Box-Muller on two hashed uniforms).
__global__ void fill_bf16_normal_kernel(__nv_bfloat16* out, size_t n, uint64_t seed, float mean, float std) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t r = mix64(seed * 0x100000001B3ull + i);
        const float u1 = (static_cast<float>(r & 0xffffff) + 1.0f) * (1.0f / 16777217.0f);
        const float u2 = static_cast<float>((r >> 24) & 0xffffff) * (1.0f / 16777216.0f);
        const float z = sqrtf(-2.0f * logf(u1)) * cosf(6.2831853f * u2);
        out[i] = __float2bfloat16(mean + std * z);
    }
}

__global__ void fill_f32_uniform_kernel(float* out, size_t n, uint64_t seed, float low, float high) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t r = mix64(seed * 0x100000001B3ull + i);
        out[i] = low + (high - low) * static_cast<float>(r & 0xffffff) * (1.0f / 16777216.0f);
    }
}

// ---- optional NCCL (latency mode), resolved at run time ------------------------------

struct NcclApi {
    void* handle = nullptr;
    int (*get_unique_id)(void*) = nullptr;
    int (*all_gather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*comm_destroy)(void*) = nullptr;
};

struct NcclUniqueIdBytes {
    char bytes[128];
};

NcclApi& nccl_api() {
    static NcclApi api;
    return api;
}

bool load_nccl() {
    NcclApi& api = nccl_api();
    if (api.handle != nullptr) {
        return true;
    }
    void* handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (handle == nullptr) {
        return false;
    }
    api.get_unique_id = reinterpret_cast<int (*)(void*)>(dlsym(handle, "ncclGetUniqueId"));
    api.all_gather =
        reinterpret_cast<int (*)(const void*, void*, size_t, int, void*, cudaStream_t)>(dlsym(handle, "ncclAllGather"));
    api.comm_destroy = reinterpret_cast<int (*)(void*)>(dlsym(handle, "ncclCommDestroy"));
    if (!api.get_unique_id || !api.all_gather || !api.comm_destroy || !dlsym(handle, "ncclCommInitRank")) {
        return false;
    }
    api.handle = handle;
    return true;
}

// ---- model -----------------------------------------------------------------------------

struct LinearW {
    uint8_t* packed = nullptr;
    uint8_t* scales = nullptr;
    int out_features = 0;  // rows held by this rank
    int in_features = 0;
    float global_scale = 1.0f;
    size_t weight_bytes() const {
        return static_cast<size_t>(out_features) * in_features / 2 + static_cast<size_t>(out_features) * in_features / 16;
    }
};

struct Layer {
    bool full = false;
    int slot = 0;  // index among layers of its kind
    __nv_bfloat16* input_norm = nullptr;
    __nv_bfloat16* post_norm = nullptr;
    LinearW gate, up, down;
    // linear attention
    LinearW in_proj, la_out;
    __nv_bfloat16* conv_weight = nullptr;
    __nv_bfloat16* a_log = nullptr;
    __nv_bfloat16* dt_bias = nullptr;
    __nv_bfloat16* out_norm = nullptr;
    int8_t* state = nullptr;
    float* state_scales = nullptr;
    float* conv_state = nullptr;
    // full attention
    LinearW qkv, o;
    __nv_bfloat16* q_norm = nullptr;
    __nv_bfloat16* k_norm = nullptr;
    float* k_scale = nullptr;
    float* v_scale = nullptr;
    uint8_t* k_cache = nullptr;
    uint8_t* v_cache = nullptr;
};

struct Phase {
    const char* label;
    cudaEvent_t event;
};

}  // namespace

struct qwc_engine {
    qwc_engine_config cfg{};
    cudaStream_t stream = nullptr;
    std::vector<void*> allocations;
    std::vector<Layer> layers;
    __nv_bfloat16* final_norm = nullptr;
    uint8_t* embed = nullptr;
    float* embed_scales = nullptr;
    uint8_t* lm_head = nullptr;
    float* lm_head_scales = nullptr;
    int vocab_local = 0;

    // dimensions
    int v_heads = 0, channels = 0, mixer_width = 0, z_offset = 0, a_offset = 0, b_offset = 0;
    int qkv_width = 0, max_blocks = 0, partitions = 1, max_edits = 0;

    // activations
    __nv_bfloat16 *residual = nullptr, *normed = nullptr, *mixer_in = nullptr, *qkv_buf = nullptr, *query = nullptr;
    __nv_bfloat16 *attention_out = nullptr, *delta_normed = nullptr, *mixer_out = nullptr, *mlp_hidden = nullptr;
    __nv_bfloat16* mlp_out = nullptr;
    // activations staged for the projection that reads them (f16, tensor-core operand layout)
    void *normed_staged = nullptr, *delta_normed_staged = nullptr, *attention_out_staged = nullptr;
    void* mlp_hidden_staged = nullptr;
    void* streamk_workspace = nullptr;
    float* split_sums = nullptr;  // fp32 partial rows of a K-split projection: [slice][batch][hidden]
    float* split_sums_wide = nullptr;  // ... of the mixer in-projection or q|k|v: [slice][batch][width]
    float *dq = nullptr, *dk = nullptr, *dv = nullptr, *dalpha = nullptr, *dbeta = nullptr, *dkq = nullptr;
    float *delta_out = nullptr, *logits = nullptr, *argmax_values = nullptr;
    uint32_t* argmax_indices = nullptr;
    void* attention_workspace = nullptr;
    size_t attention_workspace_bytes = 0;

    // device-resident tables and per-step arrays
    uint32_t *seq_tokens = nullptr, *seq_blocks = nullptr;
    __nv_bfloat16* rope_table = nullptr;
    uint32_t *state_slots = nullptr, *positions = nullptr, *context_lengths = nullptr, *physical_blocks = nullptr;
    uint32_t *block_offsets = nullptr, *block_tables = nullptr, *block_table_offsets = nullptr, *row_count = nullptr;
    __nv_bfloat16 *cosine = nullptr, *sine = nullptr;

    // step inputs / outputs: [row_slots | tokens | edits] and [sampled | pack status | wait status]
    uint32_t* in_host = nullptr;
    uint32_t* in_dev = nullptr;
    uint32_t* out_host = nullptr;
    uint32_t* out_dev = nullptr;
    size_t in_words = 0;

    std::vector<cudaGraphExec_t> graphs;  // index batch - 1
    std::vector<char> warmed;  // per batch size: lazy launcher set-up done outside capture

    // timeline (eager mode only)
    bool profiling = false;
    const char* phase_filter = nullptr;  // when set, only phases whose label starts with it are launched
    int filtered_launches = 0;
    std::vector<Phase> marks;

    // per-layer trace (parity tests): [layer][mixer_out | residual after the MLP][max_batch * hidden] bf16
    __nv_bfloat16* trace = nullptr;

    // latency mode
    void* comm = nullptr;  // NCCL all-gather form
    // fused form: the block that the ranks' projections store their slices into, and everybody's block
    // as this device addresses it
    unsigned char* exchange_block = nullptr;
    size_t exchange_bytes = 0;
    void* exchange_blocks[QWC_MAX_PEERS] = {};
    std::vector<void*> opened_peers;
    bool peers_ready = false;
    uint32_t* epoch = nullptr;
    unsigned long long* wait_profile = nullptr;  // [exchange of the step]: longest wait for a peer's word, ns
    bool profile_waits = false;  // off by default: the bookkeeping itself (atomics on one word per exchange) is
                                 // slow enough to lengthen the waits it measures
    size_t row_wide = 0, row_hidden[2] = {0, 0}, row_swiglu = 0, row_candidates = 0;  // offsets in the block

    // worker loop state
    std::vector<uint32_t> last_token;  // per state slot

    // device bytes asked for through gpu_alloc and their ceiling
    size_t memory_used = 0;
    size_t memory_limit = SIZE_MAX;
};

namespace {

int gpu_alloc(qwc_engine* e, void** out, size_t bytes, bool zero = false) {
    void* p = nullptr;
    const size_t reserved = bytes == 0 ? 16 : bytes;
    // the ceiling refuses before the driver is asked (crates/qwc-cuda/src/memory.rs:80-88)
    if (reserved > e->memory_limit || e->memory_used > e->memory_limit - reserved) {
        return cudaErrorMemoryAllocation;
    }
    const cudaError_t err = cudaMalloc(&p, reserved);
    if (err != cudaSuccess) {
        return err;
    }
    e->memory_used += reserved;
    e->allocations.push_back(p);
    if (zero) {
        const cudaError_t cleared = cudaMemsetAsync(p, 0, bytes, e->stream);
        if (cleared != cudaSuccess) {
            return cleared;
        }
    }
    *out = p;
    return 0;
}

template <typename T>
int gpu_alloc_t(qwc_engine* e, T** out, size_t count, bool zero = false) {
    return gpu_alloc(e, reinterpret_cast<void**>(out), count * sizeof(T), zero);
}

// Replicated tensors (norms, conv, caches, state, embedding) are the same on every rank of a column
// split; the split matrices hold different rows on every rank, so their seed takes the rank in.
uint64_t tensor_seed(const qwc_engine* e, int layer, int tag, bool split_tensor = false) {
    return e->cfg.seed * 1000003ull + static_cast<uint64_t>(layer) * 131ull + static_cast<uint64_t>(tag) +
           (split_tensor ? static_cast<uint64_t>(e->cfg.split_rank) * 7919ull * 65537ull : 0ull);
}

void fill_bytes(qwc_engine* e, void* p, size_t n, uint64_t seed, int kind) {
    fill_bytes_kernel<<<1184, 256, 0, e->stream>>>(static_cast<uint8_t*>(p), n, seed, kind);
}

void fill_normal(qwc_engine* e, __nv_bfloat16* p, size_t n, uint64_t seed, float mean, float std) {
    fill_bf16_normal_kernel<<<296, 256, 0, e->stream>>>(p, n, seed, mean, std);
}

void fill_uniform(qwc_engine* e, float* p, size_t n, uint64_t seed, float low, float high) {
    fill_f32_uniform_kernel<<<296, 256, 0, e->stream>>>(p, n, seed, low, high);
}

size_t scale_storage(int rows, int in_features) {
    return static_cast<size_t>((rows + 127) / 128 * 128) * static_cast<size_t>((in_features / 16 + 3) / 4 * 4);
}

int make_linear(qwc_engine* e, LinearW* w, int out_features, int in_features, int layer, int tag) {
    const int split = e->cfg.split_size;
    w->out_features = out_features / split;
    w->in_features = in_features;
    w->global_scale = 1.0f;
    const size_t packed_bytes = static_cast<size_t>(w->out_features) * in_features / 2;
    const size_t scale_bytes = scale_storage(w->out_features, in_features);
    QWC_TRY(gpu_alloc_t(e, &w->packed, packed_bytes));
    QWC_TRY(gpu_alloc_t(e, &w->scales, scale_bytes));
    fill_bytes(e, w->packed, packed_bytes, tensor_seed(e, layer, tag, true), 0);
    fill_bytes(e, w->scales, scale_bytes, tensor_seed(e, layer, tag + 1, true), 1);
    return 0;
}

int make_norm(qwc_engine* e, __nv_bfloat16** w, int n, int layer, int tag, float mean, float std) {
    QWC_TRY(gpu_alloc_t(e, w, n));
    fill_normal(e, *w, n, tensor_seed(e, layer, tag), mean, std);
    return 0;
}

void mark(qwc_engine* e, const char* label) {
    if (!e->profiling) {
        return;
    }
    cudaEvent_t event;
    cudaEventCreate(&event);
    cudaEventRecord(event, e->stream);
    e->marks.push_back({label, event});
}

// Opens a phase of the step: records its timeline mark and tells whether its kernels are to be
// launched (always, unless a phase filter selects a subset for a graph-timed measurement).
bool phase(qwc_engine* e, const char* label) {
    mark(e, label);
    if (e->phase_filter == nullptr) {
        return true;
    }
    const bool selected = std::strncmp(label, e->phase_filter, std::strlen(e->phase_filter)) == 0;
    e->filtered_launches += selected ? 1 : 0;
    return selected;
}

// Names the projection after the one about to be launched (qwc_nvfp4_prefetch_next): its first
// stages are asked of L2 while the launch drains.  Only where the two are a few small kernels apart:
// an attention pass in between would push the lines out of L2 again.
void hint_next(const qwc_engine* e, const LinearW& next) {
    if (e->cfg.split_size == 1) {
        (void)qwc_nvfp4_prefetch_next(next.packed, next.scales, nullptr, nullptr, next.out_features, next.in_features, 0);
    }
}

// ... a projection that will run as a regular K split (its CTAs start elsewhere in the matrix)
void hint_next_split(const qwc_engine* e, const LinearW& next) {
    if (e->cfg.split_size == 1) {
        (void)qwc_nvfp4_prefetch_next(next.packed, next.scales, nullptr, nullptr, next.out_features, next.in_features, 3);
    }
}

void hint_next_pair(const qwc_engine* e, const LinearW& gate, const LinearW& up) {
    if (e->cfg.split_size == 1) {
        (void)qwc_nvfp4_prefetch_next(gate.packed, gate.scales, up.packed, up.scales, gate.out_features,
                                      gate.in_features, 1);
    }
}

// One projection; in latency mode the local slice lands at this rank's offset of the full
// row and an all-gather completes it (batch 1 only, so the gathered layout is the row itself).
int project(qwc_engine* e, const LinearW& w, const __nv_bfloat16* input, __nv_bfloat16* output, int batch) {
    __nv_bfloat16* target = output + static_cast<size_t>(e->cfg.split_rank) * w.out_features;
    QWC_TRY(qwc_nvfp4_w4a16(w.packed, w.scales, input, e->cfg.split_size > 1 ? target : output, w.out_features,
                            w.in_features, batch, w.global_scale, e->stream));
    if (e->cfg.split_size > 1) {
        const int rc = nccl_api().all_gather(target, output, static_cast<size_t>(w.out_features), /*ncclBfloat16*/ 9,
                                             e->comm, e->stream);
        if (rc != 0) {
            return cudaErrorUnknown;
        }
    }
    return 0;
}

// A projection to the hidden width (mixer output, MLP down) followed by the residual RMSNorm: too few
// row tiles for the SMs, so it runs as a regular K split whose slices the norm sums (one GPU only).
int project_and_norm(qwc_engine* e, const LinearW& w, const void* staged_input, __nv_bfloat16* projection_rows,
                     const __nv_bfloat16* norm_weight, int batch, const char* gemm_label) {
    const qwc_engine_config& c = e->cfg;
    if (phase(e, gemm_label)) {
        QWC_TRY(qwc_nvfp4_w4a16_split(w.packed, w.scales, staged_input, e->split_sums, w.out_features, w.in_features,
                                      batch, e->stream));
    }
    if (phase(e, "norm")) {
        // the projection's own bf16 rows reach memory only for a caller that traces the layers
        QWC_TRY(qwc_rmsnorm_bf16_split_staged(e->split_sums, qwc_nvfp4_split_count(w.out_features, w.in_features),
                                              w.global_scale, e->trace != nullptr ? projection_rows : nullptr,
                                              e->residual, norm_weight, nullptr, e->normed_staged, batch, c.hidden,
                                              kEps, e->stream));
    }
    return 0;
}

// ---- latency mode, fused form ---------------------------------------------------------------
// One sequence; every projection computes this rank's rows and stores its K-split slices into every
// rank's exchange block, and the kernel that consumes the row sums them after a bounded wait for the
// tagged words (kernels/exchange.cuh).  Everything between projections (norms, the DeltaNet update, the
// attention pass) runs replicated on every rank: at one row it is small next to the weights.
qwc_exchange_row exchange_row(const qwc_engine* e, size_t offset, uint32_t instance, int width) {
    qwc_exchange_row row = {};
    for (int r = 0; r < e->cfg.split_size; ++r) {
        row.blocks[r] = e->exchange_blocks[r];
    }
    row.ranks = e->cfg.split_size;
    row.rank = e->cfg.split_rank;
    row.epoch = e->epoch;
    row.instance = instance;
    row.offset = offset;
    row.width = width;
    // a graph of selected phases only (timing): its consumers run on whatever the last whole step left
    row.flags = e->phase_filter != nullptr ? QWC_EXCHANGE_ANY_TAG : 0u;
    row.wait_profile = e->profile_waits ? e->wait_profile : nullptr;
    return row;
}

int decode_forward_exchange(qwc_engine* e) {
    const qwc_engine_config& c = e->cfg;
    cudaStream_t s = e->stream;
    if (!e->peers_ready) {
        return cudaErrorNotReady;  // the peers' blocks are not mapped yet
    }
    // A graph of selected phases only (qwc_engine_time_phases) does not advance the epoch and its consumers
    // take the words that are there whatever their tag (exchange_row): nothing waits.
    uint32_t* row_slots = e->in_dev;
    uint32_t* tokens = e->in_dev + c.max_batch;
    const qwc_table_edit* edits = reinterpret_cast<const qwc_table_edit*>(e->in_dev + 2 * c.max_batch);
    const int batch = 1;
    uint32_t instance = 0;
    // names the projection after the one about to be launched, so that the launch asks L2 for its first
    // stages (every projection of this mode runs as a regular K split: hint kinds 3 and 4)
    const auto hint_matrix = [](const LinearW& next) {
        (void)qwc_nvfp4_prefetch_next(next.packed, next.scales, nullptr, nullptr, next.out_features, next.in_features, 3);
    };
    const auto hint_pair = [](const LinearW& gate, const LinearW& up) {
        (void)qwc_nvfp4_prefetch_next(gate.packed, gate.scales, up.packed, up.scales, gate.out_features,
                                      gate.in_features, 4);
    };

    if (e->phase_filter == nullptr) {
        QWC_TRY(qwc_exchange_advance(e->epoch, s));
    }
    if (phase(e, "pack")) {
        QWC_TRY(qwc_page_table_apply(e->seq_tokens, e->seq_blocks, edits, e->max_edits, c.state_slots, e->max_blocks, s));
        QWC_TRY(qwc_pack_decode_batch(row_slots, nullptr, e->seq_tokens, e->seq_blocks, e->rope_table, c.max_context,
                                      e->row_count, e->state_slots, e->positions, e->context_lengths, e->physical_blocks,
                                      e->block_offsets, e->block_tables, e->block_table_offsets, nullptr, e->cosine,
                                      e->sine, e->out_dev + c.max_batch, batch, c.state_slots, e->max_blocks,
                                      c.kv_page_size, s));
    }
    if (phase(e, "embed")) {
        QWC_TRY(qwc_fp8_embedding_gather(e->embed, e->embed_scales, tokens, e->residual, batch, c.hidden, c.vocab, s));
    }
    if (phase(e, "norm")) {
        QWC_TRY(qwc_rmsnorm_bf16_staged(e->residual, nullptr, e->layers[0].input_norm, nullptr, e->normed_staged,
                                        batch, c.hidden, kEps, s));
    }

    // a projection to the hidden width, then the residual norm that sums what all ranks stored
    const auto finish_with_norm = [&](const LinearW& w, const void* staged_input, int which,
                                      __nv_bfloat16* projection_rows, const __nv_bfloat16* norm_weight,
                                      const char* label) -> int {
        const qwc_exchange_row row = exchange_row(e, e->row_hidden[which], instance++, c.hidden);
        if (phase(e, label)) {
            QWC_TRY(qwc_nvfp4_w4a16_exchange(w.packed, w.scales, staged_input, &row, w.out_features, w.in_features, s));
        }
        if (phase(e, "norm")) {
            QWC_TRY(qwc_rmsnorm_bf16_exchanged(&row, qwc_nvfp4_exchange_slices(w.out_features, w.in_features, 0),
                                               w.global_scale, e->trace != nullptr ? projection_rows : nullptr,
                                               e->residual, norm_weight, nullptr, e->normed_staged, c.hidden, kEps, s));
        }
        return 0;
    };

    for (size_t index = 0; index < e->layers.size(); ++index) {
        const Layer& layer = e->layers[index];
        if (!layer.full) {
            const LinearW& in = layer.in_proj;
            const qwc_exchange_row row = exchange_row(e, e->row_wide, instance++, e->mixer_width);
            const int slices = qwc_nvfp4_exchange_slices(in.out_features, in.in_features, 0);
            if (phase(e, "gemm.la_in")) {
                hint_matrix(layer.la_out);
                QWC_TRY(qwc_nvfp4_w4a16_exchange(in.packed, in.scales, e->normed_staged, &row, in.out_features,
                                                 in.in_features, s));
            }
            if (phase(e, "delta.prepare")) {
                QWC_TRY(qwc_delta_prepare_decode_exchanged(&row, slices, in.global_scale, e->a_offset, e->b_offset,
                                                           layer.conv_weight, layer.a_log, layer.dt_bias,
                                                           layer.conv_state, e->state_slots, e->dq, e->dk, e->dv,
                                                           e->dalpha, e->dbeta, e->dkq, c.state_slots, s));
            }
            if (phase(e, "delta.scan")) {
                QWC_TRY(qwc_delta_decode_int8_step(layer.state, layer.state_scales, e->state_slots, e->dq, e->dk, e->dv,
                                                   e->dalpha, e->dbeta, e->dkq, e->delta_out, c.state_slots, batch,
                                                   nullptr, 0, 1.0f, nullptr, e->mixer_width, e->z_offset, layer.out_norm,
                                                   kEps, nullptr, s));
            }
            if (phase(e, "delta.norm")) {
                QWC_TRY(qwc_delta_gated_rmsnorm_exchanged(e->delta_out, &row, slices, in.global_scale, e->z_offset,
                                                          layer.out_norm, nullptr, e->delta_normed_staged, kEps, s));
            }
            hint_pair(layer.gate, layer.up);
            QWC_TRY(finish_with_norm(layer.la_out, e->delta_normed_staged, 0, e->mixer_out, layer.post_norm,
                                     "gemm.la_out"));
        } else {
            const LinearW& qkv = layer.qkv;
            const qwc_exchange_row row = exchange_row(e, e->row_wide, instance++, e->qkv_width);
            if (phase(e, "gemm.attn_qkv")) {
                QWC_TRY(qwc_nvfp4_w4a16_exchange(qkv.packed, qkv.scales, e->normed_staged, &row, qkv.out_features,
                                                 qkv.in_features, s));
                QWC_TRY(qwc_nvfp4_sum_exchanged(&row, qwc_nvfp4_exchange_slices(qkv.out_features, qkv.in_features, 0),
                                                qkv.global_scale, e->qkv_buf, s));
            }
            const int q_width = kQueryHeads * 2 * kHeadDim;
            if (phase(e, "attn.prepare")) {
                QWC_TRY(qwc_prepare_attention_decode_fp8_scaled(
                    e->qkv_buf, e->qkv_buf + q_width, e->qkv_buf + q_width + kKvHeads * kHeadDim, layer.q_norm,
                    layer.k_norm, e->cosine, e->sine, e->physical_blocks, e->block_offsets, layer.k_scale, layer.v_scale,
                    e->query, layer.k_cache, layer.v_cache, batch, c.kv_page_size, e->qkv_width, e->qkv_width,
                    e->qkv_width, kEps, s));
            }
            if (phase(e, "attn.decode")) {
                QWC_TRY(qwc_paged_attention_packed_fp8_staged(
                    e->query, e->qkv_buf, layer.k_cache, layer.v_cache, e->block_tables, e->context_lengths, layer.k_scale,
                    layer.v_scale, nullptr, e->attention_out_staged, e->attention_workspace, e->attention_workspace_bytes,
                    batch, 0, e->max_blocks, c.kv_page_size, e->qkv_width, e->partitions, 1.0f / 16.0f, s));
            }
            hint_pair(layer.gate, layer.up);
            QWC_TRY(finish_with_norm(layer.o, e->attention_out_staged, 0, e->mixer_out, layer.post_norm,
                                     "gemm.attn_out"));
        }
        const size_t trace_row = static_cast<size_t>(c.max_batch) * c.hidden;
        if (e->trace != nullptr && e->phase_filter == nullptr) {
            QWC_TRY(cudaMemcpyAsync(e->trace + (2 * index) * trace_row, e->mixer_out, trace_row * 2,
                                    cudaMemcpyDeviceToDevice, s));
        }
        {
            const qwc_exchange_row row = exchange_row(e, e->row_swiglu, instance++, 2 * c.intermediate);
            if (phase(e, "gemm.mlp_gate_up")) {
                hint_matrix(layer.down);
                QWC_TRY(qwc_nvfp4_swiglu_w4a16_exchange(layer.gate.packed, layer.gate.scales, layer.up.packed,
                                                        layer.up.scales, e->normed_staged, &row, layer.gate.out_features,
                                                        layer.gate.in_features, s));
            }
            if (phase(e, "mlp.combine")) {
                QWC_TRY(qwc_swiglu_combine_exchanged(
                    &row, qwc_nvfp4_exchange_slices(layer.gate.out_features, layer.gate.in_features, 1),
                    layer.gate.global_scale, layer.up.global_scale, nullptr, e->mlp_hidden_staged, c.intermediate, s));
            }
        }
        const __nv_bfloat16* next_norm = index + 1 < e->layers.size() ? e->layers[index + 1].input_norm : e->final_norm;
        if (index + 1 < e->layers.size()) {
            const Layer& following = e->layers[index + 1];
            hint_matrix(following.full ? following.qkv : following.in_proj);
        } else {
            (void)qwc_nvfp4_prefetch_next(e->lm_head, nullptr, nullptr, nullptr, e->vocab_local, c.hidden, 2);
        }
        QWC_TRY(finish_with_norm(layer.down, e->mlp_hidden_staged, 1, e->mlp_out, next_norm, "gemm.mlp_down"));
        if (e->trace != nullptr && e->phase_filter == nullptr) {
            QWC_TRY(cudaMemcpyAsync(e->trace + (2 * index + 1) * trace_row, e->residual, trace_row * 2,
                                    cudaMemcpyDeviceToDevice, s));
        }
    }
    if (instance >= QWC_EXCHANGE_MAX_INSTANCES) {
        return cudaErrorInvalidValue;
    }
    // every rank scans its rows of the vocabulary and hands the others its best candidates
    const qwc_exchange_row candidates = exchange_row(e, e->row_candidates, instance++, 4);
    if (phase(e, "lm_head")) {
        QWC_TRY(qwc_fp8_lm_head_exchange(e->lm_head, e->lm_head_scales, e->normed_staged,
                                         c.write_logits ? e->logits : nullptr, &candidates, e->out_dev,
                                         e->out_dev + c.max_batch + 1, c.hidden, e->vocab_local, e->streamk_workspace,
                                         s));
    }
    mark(e, "end");
    return 0;
}

int decode_forward(qwc_engine* e, int batch) {
    const qwc_engine_config& c = e->cfg;
    cudaStream_t s = e->stream;
    if (c.exchange != 0) {
        return decode_forward_exchange(e);
    }
    uint32_t* row_slots = e->in_dev;
    uint32_t* tokens = e->in_dev + c.max_batch;
    const qwc_table_edit* edits = reinterpret_cast<const qwc_table_edit*>(e->in_dev + 2 * c.max_batch);

    if (phase(e, "pack")) {
        QWC_TRY(qwc_page_table_apply(e->seq_tokens, e->seq_blocks, edits, e->max_edits, c.state_slots, e->max_blocks, s));
        QWC_TRY(qwc_pack_decode_batch(row_slots, nullptr, e->seq_tokens, e->seq_blocks, e->rope_table, c.max_context,
                                      e->row_count, e->state_slots, e->positions, e->context_lengths, e->physical_blocks,
                                      e->block_offsets, e->block_tables, e->block_table_offsets, nullptr, e->cosine,
                                      e->sine, e->out_dev + c.max_batch, batch, c.state_slots, e->max_blocks,
                                      c.kv_page_size, s));
    }
    if (phase(e, "embed")) {
        QWC_TRY(qwc_fp8_embedding_gather(e->embed, e->embed_scales, tokens, e->residual, batch, c.hidden, c.vocab, s));
    }
    const bool staged = c.split_size == 1;  // one GPU: every projection reads staged activations
    if (phase(e, "norm")) {
        QWC_TRY(qwc_rmsnorm_bf16_staged(e->residual, nullptr, e->layers[0].input_norm, staged ? nullptr : e->normed,
                                        staged ? e->normed_staged : nullptr, batch, c.hidden, kEps, s));
    }

    for (size_t index = 0; index < e->layers.size(); ++index) {
        const Layer& layer = e->layers[index];
        if (!layer.full) {
            const int in_slices = qwc_nvfp4_split_count(layer.in_proj.out_features, layer.in_proj.in_features);
            if (phase(e, "gemm.la_in")) {
                hint_next_split(e, layer.la_out);
                // one GPU: a regular K split whose slices the prepare step and the gated norm sum
                QWC_TRY(staged ? qwc_nvfp4_w4a16_split(layer.in_proj.packed, layer.in_proj.scales, e->normed_staged,
                                                       e->split_sums_wide, layer.in_proj.out_features,
                                                       layer.in_proj.in_features, batch, s)
                               : project(e, layer.in_proj, e->normed, e->mixer_in, batch));
            }
            if (staged && phase(e, "delta.prepare")) {
                QWC_TRY(qwc_delta_prepare_decode_split(e->split_sums_wide, in_slices, e->mixer_width,
                                                       layer.in_proj.global_scale, e->a_offset, e->b_offset,
                                                       layer.conv_weight, layer.a_log, layer.dt_bias, layer.conv_state,
                                                       e->state_slots, e->dq, e->dk, e->dv, e->dalpha, e->dbeta,
                                                       e->dkq, c.state_slots, batch, s));
            } else if (phase(e, "delta.prepare")) {
                QWC_TRY(qwc_delta_prepare_decode(e->mixer_in, e->mixer_in + e->a_offset, e->mixer_in + e->b_offset,
                                                 layer.conv_weight, layer.a_log, layer.dt_bias, layer.conv_state,
                                                 e->state_slots, e->dq, e->dk, e->dv, e->dalpha, e->dbeta, e->dkq,
                                                 c.state_slots, batch, e->mixer_width, e->mixer_width, s));
            }
            const bool fused_norm = staged && qwc_delta_decode_fuses_norm(batch) != 0;
            if (staged && phase(e, "delta.scan")) {
                // slots and state tiles fetched while the prepare step runs; with one CTA per head the
                // gated norm rides in the same CTA and the staged result goes straight to the out projection
                QWC_TRY(qwc_delta_decode_int8_step(layer.state, layer.state_scales, e->state_slots, e->dq, e->dk, e->dv,
                                                   e->dalpha, e->dbeta, e->dkq, e->delta_out, c.state_slots, batch,
                                                   e->split_sums_wide, in_slices, layer.in_proj.global_scale, nullptr,
                                                   e->mixer_width, e->z_offset, layer.out_norm, kEps,
                                                   fused_norm ? e->delta_normed_staged : nullptr, s));
            } else if (phase(e, "delta.scan")) {
                QWC_TRY(qwc_delta_decode_int8(layer.state, layer.state_scales, e->state_slots, e->dq, e->dk, e->dv,
                                              e->dalpha, e->dbeta, e->dkq, e->delta_out, c.state_slots, batch, s));
            }
            if (fused_norm) {
            } else if (staged && phase(e, "delta.norm")) {
                QWC_TRY(qwc_delta_gated_rmsnorm_split(e->delta_out, e->split_sums_wide, in_slices, e->mixer_width,
                                                      layer.in_proj.global_scale, e->z_offset, layer.out_norm, nullptr,
                                                      e->delta_normed_staged, batch, kEps, s));
            } else if (phase(e, "delta.norm")) {
                QWC_TRY(qwc_delta_gated_rmsnorm(e->delta_out, e->mixer_in + e->z_offset, layer.out_norm, e->delta_normed,
                                                batch, kEps, e->mixer_width, s));
            }
            if (staged) {
                hint_next_pair(e, layer.gate, layer.up);
                QWC_TRY(project_and_norm(e, layer.la_out, e->delta_normed_staged, e->mixer_out, layer.post_norm, batch,
                                         "gemm.la_out"));
            } else if (phase(e, "gemm.la_out")) {
                QWC_TRY(project(e, layer.la_out, e->delta_normed, e->mixer_out, batch));
            }
        } else {
            if (staged && phase(e, "gemm.attn_qkv")) {
                QWC_TRY(qwc_nvfp4_w4a16_split(layer.qkv.packed, layer.qkv.scales, e->normed_staged, e->split_sums_wide,
                                              layer.qkv.out_features, layer.qkv.in_features, batch, s));
                QWC_TRY(qwc_nvfp4_sum_slices(e->split_sums_wide,
                                             qwc_nvfp4_split_count(layer.qkv.out_features, layer.qkv.in_features),
                                             layer.qkv.global_scale, e->qkv_buf, batch, e->qkv_width, s));
            } else if (phase(e, "gemm.attn_qkv")) {
                QWC_TRY(project(e, layer.qkv, e->normed, e->qkv_buf, batch));
            }
            const int q_width = kQueryHeads * 2 * kHeadDim;
            if (phase(e, "attn.prepare")) {
                QWC_TRY(qwc_prepare_attention_decode_fp8_scaled(
                    e->qkv_buf, e->qkv_buf + q_width, e->qkv_buf + q_width + kKvHeads * kHeadDim, layer.q_norm,
                    layer.k_norm, e->cosine, e->sine, e->physical_blocks, e->block_offsets, layer.k_scale, layer.v_scale,
                    e->query, layer.k_cache, layer.v_cache, batch, c.kv_page_size, e->qkv_width, e->qkv_width,
                    e->qkv_width, kEps, s));
            }
            if (phase(e, "attn.decode")) {
                // The output gate is the second half of each head of [q | gate], which sits at the
                // front of the fused q|k|v row.
                QWC_TRY(qwc_paged_attention_packed_fp8_staged(
                    e->query, e->qkv_buf, layer.k_cache, layer.v_cache, e->block_tables, e->context_lengths,
                    layer.k_scale, layer.v_scale, staged ? nullptr : e->attention_out,
                    staged ? e->attention_out_staged : nullptr, e->attention_workspace, e->attention_workspace_bytes,
                    batch, 0, e->max_blocks, c.kv_page_size, e->qkv_width, e->partitions, 1.0f / 16.0f, s));
            }
            if (staged) {
                hint_next_pair(e, layer.gate, layer.up);
                QWC_TRY(project_and_norm(e, layer.o, e->attention_out_staged, e->mixer_out, layer.post_norm, batch,
                                         "gemm.attn_out"));
            } else if (phase(e, "gemm.attn_out")) {
                QWC_TRY(project(e, layer.o, e->attention_out, e->mixer_out, batch));
            }
        }
        const size_t trace_row = static_cast<size_t>(c.max_batch) * c.hidden;
        if (e->trace != nullptr && e->phase_filter == nullptr) {
            QWC_TRY(cudaMemcpyAsync(e->trace + (2 * index) * trace_row, e->mixer_out, trace_row * 2,
                                    cudaMemcpyDeviceToDevice, s));
        }
        if (!staged && phase(e, "norm")) {
            QWC_TRY(qwc_rmsnorm_bf16(e->mixer_out, e->residual, layer.post_norm, e->normed, batch, c.hidden, kEps, s));
        }
        if (phase(e, "gemm.mlp_gate_up") && staged) {
            hint_next_split(e, layer.down);
            QWC_TRY(qwc_nvfp4_swiglu_w4a16_staged(layer.gate.packed, layer.gate.scales, layer.up.packed,
                                                  layer.up.scales, e->normed_staged, nullptr, e->mlp_hidden_staged,
                                                  layer.gate.out_features, layer.gate.in_features, batch,
                                                  layer.gate.global_scale, layer.up.global_scale,
                                                  e->streamk_workspace, s));
        } else if (phase(e, "gemm.mlp_gate_up")) {
            __nv_bfloat16* target = e->mlp_hidden + static_cast<size_t>(c.split_rank) * layer.gate.out_features;
            QWC_TRY(qwc_nvfp4_swiglu_w4a16(layer.gate.packed, layer.gate.scales, layer.up.packed, layer.up.scales,
                                           e->normed, c.split_size > 1 ? target : e->mlp_hidden,
                                           layer.gate.out_features, layer.gate.in_features, batch,
                                           layer.gate.global_scale, layer.up.global_scale, s));
            if (c.split_size > 1 &&
                nccl_api().all_gather(target, e->mlp_hidden, static_cast<size_t>(layer.gate.out_features), 9, e->comm,
                                      s) != 0) {
                return cudaErrorUnknown;
            }
        }
        const __nv_bfloat16* next_norm = index + 1 < e->layers.size() ? e->layers[index + 1].input_norm : e->final_norm;
        if (staged) {
            if (index + 1 < e->layers.size()) {
                const Layer& following = e->layers[index + 1];
                hint_next_split(e, following.full ? following.qkv : following.in_proj);  // both run as K splits
            } else {
                (void)qwc_nvfp4_prefetch_next(e->lm_head, nullptr, nullptr, nullptr, e->vocab_local, c.hidden, 2);
            }
            QWC_TRY(project_and_norm(e, layer.down, e->mlp_hidden_staged, e->mlp_out, next_norm, batch, "gemm.mlp_down"));
        } else {
            if (phase(e, "gemm.mlp_down")) {
                QWC_TRY(project(e, layer.down, e->mlp_hidden, e->mlp_out, batch));
            }
            if (phase(e, "norm")) {
                QWC_TRY(qwc_rmsnorm_bf16(e->mlp_out, e->residual, next_norm, e->normed, batch, c.hidden, kEps, s));
            }
        }
        if (e->trace != nullptr && e->phase_filter == nullptr) {
            QWC_TRY(cudaMemcpyAsync(e->trace + (2 * index + 1) * trace_row, e->residual, trace_row * 2,
                                    cudaMemcpyDeviceToDevice, s));
        }
    }

    if (staged) {
        // One launch streams the vocabulary and keeps the best token of every row; a small second one
        // picks the winners and stores the device status word beside them.  Logits reach memory only
        // for a caller who asked for them.
        if (phase(e, "lm_head")) {
            QWC_TRY(qwc_fp8_lm_head_staged(e->lm_head, e->lm_head_scales, e->normed_staged,
                                           c.write_logits ? e->logits : nullptr, e->out_dev,
                                           e->out_dev + c.max_batch + 1, batch, c.hidden, e->vocab_local,
                                           e->streamk_workspace, s));
        }
        mark(e, "end");
        return 0;
    }
    if (phase(e, "lm_head")) {
        float* target = e->logits + static_cast<size_t>(c.split_rank) * e->vocab_local;
        QWC_TRY(qwc_fp8_lm_head_batched(e->lm_head, e->lm_head_scales, e->normed, c.split_size > 1 ? target : e->logits,
                                        batch, c.hidden, e->vocab_local, s));
        if (c.split_size > 1 &&
            nccl_api().all_gather(target, e->logits, static_cast<size_t>(e->vocab_local), /*ncclFloat32*/ 7, e->comm,
                                  s) != 0) {
            return cudaErrorUnknown;
        }
    }
    if (phase(e, "sample")) {
        QWC_TRY(qwc_argmax(e->logits, e->argmax_values, e->argmax_indices, e->out_dev, e->vocab_local * c.split_size, batch,
                           kArgmaxParts, s));
    }
    // The sticky status word of the bounded waits rides back with the sampled tokens: a step in
    // which a wait gave up has skipped stores, and its tokens must not be committed.
    if (e->phase_filter == nullptr) {
        QWC_TRY(qwc_device_status_copy(e->out_dev + c.max_batch + 1, s));
    }
    mark(e, "end");  // closes the last phase of the timeline
    return 0;
}

int launch_decode(qwc_engine* e, int batch) {
    if (!e->cfg.use_graph || e->profiling) {
        return decode_forward(e, batch);
    }
    if (!e->warmed[batch - 1]) {
        // The launchers do one-time set-up on first use (function attributes, the status
        // word's address): the first step of each batch size runs eagerly, later ones are
        // captured and replayed.
        e->warmed[batch - 1] = 1;
        return decode_forward(e, batch);
    }
    cudaGraphExec_t& exec = e->graphs[batch - 1];
    if (exec == nullptr) {
        cudaGraph_t graph = nullptr;
        QWC_TRY(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
        const int captured = decode_forward(e, batch);
        const cudaError_t ended = cudaStreamEndCapture(e->stream, &graph);  // always end: keep the stream usable
        if (captured != 0) {
            if (graph != nullptr) {
                cudaGraphDestroy(graph);
            }
            return captured;
        }
        QWC_TRY(ended);
        const cudaError_t made = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        QWC_TRY(made);
    }
    return cudaGraphLaunch(exec, e->stream);
}

// Every page id, state slot and table index reaches the device tables through an edit, so this is
// where they are bounded: a page beyond the pool never gets into a block table that the attention
// kernels (whose ABI carries no pool size) would follow.
int check_edits(const qwc_engine* e, const qwc_table_edit* edits, size_t count) {
    for (size_t i = 0; i < count; ++i) {
        const qwc_table_edit& edit = edits[i];
        if (edit.kind > 2 || edit.slot >= static_cast<uint32_t>(e->cfg.state_slots)) {
            return cudaErrorInvalidValue;
        }
        if (edit.kind == 0 && (edit.index >= static_cast<uint32_t>(e->max_blocks) ||
                               edit.value >= static_cast<uint32_t>(e->cfg.kv_pool_blocks))) {
            return cudaErrorInvalidValue;
        }
    }
    return 0;
}

int upload_inputs(qwc_engine* e, const uint32_t* row_slots, const uint32_t* tokens, const qwc_table_edit* edits,
                  size_t num_edits, int rows) {
    const qwc_engine_config& c = e->cfg;
    if (num_edits > static_cast<size_t>(e->max_edits)) {
        // A step that admitted long prompts carries more edits than the captured launch covers.
        const size_t early = num_edits - e->max_edits;
        QWC_TRY(qwc_engine_apply_edits(e, edits, early));
        edits += early;
        num_edits = e->max_edits;
    }
    std::memcpy(e->in_host, row_slots, sizeof(uint32_t) * rows);
    std::memcpy(e->in_host + c.max_batch, tokens, sizeof(uint32_t) * rows);
    auto* staged = reinterpret_cast<qwc_table_edit*>(e->in_host + 2 * c.max_batch);
    if (num_edits > 0) {
        std::memcpy(staged, edits, sizeof(qwc_table_edit) * num_edits);
    }
    for (size_t i = num_edits; i < static_cast<size_t>(e->max_edits); ++i) {
        staged[i] = {0xffffffffu, 0, 0, 0};  // out-of-range slot: ignored by the kernel
    }
    return cudaMemcpyAsync(e->in_dev, e->in_host, e->in_words * sizeof(uint32_t), cudaMemcpyHostToDevice, e->stream);
}

}  // namespace

extern "C" {

void qwc_engine_default_config(qwc_engine_config* config) {
    std::memset(config, 0, sizeof(*config));
    config->num_layers = 64;
    config->full_attention_interval = 4;
    config->hidden = 5120;
    config->intermediate = 17408;
    config->vocab = 151936;
    config->delta_value_heads = 32;
    config->kv_page_size = 16;
    config->max_batch = 32;
    config->max_context = 32768;
    config->kv_pool_blocks = 32 * 2048;
    config->state_slots = 33;
    config->seed = 0;
    config->split_rank = 0;
    config->split_size = 1;
    config->use_graph = 1;
    config->attention_partitions = 0;
    config->write_logits = 0;
    config->exchange = 0;
}

int qwc_engine_nccl_unique_id(void* unique_id_128) {
    if (!load_nccl()) {
        return -1;
    }
    return nccl_api().get_unique_id(unique_id_128) == 0 ? 0 : -2;
}

int qwc_engine_init_split(qwc_engine* e, const void* unique_id_128) {
    if (e == nullptr || e->cfg.split_size <= 1) {
        return cudaErrorInvalidValue;
    }
    if (!load_nccl()) {
        return -1;
    }
    // ncclCommInitRank takes the 128-byte id by value; on x86-64 a struct that large is passed
    // in memory, which is what a pointer-typed trampoline cannot express, so call through the
    // real prototype.
    using InitFn = int (*)(void**, int, NcclUniqueIdBytes, int);
    InitFn init = reinterpret_cast<InitFn>(dlsym(nccl_api().handle, "ncclCommInitRank"));
    NcclUniqueIdBytes id;
    std::memcpy(id.bytes, unique_id_128, sizeof(id.bytes));
    return init(&e->comm, e->cfg.split_size, id, e->cfg.split_rank) == 0 ? 0 : -2;
}

// The fused latency mode's set-up: every rank exports the inter-process handle of its exchange block,
// the caller distributes the handles (any host-side channel), and every rank maps the others' blocks.
// After that the step needs no library collective at all.
int qwc_engine_exchange_handle(qwc_engine* e, void* handle_64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    if (e == nullptr || handle_64 == nullptr || e->exchange_block == nullptr) {
        return cudaErrorInvalidValue;
    }
    cudaIpcMemHandle_t handle;
    QWC_TRY(cudaIpcGetMemHandle(&handle, e->exchange_block));
    std::memcpy(handle_64, &handle, sizeof(handle));
    return 0;
}

int qwc_engine_profile_waits(qwc_engine* e, int enable) {
    if (e == nullptr || e->wait_profile == nullptr) {
        return cudaErrorInvalidValue;
    }
    QWC_TRY(cudaStreamSynchronize(e->stream));
    e->profile_waits = enable != 0;
    // the row descriptions are baked into captured graphs: drop them
    for (cudaGraphExec_t& exec : e->graphs) {
        if (exec != nullptr) {
            cudaGraphExecDestroy(exec);
            exec = nullptr;
        }
    }
    return cudaMemset(e->wait_profile, 0, sizeof(unsigned long long) * QWC_EXCHANGE_MAX_INSTANCES);
}

int qwc_engine_exchange_waits(qwc_engine* e, unsigned long long* nanoseconds, int capacity) {
    if (e == nullptr || nanoseconds == nullptr || e->wait_profile == nullptr || capacity < QWC_EXCHANGE_MAX_INSTANCES) {
        return cudaErrorInvalidValue;
    }
    QWC_TRY(cudaStreamSynchronize(e->stream));
    QWC_TRY(cudaMemcpy(nanoseconds, e->wait_profile, sizeof(unsigned long long) * QWC_EXCHANGE_MAX_INSTANCES,
                       cudaMemcpyDeviceToHost));
    return cudaMemset(e->wait_profile, 0, sizeof(unsigned long long) * QWC_EXCHANGE_MAX_INSTANCES);
}

int qwc_engine_open_peers(qwc_engine* e, const void* handles, int count) {
    if (e == nullptr || handles == nullptr || e->exchange_block == nullptr || count != e->cfg.split_size ||
        e->peers_ready) {
        return cudaErrorInvalidValue;
    }
    const unsigned char* bytes = static_cast<const unsigned char*>(handles);
    for (int r = 0; r < count; ++r) {
        if (r == e->cfg.split_rank) {
            continue;
        }
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, bytes + static_cast<size_t>(r) * sizeof(handle), sizeof(handle));
        void* mapped = nullptr;
        QWC_TRY(cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess));
        e->opened_peers.push_back(mapped);
        e->exchange_blocks[r] = mapped;
    }
    e->peers_ready = true;
    return 0;
}

void qwc_engine_memory_usage(const qwc_engine* e, size_t* used, size_t* limit) {
    if (used != nullptr) {
        *used = e == nullptr ? 0 : e->memory_used;
    }
    if (limit != nullptr) {
        *limit = e == nullptr || e->memory_limit == SIZE_MAX ? 0 : e->memory_limit;
    }
}

int qwc_engine_create(const qwc_engine_config* config, qwc_engine** out) {
    if (config == nullptr || out == nullptr || config->num_layers <= 0 || config->full_attention_interval <= 0 ||
        config->hidden <= 0 || config->hidden % 256 != 0 || config->intermediate % 256 != 0 || config->vocab <= 0 ||
        config->max_batch <= 0 || config->max_batch > 32 || config->max_context <= 0 || config->kv_pool_blocks <= 0 ||
        config->state_slots < config->max_batch || config->split_size < 1 || config->split_rank < 0 ||
        config->split_rank >= config->split_size || (config->split_size > 1 && config->max_batch != 1) ||
        config->split_size > QWC_MAX_PEERS || (config->exchange != 0 && config->max_batch != 1)) {
        return cudaErrorInvalidValue;
    }
    qwc_shape shape = {config->delta_value_heads, config->kv_page_size};
    QWC_TRY(qwc_configure(&shape));

    auto* e = new qwc_engine;
    e->cfg = *config;
    const qwc_engine_config& c = e->cfg;
    int status = 0;
    auto fail = [&](int code) {
        qwc_engine_destroy(e);
        return code;
    };
    if ((status = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking)) != 0) {
        return fail(status);
    }
    if (c.memory_limit != 0) {
        // Other processes live on the card too: the budget asked for may not exist, and finding that
        // out half-way through the weights is worse than taking less (memory.rs:31-58).
        constexpr size_t kFreeMargin = size_t{512} << 20;  // what cudaMalloc's rounding adds up to
        size_t limit = static_cast<size_t>(c.memory_limit);
        size_t free_bytes = 0, total_bytes = 0;
        if (cudaMemGetInfo(&free_bytes, &total_bytes) == cudaSuccess && total_bytes > 0) {
            limit = std::min(limit, free_bytes > kFreeMargin ? free_bytes - kFreeMargin : size_t{0});
        }
        if (limit == 0) {
            return fail(cudaErrorMemoryAllocation);
        }
        e->memory_limit = limit;
    }

    e->v_heads = c.delta_value_heads;
    e->channels = 2 * kDeltaKeyHeads * kDeltaDim + e->v_heads * kDeltaDim;
    e->z_offset = e->channels;
    e->a_offset = e->z_offset + e->v_heads * kDeltaDim;
    e->b_offset = e->a_offset + e->v_heads;
    e->mixer_width = e->b_offset + e->v_heads;  // crates/qwc-engine/src/weights.rs:56-60
    e->qkv_width = kQueryHeads * 2 * kHeadDim + 2 * kKvHeads * kHeadDim;
    e->max_blocks = (c.max_context + c.kv_page_size - 1) / c.kv_page_size;
    e->max_edits = 2 * c.max_batch;
    e->vocab_local = c.vocab / c.split_size;
    const int split = c.split_size;
    if (e->mixer_width % split || e->qkv_width % split || c.hidden % split || c.intermediate % split ||
        c.vocab % split) {
        return fail(cudaErrorInvalidValue);
    }

    // ---- weights ----
    e->layers.resize(c.num_layers);
    int linear_index = 0, full_index = 0;
    const int mb = c.max_batch;
    for (int i = 0; i < c.num_layers && status == 0; ++i) {
        Layer& layer = e->layers[i];
        layer.full = (i + 1) % c.full_attention_interval == 0;  // crates/qwc-core/src/arch.rs:36-43
        layer.slot = layer.full ? full_index++ : linear_index++;
#define QWC_STEP(expr) \
    if (status == 0) { \
        status = (expr); \
    }
        QWC_STEP(make_norm(e, &layer.input_norm, c.hidden, i, 1, 0.0f, 0.02f));
        QWC_STEP(make_norm(e, &layer.post_norm, c.hidden, i, 2, 0.0f, 0.02f));
        QWC_STEP(make_linear(e, &layer.gate, c.intermediate, c.hidden, i, 10));
        QWC_STEP(make_linear(e, &layer.up, c.intermediate, c.hidden, i, 12));
        QWC_STEP(make_linear(e, &layer.down, c.hidden, c.intermediate, i, 14));
        if (!layer.full) {
            QWC_STEP(make_linear(e, &layer.in_proj, e->mixer_width, c.hidden, i, 16));
            QWC_STEP(make_linear(e, &layer.la_out, c.hidden, e->v_heads * kDeltaDim, i, 18));
            QWC_STEP(make_norm(e, &layer.conv_weight, static_cast<size_t>(e->channels) * 4, i, 20, 0.0f, 0.3f));
            QWC_STEP(make_norm(e, &layer.a_log, e->v_heads, i, 21, 0.0f, 0.5f));
            QWC_STEP(make_norm(e, &layer.dt_bias, e->v_heads, i, 22, 0.0f, 0.5f));
            QWC_STEP(make_norm(e, &layer.out_norm, kDeltaDim, i, 23, 1.0f, 0.05f));
            const size_t state_elems = static_cast<size_t>(c.state_slots) * e->v_heads * kDeltaDim * kDeltaDim;
            QWC_STEP(gpu_alloc_t(e, &layer.state, state_elems));
            QWC_STEP(gpu_alloc_t(e, &layer.state_scales, state_elems / kDeltaDim));
            QWC_STEP(gpu_alloc_t(e, &layer.conv_state, static_cast<size_t>(c.state_slots) * e->channels * 3));
            if (status == 0) {
                fill_bytes(e, layer.state, state_elems, tensor_seed(e, i, 30), 3);
                fill_uniform(e, layer.state_scales, state_elems / kDeltaDim, tensor_seed(e, i, 31), 0.0005f, 0.003f);
                fill_uniform(e, layer.conv_state, static_cast<size_t>(c.state_slots) * e->channels * 3,
                             tensor_seed(e, i, 32), -1.0f, 1.0f);
            }
        } else {
            QWC_STEP(make_linear(e, &layer.qkv, e->qkv_width, c.hidden, i, 40));
            QWC_STEP(make_linear(e, &layer.o, c.hidden, kQueryHeads * kHeadDim, i, 42));
            QWC_STEP(make_norm(e, &layer.q_norm, kHeadDim, i, 44, 0.0f, 0.05f));
            QWC_STEP(make_norm(e, &layer.k_norm, kHeadDim, i, 45, 0.0f, 0.05f));
            QWC_STEP(gpu_alloc_t(e, &layer.k_scale, kKvHeads));
            QWC_STEP(gpu_alloc_t(e, &layer.v_scale, kKvHeads));
            const size_t cache_bytes = static_cast<size_t>(c.kv_pool_blocks) * kKvHeads * c.kv_page_size * kHeadDim;
            QWC_STEP(gpu_alloc_t(e, &layer.k_cache, cache_bytes));
            QWC_STEP(gpu_alloc_t(e, &layer.v_cache, cache_bytes));
            if (status == 0) {
                fill_uniform(e, layer.k_scale, kKvHeads, tensor_seed(e, i, 46), 1.0f / 96.0f, 1.0f / 48.0f);
                fill_uniform(e, layer.v_scale, kKvHeads, tensor_seed(e, i, 47), 1.0f / 96.0f, 1.0f / 48.0f);
                fill_bytes(e, layer.k_cache, cache_bytes, tensor_seed(e, i, 48), 2);
                fill_bytes(e, layer.v_cache, cache_bytes, tensor_seed(e, i, 49), 2);
            }
        }
    }
    QWC_STEP(make_norm(e, &e->final_norm, c.hidden, c.num_layers, 1, 0.0f, 0.02f));
    const size_t table_bytes = static_cast<size_t>(c.vocab) * c.hidden;
    const size_t head_bytes = static_cast<size_t>(e->vocab_local) * c.hidden;
    QWC_STEP(gpu_alloc_t(e, &e->embed, table_bytes));
    QWC_STEP(gpu_alloc_t(e, &e->embed_scales, c.vocab));
    QWC_STEP(gpu_alloc_t(e, &e->lm_head, head_bytes));
    QWC_STEP(gpu_alloc_t(e, &e->lm_head_scales, e->vocab_local));
    if (status == 0) {
        fill_bytes(e, e->embed, table_bytes, tensor_seed(e, c.num_layers, 50), 2);
        fill_uniform(e, e->embed_scales, c.vocab, tensor_seed(e, c.num_layers, 51), 0.0001f, 0.0003f);
        fill_bytes(e, e->lm_head, head_bytes, tensor_seed(e, c.num_layers, 52, true), 2);
        fill_uniform(e, e->lm_head_scales, e->vocab_local, tensor_seed(e, c.num_layers, 53, true), 0.0001f, 0.0003f);
    }

    // ---- activations ----
    QWC_STEP(gpu_alloc_t(e, &e->residual, static_cast<size_t>(mb) * c.hidden, true));
    QWC_STEP(gpu_alloc_t(e, &e->normed, static_cast<size_t>(mb) * c.hidden, true));
    QWC_STEP(gpu_alloc_t(e, &e->mixer_in, static_cast<size_t>(mb) * e->mixer_width, true));
    QWC_STEP(gpu_alloc_t(e, &e->qkv_buf, static_cast<size_t>(mb) * e->qkv_width, true));
    QWC_STEP(gpu_alloc_t(e, &e->query, static_cast<size_t>(mb) * kQueryHeads * kHeadDim, true));
    QWC_STEP(gpu_alloc_t(e, &e->attention_out, static_cast<size_t>(mb) * kQueryHeads * kHeadDim, true));
    QWC_STEP(gpu_alloc_t(e, &e->delta_normed, static_cast<size_t>(mb) * e->v_heads * kDeltaDim, true));
    QWC_STEP(gpu_alloc_t(e, &e->mixer_out, static_cast<size_t>(mb) * c.hidden, true));
    QWC_STEP(gpu_alloc_t(e, &e->mlp_hidden, static_cast<size_t>(mb) * c.intermediate, true));
    QWC_STEP(gpu_alloc_t(e, &e->mlp_out, static_cast<size_t>(mb) * c.hidden, true));
    {
        // staged copies are sized for 32 padded rows, whatever the batch
        int widest = c.hidden > c.intermediate ? c.hidden : c.intermediate;
        (void)widest;
        QWC_STEP(gpu_alloc(e, &e->normed_staged, static_cast<size_t>(c.hidden) * 32 * 2, true));
        QWC_STEP(gpu_alloc(e, &e->delta_normed_staged, static_cast<size_t>(e->v_heads) * kDeltaDim * 32 * 2, true));
        QWC_STEP(gpu_alloc(e, &e->attention_out_staged, static_cast<size_t>(kQueryHeads) * kHeadDim * 32 * 2, true));
        QWC_STEP(gpu_alloc(e, &e->mlp_hidden_staged, static_cast<size_t>(c.intermediate) * 32 * 2, true));
        QWC_STEP(gpu_alloc(e, &e->streamk_workspace, qwc_streamk_workspace_bytes(), true));
        QWC_STEP(gpu_alloc_t(e, &e->split_sums, static_cast<size_t>(16) * 32 * c.hidden, true));
        const int wide = e->mixer_width > e->qkv_width ? e->mixer_width : e->qkv_width;
        QWC_STEP(gpu_alloc_t(e, &e->split_sums_wide, static_cast<size_t>(16) * 32 * wide, true));
        if (c.exchange != 0) {
            // one allocation, so that one inter-process handle covers every row: [wide | hidden A |
            // hidden B | gate and up | candidates].  Consecutive exchanges of a step never share a row.
            size_t at = 0;
            e->row_wide = at;
            at += qwc_exchange_row_bytes(wide);
            e->row_hidden[0] = at;
            at += qwc_exchange_row_bytes(c.hidden);
            e->row_hidden[1] = at;
            at += qwc_exchange_row_bytes(c.hidden);
            e->row_swiglu = at;
            at += qwc_exchange_row_bytes(2 * c.intermediate);
            e->row_candidates = at;
            at += qwc_exchange_candidate_bytes(c.split_size);
            e->exchange_bytes = at;
            QWC_STEP(gpu_alloc_t(e, &e->exchange_block, at, true));
            QWC_STEP(gpu_alloc_t(e, &e->epoch, 4, true));
            QWC_STEP(gpu_alloc_t(e, &e->wait_profile, QWC_EXCHANGE_MAX_INSTANCES, true));
            e->exchange_blocks[c.split_rank] = e->exchange_block;
            e->peers_ready = c.split_size == 1;  // a single rank exchanges with itself
        }
    }
    QWC_STEP(gpu_alloc_t(e, &e->dq, static_cast<size_t>(mb) * kDeltaKeyHeads * kDeltaDim, true));
    QWC_STEP(gpu_alloc_t(e, &e->dk, static_cast<size_t>(mb) * kDeltaKeyHeads * kDeltaDim, true));
    QWC_STEP(gpu_alloc_t(e, &e->dv, static_cast<size_t>(mb) * e->v_heads * kDeltaDim, true));
    QWC_STEP(gpu_alloc_t(e, &e->dalpha, static_cast<size_t>(mb) * e->v_heads, true));
    QWC_STEP(gpu_alloc_t(e, &e->dbeta, static_cast<size_t>(mb) * e->v_heads, true));
    QWC_STEP(gpu_alloc_t(e, &e->dkq, static_cast<size_t>(mb) * kDeltaKeyHeads, true));
    QWC_STEP(gpu_alloc_t(e, &e->delta_out, static_cast<size_t>(mb) * e->v_heads * kDeltaDim, true));
    QWC_STEP(gpu_alloc_t(e, &e->logits, static_cast<size_t>(mb) * c.vocab, true));
    QWC_STEP(gpu_alloc_t(e, &e->argmax_values, static_cast<size_t>(mb) * kArgmaxParts, true));
    QWC_STEP(gpu_alloc_t(e, &e->argmax_indices, static_cast<size_t>(mb) * kArgmaxParts, true));

    // Attention partitions: the cap on how many tasks one row may be cut into (the kernel sizes
    // the tasks on the device from the contexts it finds).  Spans of at least 128 tokens, at most
    // 4096 partial slots per head.
    if (c.attention_partitions > 0) {
        e->partitions = c.attention_partitions;
    } else {
        const int want = (c.max_context + 127) / 128;
        int most = 4096 / mb;
        most = most < 8 ? 8 : most;
        e->partitions = want < most ? want : most;
        if (e->partitions < 1) {
            e->partitions = 1;
        }
    }
    e->attention_workspace_bytes = qwc_paged_attention_packed_workspace_bytes(mb, e->partitions);
    QWC_STEP(gpu_alloc(e, &e->attention_workspace, e->attention_workspace_bytes + 16, true));

    // ---- tables ----
    QWC_STEP(gpu_alloc_t(e, &e->seq_tokens, c.state_slots, true));
    QWC_STEP(gpu_alloc_t(e, &e->seq_blocks, static_cast<size_t>(c.state_slots) * e->max_blocks, true));
    QWC_STEP(gpu_alloc_t(e, &e->state_slots, mb, true));
    QWC_STEP(gpu_alloc_t(e, &e->positions, mb, true));
    QWC_STEP(gpu_alloc_t(e, &e->context_lengths, mb, true));
    QWC_STEP(gpu_alloc_t(e, &e->physical_blocks, mb, true));
    QWC_STEP(gpu_alloc_t(e, &e->block_offsets, mb, true));
    QWC_STEP(gpu_alloc_t(e, &e->block_tables, static_cast<size_t>(mb) * e->max_blocks, true));
    QWC_STEP(gpu_alloc_t(e, &e->block_table_offsets, mb + 1, true));
    QWC_STEP(gpu_alloc_t(e, &e->row_count, 1, true));
    QWC_STEP(gpu_alloc_t(e, &e->cosine, static_cast<size_t>(mb) * kRopeDim, true));
    QWC_STEP(gpu_alloc_t(e, &e->sine, static_cast<size_t>(mb) * kRopeDim, true));
    QWC_STEP(gpu_alloc_t(e, &e->rope_table, static_cast<size_t>(c.max_context) * 2 * kRopeDim));
    if (status == 0) {
        // crates/qwc-engine/src/executor.rs:1953-1958, built once for every position
        std::vector<uint16_t> table(static_cast<size_t>(c.max_context) * 2 * kRopeDim);
        auto to_bf16 = [](float x) {
            uint32_t bits;
            std::memcpy(&bits, &x, 4);
            if (x != x) {
                return static_cast<uint16_t>(0x7fc0);
            }
            return static_cast<uint16_t>((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
        };
        std::vector<float> inverse(kRopeDim);
        for (int d = 0; d < kRopeDim; ++d) {
            inverse[d] = powf(kRopeTheta, -(2.0f * static_cast<float>(d % (kRopeDim / 2))) / static_cast<float>(kRopeDim));
        }
        for (int position = 0; position < c.max_context; ++position) {
            for (int d = 0; d < kRopeDim; ++d) {
                const float angle = static_cast<float>(position) * inverse[d];
                table[(static_cast<size_t>(position) * 2 + 0) * kRopeDim + d] = to_bf16(cosf(angle));
                table[(static_cast<size_t>(position) * 2 + 1) * kRopeDim + d] = to_bf16(sinf(angle));
            }
        }
        status = cudaMemcpyAsync(e->rope_table, table.data(), table.size() * 2, cudaMemcpyHostToDevice, e->stream);
        if (status == 0) {
            status = cudaStreamSynchronize(e->stream);
        }
    }

    // ---- step staging ----
    e->in_words = 2 * static_cast<size_t>(mb) + 4 * static_cast<size_t>(e->max_edits);
    if (status == 0) {
        status = cudaMallocHost(reinterpret_cast<void**>(&e->in_host), e->in_words * sizeof(uint32_t));
    }
    if (status == 0) {
        status = cudaMallocHost(reinterpret_cast<void**>(&e->out_host), (mb + 2) * sizeof(uint32_t));
    }
    QWC_STEP(gpu_alloc_t(e, &e->in_dev, e->in_words, true));
    QWC_STEP(gpu_alloc_t(e, &e->out_dev, mb + 2, true));
#undef QWC_STEP
    if (status == 0) {
        status = cudaStreamSynchronize(e->stream);
    }
    if (status != 0) {
        return fail(status);
    }
    e->graphs.assign(mb, nullptr);
    e->warmed.assign(mb, 0);
    e->last_token.assign(c.state_slots, 0);
    *out = e;
    return 0;
}

void qwc_engine_destroy(qwc_engine* e) {
    if (e == nullptr) {
        return;
    }
    if (e->stream != nullptr) {
        cudaStreamSynchronize(e->stream);
    }
    for (cudaGraphExec_t exec : e->graphs) {
        if (exec != nullptr) {
            cudaGraphExecDestroy(exec);
        }
    }
    if (e->comm != nullptr && nccl_api().comm_destroy != nullptr) {
        nccl_api().comm_destroy(e->comm);
    }
    for (void* peer : e->opened_peers) {
        cudaIpcCloseMemHandle(peer);
    }
    for (void* p : e->allocations) {
        cudaFree(p);
    }
    if (e->in_host != nullptr) {
        cudaFreeHost(e->in_host);
    }
    if (e->out_host != nullptr) {
        cudaFreeHost(e->out_host);
    }
    if (e->stream != nullptr) {
        cudaStreamDestroy(e->stream);
    }
    delete e;
}

qwc_stream qwc_engine_stream(qwc_engine* e) { return e->stream; }

int qwc_engine_tensor(qwc_engine* e, const char* name, int layer, void** device_ptr, size_t* bytes) {
    if (e == nullptr || name == nullptr || device_ptr == nullptr || bytes == nullptr) {
        return 1;
    }
    const qwc_engine_config& c = e->cfg;
    const std::string n(name);
    const size_t mb = c.max_batch;
    auto set = [&](const void* p, size_t size) {
        *device_ptr = const_cast<void*>(p);
        *bytes = size;
        return p == nullptr ? 1 : 0;
    };
    auto linear = [&](const LinearW& w, bool scales) {
        return scales ? set(w.scales, scale_storage(w.out_features, w.in_features))
                      : set(w.packed, static_cast<size_t>(w.out_features) * w.in_features / 2);
    };
    // global tensors
    if (n == "final_norm") return set(e->final_norm, c.hidden * 2);
    if (n == "embed") return set(e->embed, static_cast<size_t>(c.vocab) * c.hidden);
    if (n == "embed_scales") return set(e->embed_scales, static_cast<size_t>(c.vocab) * 4);
    if (n == "lm_head") return set(e->lm_head, static_cast<size_t>(e->vocab_local) * c.hidden);
    if (n == "lm_head_scales") return set(e->lm_head_scales, static_cast<size_t>(e->vocab_local) * 4);
    if (n == "logits") return set(e->logits, mb * c.vocab * 4);
    if (n == "normed") return set(e->normed, mb * c.hidden * 2);
    if (n == "residual") return set(e->residual, mb * c.hidden * 2);
    if (n == "mixer_out") return set(e->mixer_out, mb * c.hidden * 2);
    if (n == "seq_tokens") return set(e->seq_tokens, static_cast<size_t>(c.state_slots) * 4);
    if (n == "seq_blocks") return set(e->seq_blocks, static_cast<size_t>(c.state_slots) * e->max_blocks * 4);
    if (n == "block_tables") return set(e->block_tables, mb * e->max_blocks * 4);
    if (n == "context_lengths") return set(e->context_lengths, mb * 4);
    if (n == "rope_table") return set(e->rope_table, static_cast<size_t>(c.max_context) * 2 * kRopeDim * 2);
    if (n == "trace") return set(e->trace, static_cast<size_t>(c.num_layers) * 2 * mb * c.hidden * 2);
    if (layer < 0 || layer >= c.num_layers) {
        return 1;
    }
    const Layer& l = e->layers[layer];
    if (n == "input_norm") return set(l.input_norm, c.hidden * 2);
    if (n == "post_norm") return set(l.post_norm, c.hidden * 2);
    if (n == "gate.packed") return linear(l.gate, false);
    if (n == "gate.scales") return linear(l.gate, true);
    if (n == "up.packed") return linear(l.up, false);
    if (n == "up.scales") return linear(l.up, true);
    if (n == "down.packed") return linear(l.down, false);
    if (n == "down.scales") return linear(l.down, true);
    if (!l.full) {
        const size_t state_elems = static_cast<size_t>(c.state_slots) * e->v_heads * kDeltaDim * kDeltaDim;
        if (n == "in_proj.packed") return linear(l.in_proj, false);
        if (n == "in_proj.scales") return linear(l.in_proj, true);
        if (n == "la_out.packed") return linear(l.la_out, false);
        if (n == "la_out.scales") return linear(l.la_out, true);
        if (n == "conv_weight") return set(l.conv_weight, static_cast<size_t>(e->channels) * 4 * 2);
        if (n == "a_log") return set(l.a_log, e->v_heads * 2);
        if (n == "dt_bias") return set(l.dt_bias, e->v_heads * 2);
        if (n == "out_norm") return set(l.out_norm, kDeltaDim * 2);
        if (n == "state") return set(l.state, state_elems);
        if (n == "state_scales") return set(l.state_scales, state_elems / kDeltaDim * 4);
        if (n == "conv_state") return set(l.conv_state, static_cast<size_t>(c.state_slots) * e->channels * 3 * 4);
    } else {
        const size_t cache_bytes = static_cast<size_t>(c.kv_pool_blocks) * kKvHeads * c.kv_page_size * kHeadDim;
        if (n == "qkv.packed") return linear(l.qkv, false);
        if (n == "qkv.scales") return linear(l.qkv, true);
        if (n == "o.packed") return linear(l.o, false);
        if (n == "o.scales") return linear(l.o, true);
        if (n == "q_norm") return set(l.q_norm, kHeadDim * 2);
        if (n == "k_norm") return set(l.k_norm, kHeadDim * 2);
        if (n == "k_scale") return set(l.k_scale, kKvHeads * 4);
        if (n == "v_scale") return set(l.v_scale, kKvHeads * 4);
        if (n == "k_cache") return set(l.k_cache, cache_bytes);
        if (n == "v_cache") return set(l.v_cache, cache_bytes);
    }
    return 1;
}

int qwc_engine_trace_layers(qwc_engine* e, int enable) {
    if (e == nullptr) {
        return cudaErrorInvalidValue;
    }
    QWC_TRY(cudaStreamSynchronize(e->stream));
    // The copies are part of the step's launch sequence: graphs captured without them are dropped.
    for (cudaGraphExec_t& exec : e->graphs) {
        if (exec != nullptr) {
            cudaGraphExecDestroy(exec);
            exec = nullptr;
        }
    }
    if (enable != 0 && e->trace == nullptr) {
        const size_t count = static_cast<size_t>(e->cfg.num_layers) * 2 * e->cfg.max_batch * e->cfg.hidden;
        QWC_TRY(gpu_alloc_t(e, &e->trace, count, true));
        QWC_TRY(cudaStreamSynchronize(e->stream));
    } else if (enable == 0) {
        e->trace = nullptr;  // the buffer stays with the engine's allocations until it is destroyed
    }
    return 0;
}

int qwc_engine_read(qwc_engine* e, const char* name, int layer, void* host, size_t bytes) {
    void* device = nullptr;
    size_t size = 0;
    if (host == nullptr || qwc_engine_tensor(e, name, layer, &device, &size) != 0 || size != bytes) {
        return cudaErrorInvalidValue;
    }
    QWC_TRY(cudaStreamSynchronize(e->stream));
    return cudaMemcpy(host, device, bytes, cudaMemcpyDeviceToHost);
}

int qwc_engine_write(qwc_engine* e, const char* name, int layer, const void* host, size_t bytes) {
    void* device = nullptr;
    size_t size = 0;
    if (host == nullptr || qwc_engine_tensor(e, name, layer, &device, &size) != 0 || size != bytes) {
        return cudaErrorInvalidValue;
    }
    QWC_TRY(cudaStreamSynchronize(e->stream));
    return cudaMemcpy(device, host, bytes, cudaMemcpyHostToDevice);
}

void qwc_engine_traffic(const qwc_engine* e, int rows, double context_tokens, qwc_step_traffic* out) {
    std::memset(out, 0, sizeof(*out));
    // one GPU: the head samples in its own epilogue and one small kernel picks the winners
    int gemv = 0, kernels = 3 /*table edits + pack*/ + 1 /*embed*/ + 1 /*norm*/ + 1 /*lm_head*/ +
                            (e->cfg.split_size == 1 ? 1 : 2) /*sampling*/;
    double gemv_bytes = 0.0;
    for (const Layer& l : e->layers) {
        gemv_bytes += static_cast<double>(l.gate.weight_bytes() + l.up.weight_bytes() + l.down.weight_bytes());
        gemv += 2;
        kernels += 2 + 2;  // two projections, two norms
        if (!l.full) {
            gemv_bytes += static_cast<double>(l.in_proj.weight_bytes() + l.la_out.weight_bytes());
            gemv += 2;
            kernels += 2 + 3 - (e->cfg.split_size == 1 && qwc_delta_decode_fuses_norm(rows) ? 1 : 0);
            // int8 state and fp32 row scales, read and written (delta_net.rs traffic_bytes analogue)
            out->state_bytes += 2.0 * rows * e->v_heads * (kDeltaDim * kDeltaDim + kDeltaDim * 4.0);
        } else {
            gemv_bytes += static_cast<double>(l.qkv.weight_bytes() + l.o.weight_bytes());
            gemv += 2;
            kernels += 2 + 2 + (e->partitions > 1 ? 1 : 0) + (e->cfg.split_size == 1 ? 1 : 0 /*slice sum*/);
            out->kv_bytes += context_tokens * 2.0 * kKvHeads * kHeadDim;
        }
    }
    if (e->cfg.exchange != 0) {
        // fused latency mode: epoch, edits + pack, embed, norm, head, sampling; per layer the SwiGLU pair,
        // its combine, down and its norm, and six kernels of the mixer (one more when attention merges)
        kernels = 1 + 3 + 1 + 1 + 1 + 1;
        for (const Layer& l : e->layers) {
            kernels += 4 + 6 + (l.full && e->partitions > 1 ? 1 : 0);
        }
    }
    const double head = static_cast<double>(e->vocab_local) * e->cfg.hidden + e->vocab_local * 4.0;
    out->weight_bytes = gemv_bytes + head;
    out->gemv_bytes_per_step = gemv_bytes;
    out->gemv_launches_per_step = gemv;
    out->kernel_launches_per_step = kernels;
}

namespace {
LinearW* find_linear(qwc_engine* e, const char* name, int layer) {
    if (e == nullptr || name == nullptr || layer < 0 || layer >= e->cfg.num_layers) {
        return nullptr;
    }
    Layer& l = e->layers[layer];
    const std::string n(name);
    if (n == "gate") return &l.gate;
    if (n == "up") return &l.up;
    if (n == "down") return &l.down;
    if (!l.full && n == "in_proj") return &l.in_proj;
    if (!l.full && n == "la_out") return &l.la_out;
    if (l.full && n == "qkv") return &l.qkv;
    if (l.full && n == "o") return &l.o;
    return nullptr;
}
}  // namespace

// The fp32 global divisor of an NVFP4 matrix (the checkpoint's weight_global_scale,
// crates/qwc-engine/src/weights.rs:470-476): synthetic weights carry 1; a loader sets the real one.
// The value is a launch argument, so captured graphs are dropped.
int qwc_engine_set_weight_global_scale(qwc_engine* e, const char* name, int layer, float value) {
    LinearW* w = find_linear(e, name, layer);
    if (w == nullptr || !(value > 0.0f) || !std::isfinite(value)) {
        return cudaErrorInvalidValue;
    }
    QWC_TRY(cudaStreamSynchronize(e->stream));
    w->global_scale = value;
    for (cudaGraphExec_t& exec : e->graphs) {
        if (exec != nullptr) {
            cudaGraphExecDestroy(exec);
            exec = nullptr;
        }
    }
    return 0;
}

int qwc_engine_weight_global_scale(qwc_engine* e, const char* name, int layer, float* value) {
    LinearW* w = find_linear(e, name, layer);
    if (w == nullptr || value == nullptr) {
        return cudaErrorInvalidValue;
    }
    *value = w->global_scale;
    return 0;
}

int qwc_engine_apply_edits(qwc_engine* e, const qwc_table_edit* edits, size_t count) {
    if (e == nullptr || (count > 0 && edits == nullptr)) {
        return cudaErrorInvalidValue;
    }
    if (count == 0) {
        return 0;
    }
    QWC_TRY(check_edits(e, edits, count));
    qwc_table_edit* staged = nullptr;
    QWC_TRY(cudaMalloc(reinterpret_cast<void**>(&staged), count * sizeof(qwc_table_edit)));
    int status = cudaMemcpyAsync(staged, edits, count * sizeof(qwc_table_edit), cudaMemcpyHostToDevice, e->stream);
    if (status == 0) {
        status = qwc_page_table_apply(e->seq_tokens, e->seq_blocks, staged, static_cast<int>(count), e->cfg.state_slots,
                                      e->max_blocks, e->stream);
    }
    const int synced = cudaStreamSynchronize(e->stream);
    cudaFree(staged);
    return status != 0 ? status : synced;
}

// Executor::copy_kv_block (executor.rs:825-835): the tail of a cached prefix lies in an incomplete page
// to which the new sequence will append, so it gets a copy of its own in every attention layer.
int qwc_engine_copy_kv_block(qwc_engine* e, uint32_t from, uint32_t to) {
    if (e == nullptr || from >= static_cast<uint32_t>(e->cfg.kv_pool_blocks) ||
        to >= static_cast<uint32_t>(e->cfg.kv_pool_blocks)) {
        return cudaErrorInvalidValue;
    }
    if (from == to) {
        return 0;
    }
    const size_t page = static_cast<size_t>(kKvHeads) * e->cfg.kv_page_size * kHeadDim;
    for (const Layer& layer : e->layers) {
        if (!layer.full) {
            continue;
        }
        QWC_TRY(cudaMemcpyAsync(layer.k_cache + to * page, layer.k_cache + from * page, page, cudaMemcpyDeviceToDevice,
                                e->stream));
        QWC_TRY(cudaMemcpyAsync(layer.v_cache + to * page, layer.v_cache + from * page, page, cudaMemcpyDeviceToDevice,
                                e->stream));
    }
    return 0;
}

int qwc_engine_decode(qwc_engine* e, const uint32_t* row_slots, const uint32_t* tokens, const qwc_table_edit* edits,
                      size_t num_edits, int rows, uint32_t* sampled) {
    if (e == nullptr || row_slots == nullptr || tokens == nullptr || sampled == nullptr || rows <= 0 ||
        rows > e->cfg.max_batch || (num_edits > 0 && edits == nullptr)) {
        return cudaErrorInvalidValue;
    }
    QWC_TRY(check_edits(e, edits, num_edits));
    QWC_TRY(upload_inputs(e, row_slots, tokens, edits, num_edits, rows));
    QWC_TRY(launch_decode(e, rows));
    QWC_TRY(cudaMemcpyAsync(e->out_host, e->out_dev, (e->cfg.max_batch + 2) * sizeof(uint32_t), cudaMemcpyDeviceToHost,
                            e->stream));
    QWC_TRY(cudaStreamSynchronize(e->stream));
    std::memcpy(sampled, e->out_host, sizeof(uint32_t) * rows);
    const uint32_t pack_status = e->out_host[e->cfg.max_batch];
    const uint32_t wait_status = e->out_host[e->cfg.max_batch + 1];
    if (pack_status != 0) {
        return 0x1000 + static_cast<int>(pack_status);
    }
    return wait_status == 0 ? 0 : 0x4000 + static_cast<int>(wait_status);
}

int qwc_engine_replay(qwc_engine* e, int rows) {
    if (e == nullptr || rows <= 0 || rows > e->cfg.max_batch) {
        return cudaErrorInvalidValue;
    }
    // Neutralise the staged edits so a replay does not advance the token counts again.
    auto* staged = reinterpret_cast<qwc_table_edit*>(e->in_host + 2 * e->cfg.max_batch);
    bool dirty = false;
    for (int i = 0; i < e->max_edits; ++i) {
        if (staged[i].slot != 0xffffffffu) {
            staged[i] = {0xffffffffu, 0, 0, 0};
            dirty = true;
        }
    }
    if (dirty) {
        QWC_TRY(cudaMemcpyAsync(e->in_dev, e->in_host, e->in_words * sizeof(uint32_t), cudaMemcpyHostToDevice,
                                e->stream));
    }
    return launch_decode(e, rows);
}

int qwc_engine_profile_step(qwc_engine* e, int rows, qwc_phase_time* phases, int max_phases) {
    if (e == nullptr || rows <= 0 || rows > e->cfg.max_batch || phases == nullptr || max_phases <= 0) {
        return -1;
    }
    e->profiling = true;
    e->marks.clear();
    const int status = decode_forward(e, rows);
    e->profiling = false;
    cudaStreamSynchronize(e->stream);
    int count = 0;
    if (status == 0) {
        for (size_t i = 0; i + 1 < e->marks.size(); ++i) {
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, e->marks[i].event, e->marks[i + 1].event);
            int found = -1;
            for (int j = 0; j < count; ++j) {
                if (std::strcmp(phases[j].label, e->marks[i].label) == 0) {
                    found = j;
                }
            }
            if (found < 0 && count < max_phases) {
                found = count++;
                std::snprintf(phases[found].label, sizeof(phases[found].label), "%s", e->marks[i].label);
                phases[found].milliseconds = 0.0f;
                phases[found].launches = 0;
            }
            if (found >= 0) {
                phases[found].milliseconds += ms;
                phases[found].launches += 1;
            }
        }
    }
    for (Phase& mark_entry : e->marks) {
        cudaEventDestroy(mark_entry.event);
    }
    e->marks.clear();
    return status == 0 ? count : -status;
}

int qwc_engine_time_phases(qwc_engine* e, int rows, const char* label_prefix, int replays, float* milliseconds,
                           int* launches) {
    if (e == nullptr || rows <= 0 || rows > e->cfg.max_batch || label_prefix == nullptr || replays <= 0 ||
        milliseconds == nullptr || !e->warmed[rows - 1]) {
        return -1;
    }
    // A graph of only the selected phases, on the buffers the last real step left behind.
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    e->phase_filter = label_prefix;
    e->filtered_launches = 0;
    QWC_TRY(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    const int captured = decode_forward(e, rows);
    const cudaError_t ended = cudaStreamEndCapture(e->stream, &graph);
    e->phase_filter = nullptr;
    if (launches != nullptr) {
        *launches = e->filtered_launches;
    }
    if (captured != 0 || ended != cudaSuccess || e->filtered_launches == 0) {
        if (graph != nullptr) {
            cudaGraphDestroy(graph);
        }
        return captured != 0 ? captured : (ended != cudaSuccess ? static_cast<int>(ended) : -2);
    }
    const cudaError_t made = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    QWC_TRY(made);
    cudaEvent_t begin, end;
    cudaEventCreate(&begin);
    cudaEventCreate(&end);
    int status = 0;
    for (int i = 0; i < 2 && status == 0; ++i) {
        status = cudaGraphLaunch(exec, e->stream);
    }
    cudaEventRecord(begin, e->stream);
    for (int i = 0; i < replays && status == 0; ++i) {
        status = cudaGraphLaunch(exec, e->stream);
    }
    cudaEventRecord(end, e->stream);
    const cudaError_t synced = cudaStreamSynchronize(e->stream);
    float total = 0.0f;
    cudaEventElapsedTime(&total, begin, end);
    *milliseconds = total / static_cast<float>(replays);
    cudaEventDestroy(begin);
    cudaEventDestroy(end);
    cudaGraphExecDestroy(exec);
    return status != 0 ? status : static_cast<int>(synced);
}

int qwc_worker_step(qwc_engine* e, qwc_scheduler* scheduler, uint32_t eos_token, size_t* num_decoded,
                    qwc_completion* completed, size_t max_completed, size_t* num_completed) {
    using namespace qwc::runtime;
    *num_decoded = 0;
    *num_completed = 0;
    Scheduler& sched = scheduler->scheduler;
    Batch batch;
    bool has_batch = false;
    const SchedulerError planned = sched.next_batch(&batch, &has_batch);
    if (planned != SchedulerError::None) {
        return 0x2000 + static_cast<int>(planned);
    }
    if (!has_batch) {
        return 0;
    }
    // Every error from here to the launch rolls the plan back (serve.rs:828-835,980-987).
    auto abort_with = [&](int code) {
        sched.abort_batch();
        // the rollback produced edits of its own; the device copy must follow
        const std::vector<TableEdit> undo = sched.cache_mut().drain_edits();
        qwc_engine_apply_edits(e, reinterpret_cast<const qwc_table_edit*>(undo.data()), undo.size());
        return code;
    };
    BatchLayout layout;
    SeqId offender = 0;
    const LayoutError laid = BatchLayout::build(batch, sched.cache(), &layout, &offender);
    if (laid != LayoutError::None) {
        return abort_with(0x3000 + static_cast<int>(laid));
    }
    const std::vector<TableEdit> edits = sched.cache_mut().drain_edits();
    std::vector<SeqId> stopped;
    if (!batch.decode.empty()) {
        const int rows = static_cast<int>(batch.decode.size());
        if (rows > e->cfg.max_batch) {
            return abort_with(cudaErrorInvalidValue);
        }
        std::vector<uint32_t> slots(rows), tokens(rows), sampled(rows);
        for (int row = 0; row < rows; ++row) {
            slots[row] = layout.state_slots[row];
            tokens[row] = e->last_token[slots[row]];
        }
        const int status = qwc_engine_decode(e, slots.data(), tokens.data(),
                                             reinterpret_cast<const qwc_table_edit*>(edits.data()), edits.size(), rows,
                                             sampled.data());
        if (status != 0) {
            return abort_with(status);
        }
        for (int row = 0; row < rows; ++row) {
            e->last_token[slots[row]] = sampled[row];
            if (sampled[row] == eos_token) {
                stopped.push_back(batch.decode[row]);
            }
        }
        *num_decoded = rows;
    } else if (!edits.empty()) {
        const int status =
            qwc_engine_apply_edits(e, reinterpret_cast<const qwc_table_edit*>(edits.data()), edits.size());
        if (status != 0) {
            return abort_with(status);
        }
    }
    // Prompt tokens of a prefill chunk are taken as already resident: seed the first input token.
    for (const PrefillChunk& chunk : batch.prefill) {
        const Sequence* seq = sched.cache().sequence(chunk.id);
        if (seq != nullptr) {
            e->last_token[seq->state_slot] = (chunk.id * 7919u + 1000u) % static_cast<uint32_t>(e->cfg.vocab);
        }
    }
    std::vector<Completion> done;
    const SchedulerError finished = sched.complete_batch(stopped, &done);
    if (finished != SchedulerError::None) {
        return 0x2000 + static_cast<int>(finished);
    }
    // releases of finished sequences reach the device with the next step's edits
    *num_completed = done.size();
    for (size_t i = 0; i < done.size() && i < max_completed; ++i) {
        completed[i] = {done[i].id, static_cast<uint32_t>(done[i].generated_tokens),
                        static_cast<uint32_t>(done[i].reason)};
    }
    return 0;
}

// A qwc_execute_fn over this engine, for the token-level worker loop.
int qwc_engine_execute_step(void* engine, const qwc_step_view* step, uint32_t* sampled) {
    auto* e = static_cast<qwc_engine*>(engine);
    if (e == nullptr || step == nullptr || sampled == nullptr || step->num_decode > step->num_sequences) {
        return cudaErrorInvalidValue;
    }
    const int rows = static_cast<int>(step->num_decode);
    if (rows > e->cfg.max_batch) {
        return cudaErrorInvalidValue;
    }
    // serve.rs:1268-1273: pages a restored prefix shares only in part are copied before the step (on
    // the step's stream, so the step sees them)
    for (size_t i = 0; i < step->num_restores; ++i) {
        if (step->restores[i].copy != 0) {
            const int copied = qwc_engine_copy_kv_block(e, step->restores[i].copy_from, step->restores[i].copy_to);
            if (copied != 0) {
                return copied;
            }
        }
    }
    if (rows > 0) {
        std::vector<uint32_t> tokens(rows);
        for (int row = 0; row < rows; ++row) {
            if (step->token_offsets[row + 1] - step->token_offsets[row] != 1) {
                return cudaErrorInvalidValue;  // a decode row carries one token (executor.rs:898-903)
            }
            tokens[row] = step->tokens[step->token_offsets[row]];
        }
        const int status =
            qwc_engine_decode(e, step->state_slots, tokens.data(), step->edits, step->num_edits, rows, sampled);
        if (status != 0) {
            return status;
        }
    } else if (step->num_edits > 0) {
        const int status = qwc_engine_apply_edits(e, step->edits, step->num_edits);
        if (status != 0) {
            return status;
        }
    }
    // Prompt tokens of a prefill chunk are taken as already resident; the chunk samples a token
    // derived from its sequence id.
    for (size_t row = step->num_decode; row < step->num_sequences; ++row) {
        sampled[row] = (step->seq_ids[row] * 7919u + 1000u) % static_cast<uint32_t>(e->cfg.vocab);
    }
    return 0;
}

}  // extern "C"
