// Shared device helpers for the sm_100a decode-step kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace qwc {

// Lazy launcher set-up (shared-memory opt-in of a kernel, residency probes) belongs to a device, not
// to the process: a kernel attribute set with one device current says nothing about another.
// `slots` is the caller's table, one entry per device; `setup` runs once per device, with that
// device current, and its result is returned on every later call from that device.
constexpr int kMaxDevices = 64;
template <typename T>
struct PerDevice {
    bool done[kMaxDevices] = {};
    T value[kMaxDevices] = {};
    std::mutex lock;
    template <typename Setup>
    T* get(Setup&& setup) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
            return nullptr;
        }
        std::lock_guard<std::mutex> guard(lock);
        if (!done[device]) {
            value[device] = setup();
            done[device] = true;
        }
        return &value[device];
    }
};

// Row caps shared by the launchers; garbage-argument guards, not structure
// (mirrors crates/qwc-cuda/cuda/limits.cuh).
constexpr int kMaxStepRows = 2048;
constexpr int kMaxDecodeBatch = 128;

// Model constants that are the same for the reference checkpoint and the
// synthetic 27B-shaped model (crates/qwc-core/src/arch.rs:10-98).
constexpr int kQueryHeads = 24;
constexpr int kKvHeads = 4;
constexpr int kGqaGroup = kQueryHeads / kKvHeads;
constexpr int kHeadDim = 256;
constexpr int kRopeDim = 64;
constexpr int kDeltaKeyHeads = 16;
constexpr int kDeltaHeadDim = 128;

// Codes stored in the sticky device status word by bounded waits.
constexpr int kStatusOk = 0;
constexpr int kStatusAttentionPageWait = 0x101;
constexpr int kStatusDeltaTileWait = 0x102;
constexpr int kStatusGemvWait = 0x103;
constexpr int kStatusAttentionPlanOverflow = 0x104;  // a CTA's task list would not hold its share
constexpr int kStatusStateSlotRange = 0x105;         // a row named a DeltaNet state slot beyond the pool
constexpr int kStatusPeerWait = 0x106;               // a peer rank's slice of an activation row did not arrive

// What a caller said about the projection its stream runs after the next one it launches
// (qwc_nvfp4_prefetch_next): kept per host thread, taken (and cleared) by the next projection launch.
struct NextProjection {
    const void* packed[2];  // matrix, or gate and up matrices
    const void* scales[2];
    int out_features;
    int in_features;
    int kind;  // 0 NVFP4, 1 NVFP4 SwiGLU pair, 2 e4m3 rows
};
void set_next_projection(const NextProjection& next);
NextProjection take_next_projection();

// Process-wide shape selection (see qwc_configure in the C ABI).
struct Shape {
    int delta_value_heads;
    int kv_page_size;
};
Shape current_shape();

// Device address of the sticky status word of the current device: the first bounded
// wait that gives up stores its code there.  Resolved once per device on the host.
int* status_ptr();

__device__ __forceinline__ float bf16_bits_to_float(uint16_t bits) {
    return __uint_as_float(static_cast<uint32_t>(bits) << 16);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, off);
    }
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    }
    return v;
}

// 16-byte streaming load that does not allocate in L1: weights and cache pages are
// read exactly once per launch.
__device__ __forceinline__ uint4 ldg_stream(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
    return v;
}

// ---- mbarrier / bulk-copy (TMA 1-D) wrappers -------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait: gives up after ~20 ms of polling (a bulk copy completes in microseconds),
// records `code` in the status word and returns false; callers then skip the data and
// exit cleanly.  Kernels that wait also return at once when the status word is already
// set, so one failed wait cannot serialise into a long stall over the whole grid.
// The polling loop stays out of line so that the loops that wait stay short for the instruction caches;
// a wait that is already satisfied costs one test.
static __device__ __noinline__ bool mbar_wait_bounded_slow(uint64_t* bar, uint32_t parity, int code, int* status) {
    const long long start = clock64();
    for (;;) {
#pragma unroll 1
        for (int spin = 0; spin < 128; ++spin) {
            if (mbar_try_wait(bar, parity)) {
                return true;
            }
        }
        if (clock64() - start > 40000000ll) {
            break;
        }
    }
    atomicCAS(status, 0, code);
    return false;
}

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int code, int* status) {
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    return mbar_wait_bounded_slow(bar, parity, code, status);
}

__device__ __forceinline__ bool status_is_set(const int* status) {
    return *reinterpret_cast<const volatile int*>(status) != 0;
}

// Global -> shared bulk copy; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Shared -> global bulk copy (bulk async-group completion).
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

__device__ __forceinline__ void bulk_wait_all_read() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute
// may start while its predecessor in the stream still runs; it must not touch anything the
// predecessor writes before pdl_wait() returns (which is when the predecessor has completed and
// its writes are visible).  pdl_launch_dependents() in the predecessor lets that early start happen
// as soon as every one of its CTAs has issued it.  Both are no-ops in a plain launch.
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Host side of the same: a launch that may begin before its predecessor in the stream has ended.
// Every kernel launched this way calls pdl_wait() before it reads or writes anything that an
// earlier kernel of the step touches (weights are never written during a step).
template <typename... Params, typename... Args>
cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream,
                           Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// Make generic-proxy shared-memory writes visible to the async proxy (bulk stores, tensor-core reads).
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tensor-core helpers ---------------------------------------------------------

// D += A(16x16, f16, row) * B(16x8, f16, col), fp32 accumulate.
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four e2m1 pairs (one 32-bit word, 8 nibbles) -> four f16x2; .x of each is the low nibble.
__device__ __forceinline__ void cvt_e2m1x8_to_f16x2(uint32_t word, uint32_t (&out)[4]) {
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}\n"
        : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3])
        : "r"(word));
}

// Two e4m3 (low 16 bits) -> f16x2.
__device__ __forceinline__ uint32_t cvt_e4m3x2_to_f16x2(uint32_t pair) {
    uint32_t out;
    asm("{\n"
        ".reg .b16 lo, hi;\n"
        "mov.b32 {lo, hi}, %1;\n"
        "cvt.rn.f16x2.e4m3x2 %0, lo;\n"
        "}\n"
        : "=r"(out)
        : "r"(pair));
    return out;
}

// Four e4m3 (one word) -> two f16x2: bytes (0, 1) and bytes (2, 3).
__device__ __forceinline__ void cvt_e4m3x4_to_f16x2(uint32_t word, uint32_t& lo, uint32_t& hi) {
    asm("{\n"
        ".reg .b16 a, b;\n"
        "mov.b32 {a, b}, %2;\n"
        "cvt.rn.f16x2.e4m3x2 %0, a;\n"
        "cvt.rn.f16x2.e4m3x2 %1, b;\n"
        "}\n"
        : "=r"(lo), "=r"(hi)
        : "r"(word));
}

__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t out;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(out) : "r"(a), "r"(b));
    return out;
}

// Two bf16 (one 32-bit word) -> f16x2, finite saturation at +-65504.
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t word) {
    const float lo = __uint_as_float(word << 16);
    const float hi = __uint_as_float(word & 0xffff0000u);
    uint32_t out;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
    return out;
}

}  // namespace qwc
