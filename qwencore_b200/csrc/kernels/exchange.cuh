// Latency mode: the rows that ranks hand one another inside a decode step.
//
// A projection whose weight rows are split over G ranks leaves, on every rank, fp32 partial sums for
// its own columns of the output row ([slice][width], one row: latency mode is batch 1).  Instead of
// finishing them locally and gathering the result with a collective, the projection's epilogue stores
// each partial sum straight into every rank's copy of the slice array - its own by a local store, the
// others' through the peer mapping of their exchange block - and the kernels that consume the row
// (the residual norm, the DeltaNet prepare step, ...) sum the slices of their own copy exactly as they
// do on one GPU.
//
// There is no flag and no fence: every element travels as one aligned 8-byte word {fp32 bits, tag},
// written by one store, so a reader that sees the tag sees the value.  The tag names the step and the
// exchange within it (epoch << 10 | instance; the epoch is a device word that the first kernel of
// every step advances, equal on all ranks because they run the same steps); whatever an earlier use
// of the buffer left there carries another tag.  A consumer polls the words it needs until their tags
// match, for at most a second: when it gives up it stores kStatusPeerWait in the sticky status word,
// uses zero, and every later wait of the step gives up at once.
//
// Measured alternatives (64 layers, ms per step; the form above: 4.3 on two GPUs, 4.0 on four):
// consumers that read each column from its owner's block over NVLink instead (stores stay local):
// 12.7 on two - a polling load of a peer's memory takes a link round trip; a system-scope fence per
// storing warp after the stores: 7.0 on two - the fence costs 4 - 10 us at the end of every projection
// and buys nothing, the stores arrive without it; 256-byte bulk copies from shared memory instead of
// 8-byte stores, a rotated order of destinations, a longer back-off between polls: no change.  What
// did matter is how a consumer waits (see tagged_sums below).  A per-exchange wait profile (an atomic
// maximum per word that was waited for) is available for diagnosis but lengthens the waits it
// measures by an order of magnitude; it is off unless asked for.
//
// A buffer may be written for exchange i + 2 or later while a peer still reads exchange i from it: a
// rank launches the producer of exchange i + 1 only after its consumers of exchange i have completed,
// and a peer cannot produce exchange i + 2 before it has consumed this rank's part of exchange i + 1.
// The engine therefore alternates buffers between consecutive exchanges.
//
// (Replaces the ncclAllGather after every projection of crates/qwc-engine/src/executor.rs's
// tensor-parallel decode; the arithmetic per element is the unsplit projection's.)
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

#include "../../../include/qwc_exchange.h"
#include "common.cuh"

namespace qwc {

constexpr int kMaxPeers = QWC_MAX_PEERS;
constexpr int kExchangeTagBits = 10;  // exchanges per step < 1024
constexpr int kExchangeMaxSlices = QWC_EXCHANGE_MAX_SLICES;
static_assert((1 << kExchangeTagBits) == QWC_EXCHANGE_MAX_INSTANCES, "the tag holds the instance number");
constexpr unsigned long long kExchangeWaitNs = 1000000000ull;  // a consumer waits a second for a peer's words
constexpr int kExchangeSpinLimit = 1 << 24;  // ... and never more than this many polls, whatever the timer says

// Producer side: where the partial sums go.
struct ExchangeTarget {
    uint2* copies[kMaxPeers];  // the row [slices][width] in every rank's block as this device addresses it
    int ranks;                 // 0: no exchange
    const uint32_t* epoch;     // device word, advanced once per step
    uint32_t instance;         // of this exchange within the step
    int width;                 // elements of a full row (all ranks' columns)
    int first_column;          // where this rank's columns start
};

// Consumer side: this rank's copy of the row, [slices][width] tagged words.
struct TaggedRow {
    const uint2* words;  // null: not an exchanged row
    int slices;
    int width;
    const uint32_t* epoch;
    uint32_t instance;
    int* status;
    uint32_t tag_mask;  // all ones; zero when any tag is accepted (QWC_EXCHANGE_ANY_TAG)
    unsigned long long* wait_profile;  // null, or [instance]: the longest wait seen, ns
};

__device__ __forceinline__ uint32_t exchange_tag(const uint32_t* epoch, uint32_t instance) {
    return (__ldcg(epoch) << kExchangeTagBits) | instance;
}

__device__ __forceinline__ void store_tagged(uint2* at, float value, uint32_t tag) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(at), "r"(__float_as_uint(value)), "r"(tag)
                 : "memory");
}

__device__ __forceinline__ uint2 load_tagged(const uint2* at) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(at) : "memory");
    return v;
}

__device__ __forceinline__ uint4 load_tagged_pair(const uint2* at) {  // two neighbouring elements, 16-byte aligned
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(at)
                 : "memory");
    return v;
}

// The slow path of a read: poll one word until its tag matches, for at most kExchangeWaitNs.  Gives up
// at once when the status word already holds a code (an earlier wait of this step failed: the row
// will not come).
static __device__ __noinline__ float await_tagged(const uint2* at, uint32_t tag, int* status,
                                                  unsigned long long* wait_profile) {
    unsigned long long start;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(start)::"memory");
    for (int spin = 0; spin < kExchangeSpinLimit; ++spin) {
        const uint2 word = load_tagged(at);
        if (word.y == tag) {
            if (wait_profile != nullptr) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now)::"memory");
                atomicMax(wait_profile + (tag & (QWC_EXCHANGE_MAX_INSTANCES - 1)), now - start);
            }
            return __uint_as_float(word.x);
        }
        if ((spin & 63) == 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now)::"memory");
            if (now - start > kExchangeWaitNs || *reinterpret_cast<volatile int*>(status) != kStatusOk) {
                break;
            }
        }
        __nanosleep(100);
    }
    if (atomicCAS(status, kStatusOk, kStatusPeerWait) == kStatusOk) {
        status[2] = static_cast<int>(tag);  // for the host's report: the tag waited for and the one found
        status[3] = static_cast<int>(load_tagged(at).y);
    }
    return 0.0f;
}

// A consumer's first look usually comes a link latency before its peers' words: then the whole batch
// of loads is issued again (one round trip whatever the number of words), a bounded number of times,
// before the words that are still missing are waited for one by one (which is where the time limit
// and the status word are handled).  Re-reading late words one after another cost a round trip per
// word: 32 words per thread made every exchange 10 - 25 us slower on four and eight GPUs.
constexpr int kQuickRetries = 512;

__device__ __forceinline__ bool keep_retrying(int attempt, const int* status) {
    return attempt < kQuickRetries &&
           ((attempt & 15) != 15 || *reinterpret_cast<const volatile int*>(status) == kStatusOk);
}

// Sums over slices (in slice order) of kValues columns at once: every word of up to eight slices of
// every column is asked for before the first is looked at, so the sum costs one round trip per eight
// slices whatever the number of columns.
template <int kValues>
__device__ __forceinline__ void tagged_sums(const TaggedRow& row, uint32_t tag, const int (&columns)[kValues],
                                            float (&totals)[kValues]) {
#pragma unroll
    for (int v = 0; v < kValues; ++v) {
        totals[v] = 0.0f;
    }
    for (int first = 0; first < row.slices; first += 8) {
        uint2 part[kValues][8];
        for (int attempt = 0;; ++attempt) {
            bool complete = true;
#pragma unroll
            for (int v = 0; v < kValues; ++v) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    part[v][j] = load_tagged(row.words + static_cast<size_t>(min(first + j, row.slices - 1)) * row.width +
                                             columns[v]);
                }
            }
#pragma unroll
            for (int v = 0; v < kValues; ++v) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    complete = complete && ((part[v][j].y ^ tag) & row.tag_mask) == 0;
                }
            }
            if (complete || !keep_retrying(attempt, row.status)) {
                break;
            }
            __nanosleep(100);
        }
#pragma unroll
        for (int v = 0; v < kValues; ++v) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (first + j < row.slices) {
                    totals[v] += ((part[v][j].y ^ tag) & row.tag_mask) == 0
                                     ? __uint_as_float(part[v][j].x)
                                     : await_tagged(row.words + static_cast<size_t>(first + j) * row.width + columns[v],
                                                    tag, row.status, row.wait_profile);
                }
            }
        }
    }
}

__device__ __forceinline__ float tagged_sum(const TaggedRow& row, uint32_t tag, int column) {
    const int columns[1] = {column};
    float totals[1];
    tagged_sums<1>(row, tag, columns, totals);
    return totals[0];
}

// ... of four neighbouring columns (column a multiple of four), eight slices in flight.
__device__ __forceinline__ float4 tagged_sum4(const TaggedRow& row, uint32_t tag, int column) {
    const uint2* at = row.words + column;
    float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int first = 0; first < row.slices; first += 8) {
        uint4 part[8][2];
        for (int attempt = 0;; ++attempt) {
            bool complete = true;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint2* from = at + static_cast<size_t>(min(first + j, row.slices - 1)) * row.width;
                part[j][0] = load_tagged_pair(from);
                part[j][1] = load_tagged_pair(from + 2);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                complete = complete && (((part[j][0].y ^ tag) | (part[j][0].w ^ tag) | (part[j][1].y ^ tag) |
                                         (part[j][1].w ^ tag)) &
                                        row.tag_mask) == 0;
            }
            if (complete || !keep_retrying(attempt, row.status)) {
                break;
            }
            __nanosleep(100);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (first + j < row.slices) {
                const uint2* from = at + static_cast<size_t>(first + j) * row.width;
                const uint32_t bits[4] = {part[j][0].x, part[j][0].z, part[j][1].x, part[j][1].z};
                const uint32_t tags[4] = {part[j][0].y, part[j][0].w, part[j][1].y, part[j][1].w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    total[c] += ((tags[c] ^ tag) & row.tag_mask) == 0
                                    ? __uint_as_float(bits[c])
                                    : await_tagged(from + c, tag, row.status, row.wait_profile);
                }
            }
        }
    }
    return make_float4(total[0], total[1], total[2], total[3]);
}

// ---- host side: the C description of a row -> what the kernels take ------------------------------

inline bool valid_exchange_row(const qwc_exchange_row* row) {
    if (row == nullptr || row->ranks < 1 || row->ranks > kMaxPeers || row->rank < 0 || row->rank >= row->ranks ||
        row->epoch == nullptr || row->instance >= QWC_EXCHANGE_MAX_INSTANCES || row->offset % 16 != 0 ||
        row->width <= 0 || row->width % 4 != 0) {
        return false;
    }
    for (int r = 0; r < row->ranks; ++r) {
        if (row->blocks[r] == nullptr || (reinterpret_cast<uintptr_t>(row->blocks[r]) & 15) != 0) {
            return false;
        }
    }
    return true;
}

inline ExchangeTarget exchange_target(const qwc_exchange_row& row, int first_column) {
    ExchangeTarget target = {};
    for (int r = 0; r < row.ranks; ++r) {
        target.copies[r] = reinterpret_cast<uint2*>(static_cast<unsigned char*>(row.blocks[r]) + row.offset);
    }
    target.ranks = row.ranks;
    target.epoch = static_cast<const uint32_t*>(row.epoch);
    target.instance = row.instance;
    target.width = row.width;
    target.first_column = first_column;
    return target;
}

inline TaggedRow tagged_row(const qwc_exchange_row& row, int slices, int* status) {
    TaggedRow tagged = {};
    tagged.words = reinterpret_cast<const uint2*>(static_cast<const unsigned char*>(row.blocks[row.rank]) + row.offset);
    tagged.slices = slices;
    tagged.width = row.width;
    tagged.epoch = static_cast<const uint32_t*>(row.epoch);
    tagged.instance = row.instance;
    tagged.status = status;
    tagged.tag_mask = (row.flags & QWC_EXCHANGE_ANY_TAG) != 0 ? 0u : 0xffffffffu;
    tagged.wait_profile = static_cast<unsigned long long*>(row.wait_profile);
    return tagged;
}

}  // namespace qwc
