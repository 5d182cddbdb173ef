/*
 * Latency mode (tensor-parallel decode of one sequence): the description of one activation row
 * that the ranks of a node hand one another inside a step.  Plain C; shared by qwc_abi.h and the
 * kernels.
 *
 * The reference all-gathers every projection's output with ncclAllGather
 * (crates/qwc-engine/src/executor.rs, tensor-parallel branches of the decode step); here a
 * projection's epilogue stores its partial sums into every rank's copy of the row, each element as
 * one 8-byte word {fp32 bits, tag}, and the consumers poll the tags (bounded) while they sum.
 */
#ifndef QWC_EXCHANGE_H
#define QWC_EXCHANGE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QWC_MAX_PEERS 8
#define QWC_EXCHANGE_MAX_SLICES 8
#define QWC_EXCHANGE_MAX_INSTANCES 1024

typedef struct qwc_exchange_row {
    void* blocks[QWC_MAX_PEERS]; /* every rank's exchange block as THIS device addresses it (its own block
                                    at [rank], the others through their peer mappings) */
    int ranks;                   /* 2..8 (1 is accepted: a single rank exchanging with itself) */
    int rank;
    const void* epoch;           /* device u32 that qwc_exchange_advance bumps once per step on every rank */
    uint32_t instance;           /* which exchange of the step this is, < QWC_EXCHANGE_MAX_INSTANCES; consecutive
                                    exchanges must not share `offset` */
    uint64_t offset;             /* of the row's words inside every block, bytes, a multiple of 16 */
    int width;                   /* elements of the full row (all ranks' columns), a multiple of 4 */
    uint32_t flags;              /* QWC_EXCHANGE_ANY_TAG: consumers take whatever words are there (for timing a
                                    consumer alone on the words of an earlier step; never in a real step) */
    void* wait_profile;          /* NULL, or device u64[QWC_EXCHANGE_MAX_INSTANCES]: entry [instance] is raised to the
                                    longest time, in nanoseconds, that a consumer thread has waited for a word of
                                    this exchange (the caller zeroes it).  A measurement aid that costs an atomic
                                    per late word and so lengthens the waits several times over: never in a
                                    timed run */
} qwc_exchange_row;

#define QWC_EXCHANGE_ANY_TAG 1u

#ifdef __cplusplus
}
#endif

#endif /* QWC_EXCHANGE_H */
