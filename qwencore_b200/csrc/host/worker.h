// The serving worker loop at token level (crates/qwc-engine/src/bin/serve.rs:777-1074, :1133-1156,
// :1339-1368, :1438-1442): commands in, scheduler plan, batch layout, one executor call per step, token
// emission with the stop rules, completion, rollback on failure, cancellation of abandoned jobs.
//
// What the reference's loop does with text (tokenizer, stop strings, tool-call buffering, log-probability
// rows) and its speculative branch (the MTP head) are not part of it: a token reaches the caller through
// a callback whose return value says "stop here", which is where a stop string or a closed connection
// comes in.  The executor is an interface, so the loop runs against the GPU engine and, in tests, against
// a host stand-in that fails on demand.
#pragma once

#include <condition_variable>
#include <cstdint>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "runtime.h"

namespace qwc {
namespace runtime {

// What one step hands to the executor: the plan, its ragged layout, one input token per layout token
// (decode rows first: the token sampled by the previous step; then each prefill chunk's slice of its
// prompt), and the page-table edits the plan produced.
struct StepInput {
    const Batch* batch;
    const BatchLayout* layout;
    const std::vector<uint32_t>* tokens;
    const std::vector<TableEdit>* edits;
};

class StepExecutor {
public:
    virtual ~StepExecutor() = default;
    // Runs the step; `sampled` receives one token per sequence of the layout, in layout order (the
    // last row of each segment, Executor::execute_layout, executor.rs:878-951).  0 or an error code;
    // after an error nothing of the step may be committed.
    virtual int execute(const StepInput& step, std::vector<uint32_t>* sampled) = 0;
};

enum class WorkerEvent : uint32_t {
    Token = 0,     // value = the token
    Done = 1,      // value = tokens emitted, reason = FinishReason
    Error = 2,     // value = the error code the worker stopped with, or 0x5000 + SubmitError
};

// kind Token: a non-zero return stops the sequence after this token.  Other kinds ignore the result.
using EventSink = int (*)(void* user, uint32_t id, uint32_t kind, uint32_t value, uint32_t reason);

struct Job {
    SeqId id = 0;
    std::vector<uint32_t> prompt;
    size_t max_new_tokens = 0;
    size_t history_tokens = 0;  // the snapshot point of the prompt (the prefix worth caching)
    bool ignore_eos = false;
};

enum WorkerStatus : int {
    kWorkerOk = 0,
    kWorkerSchedulerFailed = 0x2000,  // + SchedulerError
    kWorkerLayoutFailed = 0x3000,     // + LayoutError
    kWorkerMissingToken = 0x5100,     // a decode row without a sampled token
    kWorkerMissingPrompt = 0x5101,    // a prefill chunk without its job
    kWorkerShortSample = 0x5102,      // the executor returned fewer tokens than sequences
    kWorkerSubmitFailed = 0x5000,     // + SubmitError, in an Error event only
};

class Worker {
public:
    Worker(Scheduler* scheduler, StepExecutor* executor, EventSink sink, void* sink_user,
           std::vector<uint32_t> eos_ids);

    // Thread-safe: any thread may queue work while another runs the loop.
    void submit(Job job);
    void abandon(SeqId id);  // the client went away: the job is cancelled between steps
    void shutdown();         // no more commands will come: run() returns once the jobs are finished

    // One pass of the loop body.  *progressed: a step ran.  Returns kWorkerOk or the code the worker
    // failed with; a failed worker has told every job (Error event) and accepts nothing more.
    int iterate(bool* progressed);
    // The loop: waits up to 10 ms for a command when there is nothing to run (serve.rs:811-821).
    int run();

    size_t jobs() const { return jobs_.size(); }
    int failed() const { return failed_; }
    uint64_t steps() const { return steps_; }
    uint64_t aborted_steps() const { return aborted_steps_; }

private:
    struct ActiveJob {
        std::vector<uint32_t> prompt;
        size_t emitted = 0;
        bool ignore_eos = false;
    };

    void accept_commands();
    int fail_all(int code, bool abort);
    void finish(const Completion& completion);
    bool is_eos(uint32_t token) const;

    Scheduler* scheduler_;
    StepExecutor* executor_;
    EventSink sink_;
    void* sink_user_;
    std::vector<uint32_t> eos_ids_;

    std::mutex mutex_;
    std::condition_variable wake_;
    std::deque<Job> commands_;
    std::vector<SeqId> abandoned_commands_;
    bool shutdown_ = false;

    std::unordered_map<SeqId, ActiveJob> jobs_;
    std::unordered_map<SeqId, uint32_t> pending_;  // the token each sequence emits and feeds next
    std::unordered_set<SeqId> abandoned_;
    int failed_ = 0;
    uint64_t steps_ = 0;
    uint64_t aborted_steps_ = 0;
};

}  // namespace runtime
}  // namespace qwc
