// The serving worker loop at token level: see worker.h.
#include "worker.h"

#include <algorithm>
#include <chrono>

namespace qwc {
namespace runtime {

Worker::Worker(Scheduler* scheduler, StepExecutor* executor, EventSink sink, void* sink_user,
               std::vector<uint32_t> eos_ids)
    : scheduler_(scheduler), executor_(executor), sink_(sink), sink_user_(sink_user), eos_ids_(std::move(eos_ids)) {}

void Worker::submit(Job job) {
    {
        std::lock_guard<std::mutex> lock(mutex_);
        commands_.push_back(std::move(job));
    }
    wake_.notify_one();
}

void Worker::abandon(SeqId id) {
    {
        std::lock_guard<std::mutex> lock(mutex_);
        abandoned_commands_.push_back(id);
    }
    wake_.notify_one();
}

void Worker::shutdown() {
    {
        std::lock_guard<std::mutex> lock(mutex_);
        shutdown_ = true;
    }
    wake_.notify_one();
}

bool Worker::is_eos(uint32_t token) const {
    return std::find(eos_ids_.begin(), eos_ids_.end(), token) != eos_ids_.end();
}

// serve.rs:1339-1368: a job enters the scheduler with its prompt tokens and its history boundary; a
// request the scheduler refuses is answered at once and never becomes a job.
void Worker::accept_commands() {
    std::deque<Job> commands;
    std::vector<SeqId> abandoned;
    {
        std::lock_guard<std::mutex> lock(mutex_);
        commands.swap(commands_);
        abandoned.swap(abandoned_commands_);
    }
    for (Job& job : commands) {
        if (failed_ != 0) {
            sink_(sink_user_, job.id, static_cast<uint32_t>(WorkerEvent::Error), static_cast<uint32_t>(failed_), 0);
            continue;
        }
        // a snapshot point beyond the prompt is the caller's error; the scheduler would refuse it as well
        const size_t history = std::min(job.history_tokens, job.prompt.size());
        const SubmitError refused =
            scheduler_->submit_prompt(Request{job.id, job.prompt.size(), job.max_new_tokens}, job.prompt, history);
        if (refused != SubmitError::None) {
            sink_(sink_user_, job.id, static_cast<uint32_t>(WorkerEvent::Error),
                  static_cast<uint32_t>(kWorkerSubmitFailed + static_cast<int>(refused)), 0);
            continue;
        }
        jobs_[job.id] = ActiveJob{std::move(job.prompt), 0, job.ignore_eos};
    }
    for (const SeqId id : abandoned) {
        if (jobs_.count(id) != 0) {
            abandoned_.insert(id);
        }
    }
}

// serve.rs:1438-1442, with the rollback its callers do first (:828-835, :980-987).
int Worker::fail_all(int code, bool abort) {
    if (abort) {
        scheduler_->abort_batch();
        ++aborted_steps_;
    }
    for (const auto& job : jobs_) {
        sink_(sink_user_, job.first, static_cast<uint32_t>(WorkerEvent::Error), static_cast<uint32_t>(code), 0);
    }
    jobs_.clear();
    pending_.clear();
    abandoned_.clear();
    failed_ = code;
    return code;
}

// serve.rs:1133-1156
void Worker::finish(const Completion& completion) {
    const auto job = jobs_.find(completion.id);
    if (job != jobs_.end()) {
        sink_(sink_user_, completion.id, static_cast<uint32_t>(WorkerEvent::Done),
              static_cast<uint32_t>(job->second.emitted), static_cast<uint32_t>(completion.reason));
        jobs_.erase(job);
    }
    pending_.erase(completion.id);
    abandoned_.erase(completion.id);
}

int Worker::iterate(bool* progressed) {
    *progressed = false;
    accept_commands();
    if (failed_ != 0) {
        return failed_;
    }

    Batch batch;
    bool has_batch = false;
    const SchedulerError planned = scheduler_->next_batch(&batch, &has_batch);
    if (planned != SchedulerError::None) {
        return fail_all(kWorkerSchedulerFailed + static_cast<int>(planned), false);
    }
    if (has_batch) {
        BatchLayout layout;
        SeqId offender = 0;
        const LayoutError laid = BatchLayout::build(batch, scheduler_->cache(), &layout, &offender);
        if (laid != LayoutError::None) {
            return fail_all(kWorkerLayoutFailed + static_cast<int>(laid), true);
        }

        // serve.rs:949-971: decode rows feed the token the previous step sampled, prefill chunks their
        // slice of the prompt
        std::vector<uint32_t> input;
        input.reserve(layout.num_tokens());
        for (const SeqId id : batch.decode) {
            const auto token = pending_.find(id);
            if (token == pending_.end()) {
                return fail_all(kWorkerMissingToken, true);
            }
            input.push_back(token->second);
        }
        for (const PrefillChunk& chunk : batch.prefill) {
            const auto job = jobs_.find(chunk.id);
            if (job == jobs_.end() || chunk.offset + chunk.tokens > job->second.prompt.size()) {
                return fail_all(kWorkerMissingPrompt, true);
            }
            input.insert(input.end(), job->second.prompt.begin() + chunk.offset,
                         job->second.prompt.begin() + chunk.offset + chunk.tokens);
        }

        const std::vector<TableEdit> edits = scheduler_->cache_mut().drain_edits();
        std::vector<uint32_t> sampled;
        const StepInput step{&batch, &layout, &input, &edits};
        const int executed = executor_->execute(step, &sampled);
        if (executed != 0) {
            return fail_all(executed, true);
        }
        if (sampled.size() < layout.num_seqs()) {
            return fail_all(kWorkerShortSample, true);
        }
        ++steps_;
        *progressed = true;

        // serve.rs:997-1007: a decode row emits the token it was fed.  An end-of-sequence token stops
        // the sequence without being emitted; the sink stops it after the token it just took.
        std::vector<SeqId> stopped;
        for (const SeqId id : batch.decode) {
            const uint32_t token = pending_[id];
            const auto job = jobs_.find(id);
            bool stop = true;
            if (job != jobs_.end()) {
                if (!job->second.ignore_eos && is_eos(token)) {
                    stop = true;
                } else {
                    ++job->second.emitted;
                    stop = sink_(sink_user_, id, static_cast<uint32_t>(WorkerEvent::Token), token, 0) != 0;
                }
            }
            if (stop) {
                stopped.push_back(id);
            }
        }
        for (size_t row = 0; row < layout.num_seqs(); ++row) {
            pending_[layout.seq_ids[row]] = sampled[row];
        }

        std::vector<Completion> completed;
        const SchedulerError finished = scheduler_->complete_batch(stopped, &completed);
        if (finished != SchedulerError::None) {
            return fail_all(kWorkerSchedulerFailed + static_cast<int>(finished), false);
        }
        for (const Completion& completion : completed) {
            finish(completion);
        }
    }

    // serve.rs:1062-1072: jobs nobody listens to any more leave between steps.  (The reference does
    // this after a step only; with nothing in flight it is as safe when the step was empty.)
    for (auto it = abandoned_.begin(); it != abandoned_.end();) {
        bool removed = false;
        const SchedulerError cancelled = scheduler_->cancel(*it, &removed);
        if (cancelled == SchedulerError::None && removed) {
            jobs_.erase(*it);
            pending_.erase(*it);
            it = abandoned_.erase(it);
        } else {
            ++it;
        }
    }
    return kWorkerOk;
}

int Worker::run() {
    for (;;) {
        bool progressed = false;
        const int status = iterate(&progressed);
        if (status != 0) {
            return status;
        }
        if (progressed) {
            continue;
        }
        std::unique_lock<std::mutex> lock(mutex_);
        if (!commands_.empty() || !abandoned_commands_.empty()) {
            continue;
        }
        if (shutdown_ && jobs_.empty()) {
            return kWorkerOk;
        }
        wake_.wait_for(lock, std::chrono::milliseconds(10));
    }
}

}  // namespace runtime
}  // namespace qwc
