// C API of the token-level worker loop (worker.h) declared in qwc_engine.h.
#include <vector>

#include "qwc_engine.h"
#include "runtime_handles.h"
#include "worker.h"

namespace {

using namespace qwc::runtime;

// The executor interface over a C callback: the step becomes a qwc_step_view of plain arrays.
class CallbackExecutor : public StepExecutor {
public:
    CallbackExecutor(qwc_execute_fn execute, void* user) : execute_(execute), user_(user) {}

    int execute(const StepInput& step, std::vector<uint32_t>* sampled) override {
        const BatchLayout& layout = *step.layout;
        std::vector<qwc_prefix_restore_op> restores;
        for (const PrefixRestoreOp& op : step.batch->restores) {
            restores.push_back({op.id, op.state_slot, op.snapshot, op.copy ? 1u : 0u, op.copy_from, op.copy_to});
        }
        std::vector<qwc_prefix_save_op> saves;
        for (const PrefixSaveOp& op : step.batch->saves) {
            saves.push_back({op.id, op.state_slot, op.snapshot});
        }
        static_assert(sizeof(qwc_table_edit) == sizeof(TableEdit), "the C view of an edit is the edit itself");
        qwc_step_view view{};
        view.num_sequences = layout.num_seqs();
        view.num_decode = layout.num_decode;
        view.seq_ids = layout.seq_ids.data();
        view.state_slots = layout.state_slots.data();
        view.position_starts = layout.position_starts.data();
        view.context_lens = layout.context_lens.data();
        view.token_offsets = layout.token_offsets.data();
        view.block_table_offsets = layout.block_table_offsets.data();
        view.block_ids = layout.block_ids.data();
        view.num_block_ids = layout.block_ids.size();
        view.tokens = step.tokens->data();
        view.num_tokens = step.tokens->size();
        view.edits = reinterpret_cast<const qwc_table_edit*>(step.edits->data());
        view.num_edits = step.edits->size();
        view.restores = restores.data();
        view.num_restores = restores.size();
        view.saves = saves.data();
        view.num_saves = saves.size();
        sampled->assign(layout.num_seqs(), 0);
        return execute_(user_, &view, sampled->data());
    }

private:
    qwc_execute_fn execute_;
    void* user_;
};

}  // namespace

struct qwc_worker {
    qwc_worker(qwc_scheduler* scheduler, qwc_execute_fn execute, void* execute_user, qwc_event_fn event,
               void* event_user, std::vector<uint32_t> eos_ids)
        : executor(execute, execute_user),
          worker(&scheduler->scheduler, &executor, event, event_user, std::move(eos_ids)) {}
    CallbackExecutor executor;
    Worker worker;
};

extern "C" {

qwc_worker* qwc_worker_new(qwc_scheduler* scheduler, qwc_execute_fn execute, void* execute_user, qwc_event_fn event,
                           void* event_user, const uint32_t* eos_ids, size_t num_eos) {
    if (scheduler == nullptr || execute == nullptr || event == nullptr) {
        return nullptr;
    }
    return new qwc_worker(scheduler, execute, execute_user, event, event_user,
                          std::vector<uint32_t>(eos_ids, eos_ids + num_eos));
}

void qwc_worker_free(qwc_worker* worker) { delete worker; }

void qwc_worker_submit(qwc_worker* worker, uint32_t id, const uint32_t* prompt, size_t prompt_tokens,
                       size_t max_new_tokens, size_t history_tokens, int ignore_eos) {
    Job job;
    job.id = id;
    job.prompt.assign(prompt, prompt + prompt_tokens);
    job.max_new_tokens = max_new_tokens;
    job.history_tokens = history_tokens;
    job.ignore_eos = ignore_eos != 0;
    worker->worker.submit(std::move(job));
}

void qwc_worker_abandon(qwc_worker* worker, uint32_t id) { worker->worker.abandon(id); }
void qwc_worker_shutdown(qwc_worker* worker) { worker->worker.shutdown(); }

int qwc_worker_iterate(qwc_worker* worker, int* progressed) {
    bool ran = false;
    const int status = worker->worker.iterate(&ran);
    if (progressed != nullptr) {
        *progressed = ran ? 1 : 0;
    }
    return status;
}

int qwc_worker_run(qwc_worker* worker) { return worker->worker.run(); }
size_t qwc_worker_jobs(const qwc_worker* worker) { return worker->worker.jobs(); }
uint64_t qwc_worker_steps(const qwc_worker* worker) { return worker->worker.steps(); }
uint64_t qwc_worker_aborted_steps(const qwc_worker* worker) { return worker->worker.aborted_steps(); }

}  // extern "C"
