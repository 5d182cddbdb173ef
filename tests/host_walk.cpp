// Random walk over the host runtime (scheduler, cache manager with prefix cache, batch layout, worker
// loop with client threads) for the sanitizer builds of tests/test_host_sanitizers.py: the program
// checks little itself - what it is for is that AddressSanitizer, UBSan and ThreadSanitizer see every
// path of the C++ port under churn (admission, eviction, rollback, cancellation, commands queued from
// other threads) and stay silent.
#include <algorithm>
#include <cstdio>
#include <random>
#include <thread>
#include <atomic>
#include "runtime.h"
#include "worker.h"
using namespace qwc::runtime;

struct FakeExec : StepExecutor {
    std::mt19937 rng{7};
    int execute(const StepInput& step, std::vector<uint32_t>* sampled) override {
        sampled->clear();
        for (size_t i = 0; i < step.layout->num_seqs(); ++i) sampled->push_back(rng() % 1000 == 0 ? 7u : 8u + rng() % 500);
        return 0;
    }
};
static std::atomic<long> g_events{0};
static int sink(void*, uint32_t, uint32_t kind, uint32_t, uint32_t) { ++g_events; return kind == 0 && (g_events % 37 == 0); }

int main() {
    for (int seed = 0; seed < 30; ++seed) {
        std::mt19937 rng(seed);
        Scheduler s(SchedulerConfig{4, 96}, CacheManager(6, seed % 2 ? 24 : 96, 16));
        s.enable_prefix_cache(seed % 4);
        std::vector<uint32_t> live;
        uint32_t next = 1;
        std::vector<uint32_t> history(120);
        for (auto& t : history) t = rng() % 50;
        for (int op = 0; op < 2000; ++op) {
            const int draw = rng() % 100;
            if (draw < 35) {
                const size_t keep = 10 + rng() % 110;
                std::vector<uint32_t> prompt(history.begin(), history.begin() + keep);
                for (int i = 0, n = 1 + rng() % 30; i < n; ++i) prompt.push_back(50 + rng() % 50);
                Request r{next, prompt.size(), 1 + rng() % 12};
                const size_t snap = rng() % 3 ? keep : rng() % (prompt.size() + 1);
                if ((rng() % 4 ? s.submit_prompt(r, prompt, snap) : s.submit(r)) == SubmitError::None) live.push_back(next);
                ++next;
            } else if (draw < 93) {
                Batch b; bool has = false;
                if (s.next_batch(&b, &has) != SchedulerError::None || !has) continue;
                BatchLayout layout; SeqId offender;
                if (BatchLayout::build(b, s.cache(), &layout, &offender) != LayoutError::None) { std::puts("layout failed"); return 1; }
                s.cache_mut().drain_edits();
                if (draw >= 85) { s.abort_batch(); continue; }
                std::vector<SeqId> stopped;
                for (SeqId id : b.decode) if (rng() % 12 == 0) stopped.push_back(id);
                std::vector<Completion> done;
                if (s.complete_batch(stopped, &done) != SchedulerError::None) { std::puts("complete failed"); return 1; }
                for (auto& c : done) live.erase(std::find(live.begin(), live.end(), c.id));
            } else if (!live.empty()) {
                const size_t at = rng() % live.size();
                bool removed = false;
                s.cancel(live[at], &removed);
                if (!removed) { std::puts("cancel failed"); return 1; }
                live.erase(live.begin() + at);
            }
        }
    }
    // the worker with client threads
    Scheduler s(SchedulerConfig{8, 256}, CacheManager(8, 800, 16));
    s.enable_prefix_cache(3);
    FakeExec exec;
    Worker worker(&s, &exec, sink, nullptr, {7u});
    std::thread loop([&] { worker.run(); });
    std::vector<std::thread> clients;
    for (int c = 0; c < 4; ++c) clients.emplace_back([&, c] {
        for (uint32_t i = 0; i < 200; ++i) {
            Job job; job.id = 1000 * c + i + 1; job.prompt.assign(20 + i % 40, i % 5); job.max_new_tokens = 1 + i % 7; job.history_tokens = 16;
            worker.submit(job);
            if (i % 6 == 0) worker.abandon(job.id);
        }
    });
    for (auto& t : clients) t.join();
    worker.shutdown();
    loop.join();
    std::printf("ok events=%ld steps=%llu failed=%d\n", g_events.load(), (unsigned long long)worker.steps(), worker.failed());
    return worker.failed();
}
