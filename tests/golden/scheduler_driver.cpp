// Drives the reference's own host-side scheduler and block manager (engine/scheduler.cpp, engine/block_manager.cpp,
// engine/sequence.h; they need no GPU and no libtorch) through a small workload and prints, per step, the
// requests scheduled with their token counts and whether they sample.  The JSON it printed is committed as
// scheduler_golden.json; tests/test_scheduler.py replays the same workload through this package's scheduler.
//
// Build and run (on a machine that has the reference checked out at $REF):
//   g++ -std=c++20 -I$REF/engine tests/golden/scheduler_driver.cpp $REF/engine/scheduler.cpp \
//       $REF/engine/block_manager.cpp -o /tmp/sched_driver && /tmp/sched_driver > tests/golden/scheduler_golden.json
#include "scheduler.h"

#include <cstdio>
#include <memory>
#include <vector>

int main() {
    struct Case { int blocks; size_t budget, chunk, max_seqs; std::vector<int> prompts; int max_tokens; };
    const std::vector<Case> cases = {
        {12, 64, 24, 4, {5, 17, 33, 65, 100}, 4},
        {8, 32, 0, 8, {20, 40, 30, 10}, 20},
        {40, 48, 16, 3, {1, 31, 32, 65, 100, 7}, 12},
    };
    std::printf("[\n");
    for (size_t ci = 0; ci < cases.size(); ++ci) {
        const Case& c = cases[ci];
        SchedulerConfig cfg;
        cfg.max_num_batched_tokens = c.budget;
        cfg.max_chunk_tokens = c.chunk;
        cfg.max_num_seqs = c.max_seqs;
        cfg.eos_token_id = -5;
        Scheduler sched(cfg, c.blocks);
        std::vector<std::unique_ptr<Sequence>> seqs;
        int next_tok = 1000;
        for (size_t i = 0; i < c.prompts.size(); ++i) {
            std::vector<int32_t> p(c.prompts[i]);
            for (auto& t : p) t = next_tok++;                 // distinct tokens: the prefix cache never hits
            SamplingParams sp;
            sp.max_tokens = c.max_tokens;
            sp.ignore_eos = true;
            seqs.push_back(std::make_unique<Sequence>(i, p, sp));
            sched.add_request(seqs.back().get());
        }
        std::printf(" {\"blocks\": %d, \"budget\": %zu, \"chunk\": %zu, \"max_seqs\": %zu, \"max_tokens\": %d, \"prompts\": [",
                    c.blocks, c.budget, c.chunk, c.max_seqs, c.max_tokens);
        for (size_t i = 0; i < c.prompts.size(); ++i) std::printf("%s%d", i ? ", " : "", c.prompts[i]);
        std::printf("],\n  \"steps\": [\n");
        bool first = true;
        int guard = 0;
        while (!sched.is_finished() && guard++ < 1000) {
            ScheduledBatch b;
            sched.schedule(b, /*allow_preempt=*/true);
            std::printf("%s   [", first ? "" : ",\n");
            first = false;
            std::vector<int32_t> sampled(b.seqs.size(), -1);
            for (size_t i = 0; i < b.seqs.size(); ++i) {
                const Sequence* s = b.seqs[i];
                std::printf("%s[%llu, %u, %d]", i ? ", " : "", (unsigned long long)s->seq_id, s->num_scheduled_tokens,
                            samples_this_step(*s) ? 1 : 0);
                sampled[i] = next_tok++;
            }
            std::printf("]");
            sched.on_launched(b);
            sched.postprocess(b, sampled);
        }
        std::printf("\n  ], \"preemptions\": %zu}%s\n", sched.num_preemptions(), ci + 1 < cases.size() ? "," : "");
    }
    std::printf("]\n");
    return 0;
}
