// Steps the reference's own Scheduler and KVCacheManager (csrc/scheduler/scheduler.cpp, kv_cache_manager.cpp,
// compiled unchanged from the reference's checkout) through a scenario read from standard input, and prints every
// scheduling decision.  The model is replaced by "every request that wants a sample gets token 1".
//
// Input lines:   config <max_num_seqs> <token budget> <max_model_len> <block size> <num blocks>
//                add <id> <prompt tokens> <max output tokens>
//                abort <id>
//                step
// Output lines:  sched <step> <id> <position_offset> <n> <needs_sampling> <is_prefill> <block ids...>
//                out <step> <id> <finish reason 0|1|2>
//                idle <step>            (nothing was scheduled)
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "engine/config.h"
#include "model/model_config.h"
#include "scheduler/scheduler.h"

using namespace cuinfer;

int main()
{
    std::unique_ptr<Scheduler> scheduler;
    int step = 0;
    for (std::string line; std::getline(std::cin, line);) {
        std::istringstream in(line);
        std::string op;
        in >> op;
        if (op == "config") {
            Config config;
            ModelConfig model{};
            int block_size = 0;
            int num_blocks = 0;
            in >> config.max_num_seqs >> config.max_num_scheduled_tokens >> model.max_model_len >> block_size >> num_blocks;
            config.block_size = block_size;
            scheduler = std::make_unique<Scheduler>(config, model, KVCacheConfig{
                .num_block_slots = block_size, .num_blocks = num_blocks, .enable_prefix_caching = false});
        } else if (op == "add") {
            Request r{};
            int n = 0;
            in >> r.id >> n >> r.max_output_tokens;
            r.ignore_eos = true;
            r.token_ids.assign(n, 2);
            r.sample_params = SampleParams{.temperature = 0.f, .top_k = 0, .top_p = 1.f};
            scheduler->add_request(std::move(r));
        } else if (op == "abort") {
            std::string id;
            in >> id;
            scheduler->abort_requests({id});
        } else if (op == "step") {
            const std::vector<ScheduledRequest> scheduled = scheduler->schedule();
            if (scheduled.empty()) {
                std::cout << "idle " << step << "\n";
            }
            std::vector<SampledToken> sampled;
            for (const ScheduledRequest& s : scheduled) {
                std::cout << "sched " << step << " " << s.request_id << " " << s.position_offset << " "
                          << s.tokens_to_compute.size() << " " << (s.needs_sampling ? 1 : 0) << " "
                          << (s.is_prefill ? 1 : 0);
                for (int b : s.allocated_blocks) {
                    std::cout << " " << b;
                }
                std::cout << "\n";
                if (s.needs_sampling) {
                    sampled.push_back({.request_id = s.request_id, .token_id = 1, .eos_token = false});
                }
            }
            for (const EngineCoreOutput& o : scheduler->update(sampled)) {
                std::cout << "out " << step << " " << o.request_id << " " << static_cast<int>(o.finish_reason) << "\n";
            }
            step++;
        }
    }
    return 0;
}
