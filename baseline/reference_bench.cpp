// Driver for the UNMODIFIED reference engine (typr7/cuInfer), used by `bench.py --impl reference`.
//
// The reference's engine loop (csrc/engine/engine_core.cpp:93-105) is
//     schedule -> ModelRunner::run_model -> ModelRunner::finish -> Scheduler::update
// between a ZeroMQ input and output socket.  This program runs exactly that loop on the reference's own
// Scheduler and ModelRunner classes (stock code path: its batch buffer, CUDA graphs, kernels, cuBLAS calls and
// sampler), with requests added directly instead of arriving over the socket.  Nothing of cuinfer_b200 is
// linked or loaded.  The KV pool is sized the way the reference sizes it
// (csrc/engine/engine_core.cpp:107-137).
//
// Modes:
//   bench     B requests decode to --context tokens; K timed decode steps after W warm-up steps; then
//             2048-token prompts one at a time (prefill).  Prints one JSON object.
//   serve     the reference's own benchmark workload (benchmark.sh:67-97) without HTTP: prompts of --prompt-len random
//             tokens, --max-tokens outputs, --batch requests in flight (a new one is added when one ends), 3 x batch
//             requests timed after batch warm-up requests.  Prints one JSON object.
//   generate  reads prompts (one line of space-separated ids each) from --prompts, generates --max-tokens
//             greedy tokens for each and prints one line of ids per prompt (golden tokens for the tests).
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <random>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "engine/config.h"
#include "executor/model_runner.h"
#include "scheduler/kv_cache_manager.h"
#include "scheduler/request.h"
#include "scheduler/scheduler.h"

using namespace cuinfer;
using Clock = std::chrono::steady_clock;

namespace
{

struct Args
{
    std::string mode = "bench";
    std::string model;
    std::string prompts;
    int batch = 8;
    int context = 4096;
    int steps = 20;
    int warmup = 5;
    int prefill_tokens = 2048;
    int prefill_runs = 5;
    int max_tokens = 16;
    int prompt_len = 1024;
    int block_size = 16;
    int max_num_scheduled_tokens = 8192;
    int max_num_seqs = 256;
    float gpu_memory_utilization = 0.9f;
    bool cuda_graph = true;
    unsigned seed = 1234;
};

Args parse(int argc, char** argv)
{
    Args a;
    for (int i = 1; i < argc; i++) {
        const std::string k = argv[i];
        auto next = [&]() -> std::string {
            if (i + 1 >= argc) {
                throw std::runtime_error("missing value for " + k);
            }
            return argv[++i];
        };
        if (k == "--mode") a.mode = next();
        else if (k == "--model") a.model = next();
        else if (k == "--prompts") a.prompts = next();
        else if (k == "--batch") a.batch = std::stoi(next());
        else if (k == "--context") a.context = std::stoi(next());
        else if (k == "--steps") a.steps = std::stoi(next());
        else if (k == "--warmup") a.warmup = std::stoi(next());
        else if (k == "--prefill-tokens") a.prefill_tokens = std::stoi(next());
        else if (k == "--prefill-runs") a.prefill_runs = std::stoi(next());
        else if (k == "--max-tokens") a.max_tokens = std::stoi(next());
        else if (k == "--prompt-len") a.prompt_len = std::stoi(next());
        else if (k == "--block-size") a.block_size = std::stoi(next());
        else if (k == "--max-num-scheduled-tokens") a.max_num_scheduled_tokens = std::stoi(next());
        else if (k == "--max-num-seqs") a.max_num_seqs = std::stoi(next());
        else if (k == "--gpu-memory-utilization") a.gpu_memory_utilization = std::stof(next());
        else if (k == "--disable-cuda-graph") a.cuda_graph = false;
        else if (k == "--seed") a.seed = static_cast<unsigned>(std::stoul(next()));
        else throw std::runtime_error("unknown option " + k);
    }
    if (a.model.empty()) {
        throw std::runtime_error("--model is required");
    }
    return a;
}

// The reference's own sizing of the KV pool (csrc/engine/engine_core.cpp:107-137).
KVCacheConfig initialize_kv_cache(ModelRunner& runner, const Config& config)
{
    const std::size_t bytes = runner.profile_available_kv_cache_memory(config.gpu_memory_utilization);
    const int num_blocks = static_cast<int>(bytes / runner.kv_cache_block_bytes());
    if (num_blocks * config.block_size < runner.model_config().max_model_len) {
        throw std::runtime_error("kv cache smaller than one request of max_model_len");
    }
    runner.allocate_kv_cache(num_blocks);
    return KVCacheConfig{
        .num_block_slots = config.block_size,
        .num_blocks = num_blocks,
        .enable_prefix_caching = config.enable_prefix_caching
    };
}

struct Engine
{
    explicit Engine(const Config& config)
        : runner(config), scheduler(config, runner.model_config(), initialize_kv_cache(runner, config))
    {
    }

    // One iteration of the reference's engine loop.  With `device_ms`, the step's time on the device is taken
    // with two events on the legacy default stream: the reference's stream is a blocking stream
    // (csrc/cuda/cuda_context.cpp:10), so the second event completes after everything run_model enqueued
    // (input copies, graphs and kernels, sampler, copy of the sampled ids).
    EngineCoreOutputs step(float* device_ms = nullptr)
    {
        std::vector<ScheduledRequest> scheduled = scheduler.schedule();
        if (device_ms != nullptr) {
            cudaEventRecord(begin, nullptr);
        }
        runner.run_model(scheduled);
        if (device_ms != nullptr) {
            cudaEventRecord(end, nullptr);
        }
        std::vector<SampledToken> sampled = runner.finish();
        if (device_ms != nullptr) {
            cudaEventSynchronize(end);
            cudaEventElapsedTime(device_ms, begin, end);
        }
        return scheduler.update(sampled);
    }

    void make_events()
    {
        if (cudaEventCreate(&begin) != cudaSuccess || cudaEventCreate(&end) != cudaSuccess) {
            throw std::runtime_error("cudaEventCreate failed");
        }
    }

    cudaEvent_t begin = nullptr;
    cudaEvent_t end = nullptr;

    ModelRunner runner;
    Scheduler scheduler;
};

std::vector<int> random_prompt(std::mt19937& rng, int n, int vocab)
{
    std::uniform_int_distribution<int> dist(0, vocab - 1);
    std::vector<int> ids(n);
    for (int& id : ids) {
        id = dist(rng);
    }
    return ids;
}

Request make_request(std::string id, std::vector<int> tokens, int max_output_tokens)
{
    Request r{};
    r.id = std::move(id);
    r.max_output_tokens = max_output_tokens;
    r.ignore_eos = true;
    r.token_ids = std::move(tokens);
    r.sample_params = SampleParams{.temperature = 0.f, .top_k = 0, .top_p = 1.f};
    return r;
}

double ms_since(Clock::time_point t0)
{
    return std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
}

int run_bench(const Args& a, const Config& config)
{
    Engine engine(config);
    const int vocab = engine.runner.model_config().vocab_size;
    std::mt19937 rng(a.seed + a.batch);

    // the same workload as the other arm: prompts such that decoding ends at `context` tokens
    const int total_steps = a.warmup + a.steps;
    const int prefill_steps = (a.batch * a.context + a.max_num_scheduled_tokens - 1) / a.max_num_scheduled_tokens + 2;
    const int prompt_len = a.context - total_steps - prefill_steps - 1;
    if (prompt_len < 1) {
        throw std::runtime_error("steps + warmup do not fit below the context length");
    }
    for (int i = 0; i < a.batch; i++) {
        engine.scheduler.add_request(
            make_request("b" + std::to_string(i), random_prompt(rng, prompt_len, vocab), a.context - prompt_len));
    }
    std::map<std::string, int> produced;
    int guard = 0;
    while (static_cast<int>(produced.size()) < a.batch) {
        for (const EngineCoreOutput& o : engine.step()) {
            produced[o.request_id] += static_cast<int>(o.new_token_ids.size());
        }
        if (++guard > 10000) {
            throw std::runtime_error("prefill did not finish");
        }
    }
    for (int i = 0; i < a.warmup; i++) {
        engine.step();
    }
    engine.make_events();
    std::vector<double> step_ms;
    step_ms.reserve(a.steps);
    double device_total_ms = 0.0;
    long tokens = 0;
    const auto t0 = Clock::now();
    for (int i = 0; i < a.steps; i++) {
        const auto s0 = Clock::now();
        float device_ms = 0.f;
        const EngineCoreOutputs outs = engine.step(&device_ms);
        step_ms.push_back(ms_since(s0));
        device_total_ms += device_ms;
        for (const EngineCoreOutput& o : outs) {
            tokens += static_cast<long>(o.new_token_ids.size());
        }
    }
    const double wall_ms = ms_since(t0);
    if (tokens != static_cast<long>(a.batch) * a.steps) {
        throw std::runtime_error("a timed step did not decode every request");
    }
    std::vector<std::string> ids;
    for (int i = 0; i < a.batch; i++) {
        ids.push_back("b" + std::to_string(i));
    }
    engine.scheduler.abort_requests(ids);

    // prefill: one prompt per step, different ids every time (the prefix cache would serve a repeated prompt)
    std::vector<double> prefill_ms;
    for (int it = 0; it < 3 + a.prefill_runs && a.prefill_tokens > 0; it++) {
        engine.scheduler.add_request(
            make_request("p" + std::to_string(it), random_prompt(rng, a.prefill_tokens, vocab), 1));
        const auto s0 = Clock::now();
        const EngineCoreOutputs outs = engine.step();
        const double ms = ms_since(s0);
        if (outs.size() != 1 || outs[0].finish_reason == FinishReason::kRunning) {
            throw std::runtime_error("prefill step did not finish its request");
        }
        if (it >= 3) {
            prefill_ms.push_back(ms);
        }
    }
    std::sort(prefill_ms.begin(), prefill_ms.end());
    std::vector<double> sorted = step_ms;
    std::sort(sorted.begin(), sorted.end());

    long bucket = 1;
    while (bucket < a.batch) {
        bucket *= 2;
    }
    std::printf(
        "{\"tokens\": %ld, \"steps\": %d, \"warmup\": %d, \"batch\": %d, \"context\": %d, \"prompt_len\": %d, "
        "\"wall_ms\": %.4f, \"device_ms_per_step\": %.5f, \"ms_per_step\": %.5f, \"median_ms_per_step\": %.5f, \"prefill_tokens\": %d, "
        "\"prefill_ms\": %.4f, \"h2d_bytes_per_step\": %ld, \"d2h_bytes_per_step\": %ld}\n",
        tokens, a.steps, a.warmup, a.batch, a.context, prompt_len, wall_ms, device_total_ms / a.steps,
        wall_ms / a.steps,
        sorted[sorted.size() / 2], a.prefill_tokens,
        prefill_ms.empty() ? 0.0 : prefill_ms[prefill_ms.size() / 2],
        // what csrc/executor/batch_buffer.cpp:60-165 uploads for B single-token entries: token ids, positions and
        // slot mapping padded to the graph bucket, query_start_loc (B+1), seq_lens, logits indices, the sampling
        // options (3 words per request), the token count, and the block-table rows the requests hold
        static_cast<long>(4L * (3L * bucket + (a.batch + 1) + a.batch + a.batch + 3L * a.batch + 1
                                + static_cast<long>(a.batch) * ((a.context + a.block_size - 1) / a.block_size))),
        static_cast<long>(4L * a.batch));
    return 0;
}

int run_serve(const Args& a, const Config& config)
{
    Engine engine(config);
    const int vocab = engine.runner.model_config().vocab_size;
    std::mt19937 rng(a.seed + a.batch);
    const int total = 3 * a.batch;
    int next_id = 0;
    auto add = [&]() {
        engine.scheduler.add_request(
            make_request("s" + std::to_string(next_id++), random_prompt(rng, a.prompt_len, vocab), a.max_tokens));
    };
    auto run = [&](int count, long& tokens, int& steps) {
        int added = 0;
        for (; added < std::min(a.batch, count); added++) {
            add();
        }
        while (engine.scheduler.has_requests()) {
            for (const EngineCoreOutput& o : engine.step()) {
                tokens += static_cast<long>(o.new_token_ids.size());
                if (o.finish_reason != FinishReason::kRunning && added < count) {
                    add();
                    added++;
                }
            }
            steps++;
        }
    };
    long warm_tokens = 0;
    int warm_steps = 0;
    run(a.batch, warm_tokens, warm_steps);
    long tokens = 0;
    int steps = 0;
    const auto t0 = Clock::now();
    run(total, tokens, steps);
    const double wall_ms = ms_since(t0);
    std::printf(
        "{\"output_tokens_per_s\": %.1f, \"total_tokens_per_s\": %.1f, \"requests\": %d, \"steps\": %d, "
        "\"wall_s\": %.3f, \"in_flight\": %d, \"prompt_len\": %d, \"outputs\": %d}\n",
        tokens * 1e3 / wall_ms, (tokens + static_cast<double>(total) * a.prompt_len) * 1e3 / wall_ms, total, steps,
        wall_ms / 1e3, a.batch, a.prompt_len, a.max_tokens);
    return 0;
}

int run_generate(const Args& a, const Config& config)
{
    Engine engine(config);
    std::ifstream in(a.prompts);
    if (!in) {
        throw std::runtime_error("cannot open " + a.prompts);
    }
    std::vector<std::vector<int>> prompts;
    for (std::string line; std::getline(in, line);) {
        std::istringstream ss(line);
        std::vector<int> ids;
        for (int v; ss >> v;) {
            ids.push_back(v);
        }
        if (!ids.empty()) {
            prompts.push_back(std::move(ids));
        }
    }
    std::map<std::string, std::vector<int>> out;
    for (std::size_t i = 0; i < prompts.size(); i++) {
        engine.scheduler.add_request(make_request("g" + std::to_string(i), prompts[i], a.max_tokens));
    }
    int guard = 0;
    while (engine.scheduler.has_requests()) {
        for (const EngineCoreOutput& o : engine.step()) {
            out[o.request_id].insert(out[o.request_id].end(), o.new_token_ids.begin(), o.new_token_ids.end());
        }
        if (++guard > 100000) {
            throw std::runtime_error("generation did not finish");
        }
    }
    for (std::size_t i = 0; i < prompts.size(); i++) {
        const std::vector<int>& ids = out["g" + std::to_string(i)];
        for (std::size_t j = 0; j < ids.size(); j++) {
            std::printf(j ? " %d" : "%d", ids[j]);
        }
        std::printf("\n");
    }
    return 0;
}

}

int main(int argc, char** argv)
{
    try {
        const Args a = parse(argc, argv);
        Config config;
        config.model_path = a.model;
        config.gpu_memory_utilization = a.gpu_memory_utilization;
        config.block_size = a.block_size;
        config.max_num_scheduled_tokens = a.max_num_scheduled_tokens;
        config.max_num_seqs = a.max_num_seqs;
        config.enable_prefix_caching = true;    // the reference's default
        config.enable_cuda_graph = a.cuda_graph;
        if (a.mode == "bench") {
            return run_bench(a, config);
        }
        if (a.mode == "serve") {
            return run_serve(a, config);
        }
        if (a.mode == "generate") {
            return run_generate(a, config);
        }
        throw std::runtime_error("unknown mode " + a.mode);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "reference_bench: %s\n", e.what());
        return 1;
    }
}
