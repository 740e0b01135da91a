// The engine: load a model folder, generate tokens.
//
// `Engine` mirrors the reference's public surface where it has one:
// `Engine::create(config)`, `generate_tokens(tokens, params, callback)`, `cancel`,
// `describe`, generation statistics (include/liyab/engine.h:634-1052,
// include/liyab/liyab_c_api.h:137-189, 223-275).  Token ids go in and come out;
// there is no tokenizer.  Several requests are served together by the scheduler
// (`generate_batch`), each with its own sampling options.
#pragma once

#include <atomic>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "arch.h"
#include "decoder.h"
#include "sampling.h"
#include "scheduler.h"
#include "step.h"
#include "weights.h"

namespace liyab {

// A model on the device: its configuration, its weights, its parts and the stream its kernels run on.
// The reference's load runs the same stages: describe, bind by name, size the cache, build
// (src/core/transformer.cpp:712-1046).
class LoadedModel {
public:
    LoadedModel(const std::string& model_dir, const std::string& dtype, int device);
    ~LoadedModel();
    LoadedModel(const LoadedModel&) = delete;
    LoadedModel& operator=(const LoadedModel&) = delete;

    std::unique_ptr<ArchitectureConfig> config;
    Runtime runtime;
    std::unique_ptr<WeightStore> weights;
    std::unique_ptr<DecoderModel> model;
    std::string dtype_name;
};

// Options of `Engine`; names follow the reference's engine config and command line where they exist
// (`context_length` is --ctx, tools/liyab_cli.cpp:242-334).
struct EngineConfig {
    std::string model;                  // folder with config.json and model.safetensors
    std::string dtype = "bfloat16";     // bfloat16 | float32
    int device = 0;
    int context_length = 0;             // 0: the model's positions
    int max_batched_tokens = 2048;      // token budget of one step
    int max_requests = 64;              // requests served together
    int page_size = 16;                 // positions per cache page
    int num_pages = 0;                  // 0: enough for max_requests full contexts, within kv_memory_fraction
    double kv_memory_fraction = 0.5;    // of the free device memory, at most, for the cache when num_pages is 0
    bool cuda_graphs = true;            // replay captured graphs for steps whose shape repeats
    bool fused_decode = false;          // decode steps of up to 16 requests as one persistent kernel (bfloat16), where it takes the model
    bool pipeline = true;               // plan and launch step n+1 while step n runs (tokens stay on the device)
    bool profile_phases = false;        // time every step's phases (steps then run part by part, one at a time)
};

// Per request, in the reference's names (include/liyab/liyab_c_api.h:137-189).
struct GenerationStats {
    int prompt_tokens = 0, generated_tokens = 0;
    double prefill_ms = 0, decode_ms = 0, ttft_ms = 0, tokens_per_second = 0;
    uint64_t kv_cache_bytes = 0;
    bool cancelled = false;
    int preemptions = 0;
    int decode_steps = 0;
    double phase_ms[static_cast<int>(Phase::Count)] = {0, 0, 0, 0, 0};      // decode steps only, when phases are profiled
};

struct GenerationRequest {
    std::vector<int32_t> prompt;
    SamplingParams params;
    std::function<bool(int32_t)> callback;
};

struct GenerationResult {
    std::vector<int32_t> tokens;
    FinishReason finish_reason = FinishReason::None;
    GenerationStats stats;
    std::optional<Error> error;
};

struct EngineCounters {
    SchedulerStats scheduler;
    uint64_t steps = 0, graph_steps = 0, fused_steps = 0, eager_steps = 0, graphs_captured = 0, kernel_launches = 0;
    int pages_in_use = 0, pages_total = 0;
    uint64_t h2d_bytes = 0, d2h_bytes = 0;       // copied by steps since the engine was created
    int device_faults = 0;                       // steps whose kernels reported a bounded wait that ran out
};

class Engine {
public:
    explicit Engine(const EngineConfig& config);

    // Serves all requests together; blocks until every one has finished.  BUSY when a call is already running.
    std::vector<GenerationResult> generate_batch(const std::vector<GenerationRequest>& requests);
    GenerationResult generate_tokens(const std::vector<int32_t>& tokens, const SamplingParams& params, std::function<bool(int32_t)> callback = {});
    // Thread-safe: the running call's requests stop at their next token.
    void cancel() { cancel_requested_.store(true); }
    // One line about the loaded model (the reference prints the like at load: src/core/transformer.cpp:880-884).
    std::string describe() const;
    EngineCounters counters() const;

    EngineConfig config;
    double load_ms = 0;
    int64_t max_positions = 0;
    LoadedModel& loaded() { return *loaded_; }
    CacheManager& cache() { return *cache_; }
    Stepper& stepper() { return *stepper_; }
    Scheduler& scheduler() { return *scheduler_; }

private:
    struct Launched {
        StepPlan plan;
        std::vector<Request*> sampling;
        int ticket = -1;
        bool valid = false;
        bool decode_only = false;
    };
    struct Timing { double prefill = 0, decode = 0, ttft = 0; int decode_steps = 0; double phases[static_cast<int>(Phase::Count)] = {0, 0, 0, 0, 0}; };

    void run(const std::vector<Request*>& watch);
    Launched launch(StepPlan plan);
    void resolve(Launched& l);
    GenerationResult result_of(const Request& r, const Timing& t) const;

    std::unique_ptr<LoadedModel> loaded_;
    std::unique_ptr<CacheManager> cache_;
    std::unique_ptr<Stepper> stepper_;
    std::unique_ptr<Scheduler> scheduler_;
    std::unique_ptr<DeviceSampler> sampler_;
    std::mutex busy_;
    std::atomic<bool> cancel_requested_{false};
    RequestId next_id_ = 0;
    std::map<RequestId, Timing> times_;
    double t_start_ = 0, t_last_ = 0;
    PhaseTimer phase_timer_;
    double phase_totals_[static_cast<int>(Phase::Count)] = {0, 0, 0, 0, 0};
    uint64_t h2d_bytes_ = 0, d2h_bytes_ = 0;
    int device_faults_ = 0;
};

}  // namespace liyab
