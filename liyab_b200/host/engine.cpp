#include "engine.h"

#include <chrono>
#include <cstring>

#include "kernels.h"
#include "log.h"

namespace liyab {
namespace {
double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
}  // namespace

LoadedModel::LoadedModel(const std::string& model_dir, const std::string& dtype, int device) {
    const DType compute = compute_dtype_from_name(dtype);
    dtype_name = liyab::dtype_name(compute);
    int count = 0;
    const cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count == 0)
        throw backend_error("no CUDA device is available ({}); the engine has no CPU path", err != cudaSuccess ? cudaGetErrorString(err) : "none found");
    if (device < 0 || device >= count) throw backend_error("CUDA device {} does not exist ({} found)", device, count);
    LIYAB_CUDA(cudaSetDevice(device));
    config = read_config(model_dir);
    runtime.dtype = compute;
    runtime.device = device;
    LIYAB_CUDA(cudaDeviceGetAttribute(&runtime.sm_count, cudaDevAttrMultiProcessorCount, device));
    LIYAB_CUDA(cudaStreamCreateWithFlags(&runtime.stream, cudaStreamNonBlocking));
    const auto host = load_parameters(model_dir, *config, compute);
    weights = std::make_unique<WeightStore>(host);
    model = std::make_unique<DecoderModel>(config->model_spec(), weights->params(), runtime);
}

LoadedModel::~LoadedModel() {
    if (runtime.stream != nullptr) {
        cudaStreamSynchronize(runtime.stream);
        model.reset();
        cudaStreamDestroy(runtime.stream);
    }
}

Engine::Engine(const EngineConfig& cfg) : config(cfg) {
    if (cfg.model.empty()) throw invalid_argument("the engine configuration needs model_path (a model folder)");
    if (cfg.max_requests <= 0 || cfg.max_batched_tokens <= 0 || cfg.page_size <= 0)
        throw invalid_argument("max_requests, max_batched_tokens and page_size must be positive");
    const double t0 = now_ms();
    loaded_ = std::make_unique<LoadedModel>(cfg.model, cfg.dtype, cfg.device);
    DecoderModel& model = *loaded_->model;
    max_positions = model.max_positions();
    if (cfg.context_length > 0) max_positions = std::min<int64_t>(max_positions, cfg.context_length);
    const auto kv_needs = model.kv_needs();
    const auto state_needs = model.state_needs();
    int num_pages = cfg.num_pages;
    if (num_pages <= 0) {
        const CacheManager probe(kv_needs, state_needs, cfg.page_size, 1, 1, model.runtime.dtype, false);
        const size_t per_page = std::max<size_t>(1, probe.bytes_per_token() * static_cast<size_t>(cfg.page_size));
        const int64_t want = static_cast<int64_t>(cfg.max_requests) * ((max_positions + cfg.page_size - 1) / cfg.page_size);
        size_t free_bytes = 0, total_bytes = 0;
        LIYAB_CUDA(cudaMemGetInfo(&free_bytes, &total_bytes));
        // What the steps' scratch will take is set aside before the cache is sized from what is free.
        const size_t scratch = static_cast<size_t>(cfg.max_batched_tokens) * static_cast<size_t>(model.spec.hidden()) * 64 +
                               static_cast<size_t>(cfg.max_requests) * static_cast<size_t>(model.spec.vocab_size()) * 8;
        const size_t usable = free_bytes > scratch ? free_bytes - scratch : 0;
        num_pages = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, static_cast<int64_t>(static_cast<double>(usable) * cfg.kv_memory_fraction / static_cast<double>(per_page)))));
    }
    cache_ = std::make_unique<CacheManager>(kv_needs, state_needs, cfg.page_size, num_pages, cfg.max_requests, model.runtime.dtype, true);
    StepperOptions so;
    so.max_step_tokens = cfg.max_batched_tokens;
    so.max_logit_rows = cfg.max_requests;
    so.cuda_graphs = cfg.cuda_graphs;
    so.fused_decode = cfg.fused_decode;
    so.max_positions = static_cast<int>(max_positions);
    stepper_ = std::make_unique<Stepper>(model, *cache_, so);
    if (cfg.profile_phases) stepper_->set_phase_timer(&phase_timer_, phase_totals_);
    scheduler_ = std::make_unique<Scheduler>(*cache_, max_positions, cfg.max_batched_tokens, cfg.max_requests, model.spec.eos_token_id);
    sampler_ = std::make_unique<DeviceSampler>(model.runtime.stream, cfg.max_requests);
    kernels::status_words_clear(model.runtime.stream);
    load_ms = now_ms() - t0;
    log(LogLevel::Info, "{} (loaded in {:.0f} ms)", describe(), load_ms);
}

std::string Engine::describe() const {
    const ModelSpec& s = loaded_->model->spec;
    int pages = 0;
    for (const auto& g : cache_->groups) pages += g.pool.num_pages();
    return std::format("{}: {} layers, width {}, vocab {}, {} positions, {}, weights {:.1f} MiB, cache {} pages x {} positions ({} B/position), "
                       "up to {} requests, {} tokens a step",
                       s.architecture, s.run_order.size(), s.hidden(), s.vocab_size(), max_positions, loaded_->dtype_name,
                       static_cast<double>(loaded_->model->weight_bytes()) / 1048576.0, pages, cache_->page_size, cache_->bytes_per_token(),
                       config.max_requests, config.max_batched_tokens);
}

EngineCounters Engine::counters() const {
    EngineCounters c;
    c.scheduler = scheduler_->stats;
    c.steps = stepper_->steps;
    c.graph_steps = stepper_->graph_steps;
    c.fused_steps = stepper_->fused_steps;
    c.eager_steps = stepper_->eager_steps;
    c.graphs_captured = stepper_->graphs_captured;
    c.kernel_launches = kernels::launches.load();
    for (const auto& g : cache_->groups) {
        c.pages_in_use += g.pool.held_count();
        c.pages_total += g.pool.num_pages();
    }
    c.h2d_bytes = h2d_bytes_;
    c.d2h_bytes = d2h_bytes_;
    c.device_faults = device_faults_;
    return c;
}

GenerationResult Engine::generate_tokens(const std::vector<int32_t>& tokens, const SamplingParams& params, std::function<bool(int32_t)> callback) {
    return generate_batch({GenerationRequest{tokens, params, std::move(callback)}})[0];
}

std::vector<GenerationResult> Engine::generate_batch(const std::vector<GenerationRequest>& requests) {
    std::unique_lock<std::mutex> lock(busy_, std::try_to_lock);
    if (!lock.owns_lock()) throw make_error(Code::Busy, "the engine is already generating; one call at a time");
    LIYAB_CUDA(cudaSetDevice(config.device));
    cancel_requested_.store(false);
    const int64_t vocab = loaded_->model->spec.vocab_size();
    std::vector<std::unique_ptr<Request>> owned;
    for (const auto& g : requests) {
        for (const int32_t t : g.prompt)
            if (t < 0 || t >= vocab) throw invalid_argument("a prompt has a token id outside [0, {})", vocab);
        auto r = std::make_unique<Request>();
        r->id = next_id_++;
        r->prompt = g.prompt;
        r->params = g.params;
        r->callback = g.callback;
        owned.push_back(std::move(r));
    }
    std::vector<Request*> watch;
    try {
        for (auto& r : owned) {
            scheduler_->add(r.get());
            watch.push_back(r.get());
        }
        times_.clear();
        run(watch);
    } catch (...) {
        // Nothing of a failed call stays behind: its requests leave the queues and give their pages back.
        for (Request* r : watch)
            if (r->state != RequestState::Finished) scheduler_->fail(r, internal_error("the call failed"));
        cudaStreamSynchronize(loaded_->runtime.stream);
        throw;
    }
    std::vector<GenerationResult> out;
    for (auto& r : owned) out.push_back(result_of(*r, times_[r->id]));
    return out;
}

void Engine::run(const std::vector<Request*>& watch) {
    // With `pipeline` the host runs one step ahead of the GPU: step n+1 is planned, laid out and launched
    // while step n computes; the ids step n samples go into step n+1's token array on the device, and
    // reach the host (for end-of-sequence checks, callbacks and the results) while step n+1 runs.
    // Every step still copies its layout from pinned host memory to the device and its ids back.
    Scheduler& sched = *scheduler_;
    t_start_ = t_last_ = now_ms();
    const bool pipelined = config.pipeline && !config.profile_phases;
    auto all_done = [&] {
        for (const Request* r : watch)
            if (r->state != RequestState::Finished) return false;
        return true;
    };
    Launched inflight;
    int idle = 0;
    while (true) {
        if (cancel_requested_.exchange(false)) sched.cancel_all();
        Launched launched;
        bool progressed = inflight.valid;
        if (sched.has_work() && !all_done()) {
            StepPlan plan = sched.plan(nullptr);
            if (!plan.entries.empty()) {
                launched = launch(std::move(plan));
                progressed = true;
                sched.begin_step(launched.plan);
                if (!pipelined) {
                    resolve(launched);
                    launched = Launched{};
                }
            }
        }
        if (inflight.valid) resolve(inflight);
        inflight = std::move(launched);
        if (!inflight.valid && (!sched.has_work() || all_done())) break;
        idle = progressed ? 0 : idle + 1;
        if (idle > 3) throw internal_error("the scheduler has work but plans no step");
    }
}

Engine::Launched Engine::launch(StepPlan plan) {
    // Lays the plan out, launches its kernels and its sampling, and starts the copy of the ids to the host.
    Launched l;
    l.valid = true;
    l.plan = std::move(plan);
    std::vector<StepEntry> entries;
    std::vector<int32_t> want_storage(l.plan.entries.size());
    static const int32_t zero = 0;
    DeviceTokens dt;
    dt.source = sampler_->out_ids();
    bool on_device = false;
    l.decode_only = true;
    for (size_t i = 0; i < l.plan.entries.size(); ++i) {
        const PlannedEntry& e = l.plan.entries[i];
        const int32_t* toks = e.request->tokens.data() + e.start;
        StepEntry se;
        se.request = e.request->id;
        se.n_tokens = static_cast<int>(e.count);
        if (e.count == 1 && toks[0] < 0) {       // sampled by the step in flight: still on the device
            dt.index.push_back(e.request->sample_slot);
            se.tokens = &zero;
            on_device = true;
        } else {
            dt.index.push_back(-1);
            se.tokens = toks;
        }
        want_storage[i] = static_cast<int32_t>(e.count - 1);
        if (e.sample) {
            se.want = &want_storage[i];
            se.n_want = 1;
            l.sampling.push_back(e.request);
        }
        l.decode_only = l.decode_only && e.count == 1 && e.start + e.count > static_cast<int64_t>(e.request->prompt.size());
        entries.push_back(se);
    }
    std::vector<double> uniforms;
    std::vector<const SamplingParams*> params;
    for (const Request* r : l.sampling) {
        uniforms.push_back(r->next_uniform());
        params.push_back(&r->params);
    }
    const StepOutput out = stepper_->step(entries, on_device ? &dt : nullptr);
    h2d_bytes_ += static_cast<uint64_t>(l.plan.n_tokens()) * 4 * (3 + cache_->groups.size()) + entries.size() * 16;
    if (!l.sampling.empty()) {
        sampler_->sample(out.logits, params, uniforms);
        h2d_bytes_ += sampler_->h2d_bytes_last;
        for (size_t slot = 0; slot < l.sampling.size(); ++slot) l.sampling[slot]->sample_slot = static_cast<int>(slot);
    }
    l.ticket = sampler_->fetch_async(static_cast<int>(l.sampling.size()));
    d2h_bytes_ += l.sampling.size() * 4 + 8;
    return l;
}

void Engine::resolve(Launched& l) {
    // Waits for a launched step's ids and lets the scheduler finish the step.
    int status[2] = {0, 0};
    const std::vector<int32_t> ids = sampler_->wait(l.ticket, static_cast<int>(l.sampling.size()), status);
    const double now = now_ms();
    const double dt = now - t_last_;
    t_last_ = now;
    for (const PlannedEntry& e : l.plan.entries) {
        Timing& t = times_[e.request->id];
        const int64_t n_prompt = static_cast<int64_t>(e.request->prompt.size());
        const bool first = e.sample && e.token_index == n_prompt;
        if (e.start + e.count <= n_prompt || first) {
            t.prefill += dt;
            if (first) t.ttft = now - t_start_;
        } else {
            t.decode += dt;
            ++t.decode_steps;
            if (config.profile_phases && l.decode_only)
                for (int p = 0; p < static_cast<int>(Phase::Count); ++p) t.phases[p] += phase_totals_[p];
        }
    }
    if (config.profile_phases) std::memset(phase_totals_, 0, sizeof phase_totals_);
    if (status[0] != 0 || status[1] != 0) {
        // A bounded wait inside a kernel ran out: the step's numbers cannot be trusted.  Its requests end with an
        // error, the words are cleared, and a failing fused step is not used again.
        ++device_faults_;
        kernels::status_words_clear(loaded_->runtime.stream);
        if (status[1] != 0 && stepper_->has_fused()) stepper_->disable_fused();
        const Error err = internal_error("a kernel's bounded wait ran out (status words {:#x}, {:#x}); the step's requests end here{}", status[0],
                                         status[1], status[1] != 0 ? "; the one-kernel decode step is switched off" : "");
        log(LogLevel::Error, "{}", err.message());
        for (const PlannedEntry& e : l.plan.entries) scheduler_->fail(e.request, err);
        return;
    }
    scheduler_->finish_step(l.plan, ids);
}

GenerationResult Engine::result_of(const Request& r, const Timing& t) const {
    GenerationResult out;
    out.tokens.assign(r.tokens.begin() + static_cast<ptrdiff_t>(r.prompt.size()), r.tokens.end());
    while (!out.tokens.empty() && out.tokens.back() == kPlaceholder) out.tokens.pop_back();
    out.finish_reason = r.finish_reason;
    out.error = r.error;
    GenerationStats& s = out.stats;
    s.prompt_tokens = static_cast<int>(r.prompt.size());
    s.generated_tokens = static_cast<int>(out.tokens.size());
    s.prefill_ms = t.prefill;
    s.decode_ms = t.decode;
    s.ttft_ms = t.ttft;
    s.tokens_per_second = t.decode > 0 ? std::max(0, s.generated_tokens - 1) / (t.decode / 1e3) : 0.0;
    s.kv_cache_bytes = cache_->bytes_per_token() * (r.prompt.size() + out.tokens.size());
    s.cancelled = r.finish_reason == FinishReason::Cancelled;
    s.preemptions = r.preemptions;
    s.decode_steps = t.decode_steps;
    std::memcpy(s.phase_ms, t.phases, sizeof s.phase_ms);
    return out;
}

}  // namespace liyab
