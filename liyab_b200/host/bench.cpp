#include "bench.h"

#include <algorithm>
#include <chrono>

#include "kernels.h"

namespace liyab {
namespace {

uint64_t mix(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

std::vector<int32_t> random_ids(uint64_t seed, uint64_t stream, int n, int64_t vocab) {
    std::vector<int32_t> out(static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) out[static_cast<size_t>(i)] = static_cast<int32_t>(mix(seed * 0x632BE59BD9B4E019ull + stream * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(i)) % static_cast<uint64_t>(vocab));
    return out;
}

double wall_ms() { return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

}  // namespace

BenchResult bench_decode(Replayer& r, int batch, int prompt_len, int steps, int warmup, uint64_t seed) {
    if (batch <= 0 || steps <= 0 || prompt_len <= 0 || warmup < 0) throw invalid_argument("bench: batch, prompt_len and steps must be positive");
    LIYAB_CUDA(cudaSetDevice(r.loaded->runtime.device));
    DecoderModel& model = *r.loaded->model;
    CacheManager& cache = *r.cache;
    Stepper& stepper = *r.stepper;
    cudaStream_t stream = model.runtime.stream;
    const int64_t P = stepper.max_positions, V = model.spec.vocab_size();
    if (prompt_len >= P) throw invalid_argument("bench: prompts of {} tokens leave no position to decode at (the model has {})", prompt_len, P);
    DeviceSampler sampler(stream, batch);
    const SamplingParams greedy_params{0.0f, 0, 1.0f, 1, 1 << 30, true};
    const std::vector<const SamplingParams*> greedy(static_cast<size_t>(batch), &greedy_params);
    const std::vector<double> zeros(static_cast<size_t>(batch), 0.0);
    const RequestId base = 1'000'000;
    for (int i = 0; i < batch; ++i) cache.open(base + i);
    // Prompts, two at a time.
    const int32_t last = prompt_len - 1;
    for (int i = 0; i < batch; i += 2) {
        std::vector<std::vector<int32_t>> toks;
        std::vector<StepEntry> entries;
        for (int j = i; j < std::min(batch, i + 2); ++j) toks.push_back(random_ids(seed, static_cast<uint64_t>(j), prompt_len, V));
        for (size_t j = 0; j < toks.size(); ++j) entries.push_back({base + i + static_cast<int>(j), toks[j].data(), prompt_len, &last, 1});
        stepper.step(entries);
    }
    // Any valid ids start the decode loop; from then on they are the sampled ones.
    {
        std::vector<int32_t> ones(static_cast<size_t>(batch), 1);
        LIYAB_CUDA(cudaMemcpyAsync(sampler.out_ids_mutable(), ones.data(), ones.size() * 4, cudaMemcpyHostToDevice, stream));
        LIYAB_CUDA(cudaStreamSynchronize(stream));
    }
    DeviceTokens dt;
    dt.source = sampler.out_ids();
    for (int i = 0; i < batch; ++i) dt.index.push_back(i);
    static const int32_t zero = 0;
    std::vector<StepEntry> entries;
    for (int i = 0; i < batch; ++i) entries.push_back({base + i, &zero, 1, &zero, 1});
    int pending = -1;
    double ctx_sum = 0;
    uint64_t checksum = 0, h2d = 0;
    bool counting = false;
    auto one_step = [&] {
        // One decode step the way the engine runs it: the ids of the step before stay on the device and feed
        // this step; they are copied to the host while this step computes, and waited for after it is launched.
        if (cache.length(base) + 1 > P)
            for (int i = 0; i < batch; ++i) cache.truncate(base + i, prompt_len);
        for (int i = 0; i < batch; ++i) ctx_sum += static_cast<double>(cache.length(base + i) + 1);
        const StepOutput out = stepper.step(entries, &dt);
        sampler.sample(out.logits, greedy, zeros);
        h2d += sampler.h2d_bytes_last;
        const int ticket = sampler.fetch_async(batch);
        if (pending >= 0) {
            const auto ids = sampler.wait(pending, batch);
            if (counting)
                for (const int32_t id : ids) checksum = mix(checksum ^ static_cast<uint64_t>(id));
        }
        pending = ticket;
    };
    for (int i = 0; i < warmup; ++i) one_step();
    if (pending >= 0) sampler.wait(pending, batch);
    pending = -1;
    LIYAB_CUDA(cudaStreamSynchronize(stream));
    ctx_sum = 0;
    h2d = 0;
    counting = true;
    const uint64_t launches0 = kernels::launches.load(), graph0 = stepper.graph_steps, fused0 = stepper.fused_steps, eager0 = stepper.eager_steps;
    Event start(true), end(true);
    const double t0 = wall_ms();
    start.record(stream);
    for (int i = 0; i < steps; ++i) one_step();
    {
        const auto ids = sampler.wait(pending, batch);
        for (const int32_t id : ids) checksum = mix(checksum ^ static_cast<uint64_t>(id));
    }
    end.record(stream);
    end.synchronize();
    LIYAB_CUDA(cudaStreamSynchronize(stream));
    const double wall = wall_ms() - t0;
    float ms = 0;
    LIYAB_CUDA(cudaEventElapsedTime(&ms, start.get(), end.get()));
    BenchResult out;
    out.ms_total = ms;
    out.ms_per_step = ms / steps;
    out.wall_ms_per_step = wall / steps;
    out.mean_context = ctx_sum / (static_cast<double>(steps) * batch);
    out.kernel_launches = kernels::launches.load() - launches0;
    out.graph_steps = stepper.graph_steps - graph0;
    out.fused_steps = stepper.fused_steps - fused0;
    out.eager_steps = stepper.eager_steps - eager0;
    const size_t width = static_cast<size_t>((P + cache.page_size - 1) / cache.page_size);
    // layout arrays (tokens, positions, request of token, slots, map: 5 per token; starts, lengths, state slots, wanted row: 4 per
    // request + 1) and the block table, each piece rounded up to 16 bytes, plus the sampler's options when they travel
    out.h2d_bytes_per_step = 4 * (5 * ((static_cast<size_t>(batch) + 3) / 4 * 4) + 4 * ((static_cast<size_t>(batch) + 4) / 4 * 4) +
                                  static_cast<size_t>(batch) * width) + h2d / static_cast<uint64_t>(steps);
    out.d2h_bytes_per_step = 4 * static_cast<uint64_t>(batch) + 8;
    out.checksum = checksum;
    for (int i = 0; i < batch; ++i) cache.close(base + i);
    return out;
}

BenchResult bench_prefill(Replayer& r, int n_seq, int seq_len, int repeats, uint64_t seed) {
    if (n_seq <= 0 || seq_len <= 0 || repeats <= 0) throw invalid_argument("bench: n_seq, seq_len and repeats must be positive");
    LIYAB_CUDA(cudaSetDevice(r.loaded->runtime.device));
    DecoderModel& model = *r.loaded->model;
    CacheManager& cache = *r.cache;
    Stepper& stepper = *r.stepper;
    cudaStream_t stream = model.runtime.stream;
    const int64_t V = model.spec.vocab_size();
    const RequestId base = 2'000'000;
    const int32_t last = seq_len - 1;
    std::vector<double> times;
    const uint64_t graph0 = stepper.graph_steps, eager0 = stepper.eager_steps;
    uint64_t launches = 0;
    for (int it = 0; it < repeats + 2; ++it) {
        std::vector<std::vector<int32_t>> toks;
        std::vector<StepEntry> entries;
        for (int i = 0; i < n_seq; ++i) {
            cache.open(base + i);
            toks.push_back(random_ids(seed + static_cast<uint64_t>(it), static_cast<uint64_t>(i), seq_len, V));
        }
        for (int i = 0; i < n_seq; ++i) entries.push_back({base + i, toks[static_cast<size_t>(i)].data(), seq_len, &last, 1});
        Event start(true), end(true);
        LIYAB_CUDA(cudaStreamSynchronize(stream));
        const uint64_t l0 = kernels::launches.load();
        start.record(stream);
        stepper.step(entries);
        end.record(stream);
        end.synchronize();
        launches = kernels::launches.load() - l0;
        float ms = 0;
        LIYAB_CUDA(cudaEventElapsedTime(&ms, start.get(), end.get()));
        if (it >= 2) times.push_back(ms);
        for (int i = 0; i < n_seq; ++i) cache.close(base + i);
    }
    std::sort(times.begin(), times.end());
    BenchResult out;
    out.ms_per_step = times.front();
    out.wall_ms_per_step = times[times.size() / 2];
    out.ms_total = 0;
    for (const double t : times) out.ms_total += t;
    out.mean_context = seq_len;
    out.kernel_launches = launches;
    out.graph_steps = stepper.graph_steps - graph0;
    out.eager_steps = stepper.eager_steps - eager0;
    return out;
}

}  // namespace liyab
