// Sampling options, the engine's random draws and the batched next-token choice
// on the device.
//
// Names, meanings and defaults are the reference's `SamplingParams`
// (include/liyab/types.h:215-222; C mirror include/liyab/liyab_c_api.h:128-135):
// temperature <= 0 is greedy, top_k <= 0 and top_p >= 1 switch those cuts off, seed
// 0 picks a random seed.  `ignore_eos` is an addition for benchmarks, where a fixed
// number of tokens must be generated.
//
// The reference draws from std::mt19937_64 (src/core/sampling.cpp:9-10, 66-69); a
// sampler on the GPU cannot share that stream, so draws here are counter-based:
// uniform(seed, stream, counter) is SplitMix64 of a key built from the three, top
// 53 bits scaled by 2^-53.  A request's n-th draw is therefore the same number
// whatever the batch it is drawn in, and after a preemption too.
//
// One kernel launch picks a token for every row of logits, each row with its own
// temperature, top-k, top-p and uniform draw (csrc/sampling.cu restates the
// reference's sampler, src/core/sampling.cpp:16-79).  The per-row options travel
// in one pinned staging buffer per step.
#pragma once

#include <cstdint>
#include <memory>
#include <vector>

#include "device.h"

namespace liyab {

struct SamplingParams {
    float temperature = 0.8f;     // <= 0 selects greedy decoding
    int32_t top_k = 40;           // <= 0 disables
    float top_p = 0.95f;          // >= 1 disables
    uint64_t seed = 0;            // 0 picks a random seed
    int32_t max_tokens = 256;
    bool ignore_eos = false;

    void validate() const;
    bool greedy() const { return temperature <= 0.0f; }
    uint64_t resolved_seed() const;      // the seed itself, or a random one when it is 0
};

// The `counter`-th draw in [0, 1) of stream `stream` under `seed`.
double uniform_draw(uint64_t seed, uint64_t stream, uint64_t counter);

class DeviceSampler {
public:
    DeviceSampler(cudaStream_t stream, int max_rows);

    // Token ids (int32, on the device: out_ids()) for rows 0 .. n-1 of `logits`.
    void sample(const Rows& logits, const std::vector<const SamplingParams*>& params, const std::vector<double>& uniforms);
    const int32_t* out_ids() const { return static_cast<const int32_t*>(out_ids_.data()); }
    int32_t* out_ids_mutable() { return static_cast<int32_t*>(out_ids_.data()); }
    // Starts copying the last `n` sampled ids (and the device status words) to the host; returns a ticket for
    // `wait`.  Two tickets are live at most: the one before last must have been waited for.
    int fetch_async(int n);
    // The ids of the ticket; `status` (two ints) receives the status words fetched with them.
    std::vector<int32_t> wait(int ticket, int n, int* status = nullptr);
    size_t h2d_bytes_last = 0;

private:
    void grow(int rows);
    cudaStream_t stream_;
    int cap_ = 0;
    int greedy_rows_ = 0;        // leading rows of the device options known to be greedy
    PinnedBuffer hosts_[2];
    std::unique_ptr<Event> copied_[2];
    int turn_ = 0;
    DeviceBuffer dev_, out_ids_;
    PinnedBuffer ticket_host_[2];
    std::unique_ptr<Event> ticket_event_[2];
    int next_ticket_ = 0;
};

}  // namespace liyab
