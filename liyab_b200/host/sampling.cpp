#include "sampling.h"

#include <cstring>
#include <random>

#include "kernels.h"

namespace liyab {

void SamplingParams::validate() const {
    if (max_tokens <= 0) throw invalid_argument("max_tokens must be positive (got {})", max_tokens);
    if (temperature != temperature || top_p != top_p) throw invalid_argument("temperature and top_p must be numbers");
    if (top_p <= 0 && temperature > 0) throw invalid_argument("top_p must be positive (got {})", top_p);
}

uint64_t SamplingParams::resolved_seed() const {
    if (seed != 0) return seed;
    std::random_device rd;
    return (static_cast<uint64_t>(rd()) << 32 | rd()) | 1;
}

double uniform_draw(uint64_t seed, uint64_t stream, uint64_t counter) {
    const uint64_t x = seed * 0x9E3779B97F4A7C15ull + stream * 0xD1B54A32D192ED03ull + counter * 0x8CB92BA72F3D8DD7ull;
    uint64_t z = x + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return static_cast<double>(z >> 11) * (1.0 / 9007199254740992.0);
}

DeviceSampler::DeviceSampler(cudaStream_t stream, int max_rows) : stream_(stream) { grow(std::max(1, max_rows)); }

void DeviceSampler::grow(int rows) {
    if (rows <= cap_) return;
    cap_ = rows;
    greedy_rows_ = 0;
    // [temperature f32 x cap | top_p f32 x cap | top_k i32 x cap | pad x cap | uniform f64 x cap] in one allocation, so that
    // one copy moves them all.  Two pinned staging buffers used in turn: one is rewritten only after the copy
    // that last read it has run on the device (the host may be a step ahead of the GPU).
    const size_t bytes = static_cast<size_t>(rows) * 6 * 4;
    for (int i = 0; i < 2; ++i) {
        hosts_[i] = PinnedBuffer(bytes);
        copied_[i] = std::make_unique<Event>();
        ticket_host_[i] = PinnedBuffer(static_cast<size_t>(rows) * 4 + 8);
        ticket_event_[i] = std::make_unique<Event>();
    }
    dev_ = DeviceBuffer(bytes);
    out_ids_ = DeviceBuffer(static_cast<size_t>(rows) * 4, true);
}

void DeviceSampler::sample(const Rows& logits, const std::vector<const SamplingParams*>& params, const std::vector<double>& uniforms) {
    const int n = static_cast<int>(params.size());
    grow(n);
    const size_t cap = static_cast<size_t>(cap_);
    bool all_greedy = true;
    for (const auto* p : params) all_greedy = all_greedy && p->temperature <= 0;
    h2d_bytes_last = 0;
    if (!(all_greedy && n <= greedy_rows_)) {
        turn_ = 1 - turn_;
        copied_[turn_]->synchronize();
        char* h = static_cast<char*>(hosts_[turn_].data());
        auto* temp = reinterpret_cast<float*>(h);
        auto* top_p = reinterpret_cast<float*>(h + cap * 4);
        auto* top_k = reinterpret_cast<int32_t*>(h + cap * 8);
        auto* uni = reinterpret_cast<double*>(h + cap * 16);
        for (int i = 0; i < n; ++i) {
            temp[i] = params[static_cast<size_t>(i)]->temperature;
            top_p[i] = params[static_cast<size_t>(i)]->top_p;
            top_k[i] = params[static_cast<size_t>(i)]->top_k;
            uni[i] = uniforms[static_cast<size_t>(i)];
        }
        for (int i = n; i < greedy_rows_; ++i) temp[i] = 0.0f;        // rows beyond n keep what the device believes of them
        LIYAB_CUDA(cudaMemcpyAsync(dev_.data(), h, cap * 24, cudaMemcpyHostToDevice, stream_));
        copied_[turn_]->record(stream_);
        h2d_bytes_last = cap * 24;
        greedy_rows_ = all_greedy ? n : 0;
    }
    char* d = static_cast<char*>(dev_.data());
    kernels::sample(stream_, logits.f32(), logits.stride, n, static_cast<int>(logits.cols), reinterpret_cast<const float*>(d),
                    reinterpret_cast<const int32_t*>(d + cap * 8), reinterpret_cast<const float*>(d + cap * 4),
                    reinterpret_cast<const double*>(d + cap * 16), static_cast<int32_t*>(out_ids_.data()));
}

int DeviceSampler::fetch_async(int n) {
    const int ticket = next_ticket_;
    next_ticket_ = 1 - ticket;
    char* host = static_cast<char*>(ticket_host_[ticket].data());
    if (n > 0) LIYAB_CUDA(cudaMemcpyAsync(host + 8, out_ids_.data(), static_cast<size_t>(n) * 4, cudaMemcpyDeviceToHost, stream_));
    kernels::status_words_fetch(stream_, reinterpret_cast<int*>(host));
    ticket_event_[ticket]->record(stream_);
    return ticket;
}

std::vector<int32_t> DeviceSampler::wait(int ticket, int n, int* status) {
    ticket_event_[ticket]->synchronize();
    const char* host = static_cast<const char*>(ticket_host_[ticket].data());
    if (status != nullptr) std::memcpy(status, host, 8);
    const auto* ids = reinterpret_cast<const int32_t*>(host + 8);
    return std::vector<int32_t>(ids, ids + n);
}

}  // namespace liyab
