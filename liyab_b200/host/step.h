// The one step function: a batch of (request, its next tokens) in, logits at
// the wanted places out.
//
// A step may hold portions of prompts beside single decoded tokens, cut anywhere.
// It runs only the tokens it is given, as one flat batch, against what earlier
// steps left in the cache, and then makes every request longer by what it brought.
// This is the reference's `forward_batch` (src/core/transformer.h:731-764,
// src/core/transformer.cpp:6589-6769): items of 1..n tokens appended at each
// sequence's own n_past, pages mapped for every item before any compute so that a
// failure leaves every position as it was (:6652-6654), n_past advanced after all
// blocks ran (:6726-6735), logits only for the rows asked for (:6739-6767).
// Refusals follow :6596-6624: an empty batch or item, a token id outside the
// vocabulary, a request named twice; plus an unknown request and a sequence that
// would pass the model's positions (ContextFull, :2791-2808).
//
// Three ways to run the model, chosen per step: the one-kernel fused step (decode
// steps of up to 16 tokens of a model made of the standard parts, bfloat16), a
// captured CUDA graph (decode steps of any size; any step shape that came up three
// times; only for models whose parts are all capturable), or part by part
// (everything else, all of float32).  The kernels and the cache are the same.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <tuple>
#include <vector>

#include "decoder.h"
#include "fused_decode.h"

namespace liyab {

// A request's next tokens and the places among them whose logits are wanted (views; the caller keeps them alive).
struct StepEntry {
    RequestId request = 0;
    const int32_t* tokens = nullptr;
    int n_tokens = 0;
    const int32_t* want = nullptr;
    int n_want = 0;
};

// Tokens of a step that are still on the device: entry i's (single) token is source[index[i]] where
// index[i] >= 0; other entries bring their tokens from the host as usual.
struct DeviceTokens {
    const int32_t* source = nullptr;        // int32 on the device, e.g. the ids the previous step sampled
    std::vector<int32_t> index;
};

struct StepOutput {
    Rows logits;                                            // [R, vocab] float32 on the device; valid until the next step
    std::vector<std::pair<RequestId, int>> rows;            // (request, index among its tokens) per row
};

struct StepperOptions {
    int max_step_tokens = 0;        // scratch is sized for this many tokens up front (0: grows on demand)
    int max_logit_rows = 0;         // and for this many wanted rows
    bool cuda_graphs = false;
    bool fused_decode = false;
    int max_positions = 0;          // 0: the model's
};

class Stepper {
public:
    Stepper(DecoderModel& model, CacheManager& cache, const StepperOptions& options);
    ~Stepper();

    StepOutput step(const std::vector<StepEntry>& entries, const DeviceTokens* device_tokens = nullptr);
    // Checks a step before anything is touched; fills the requests' rows and token counts.
    void validate(const std::vector<StepEntry>& entries, const DeviceTokens* device_tokens, std::vector<int>* rows,
                  std::vector<int64_t>* q_len) const;
    // Parts' outputs of every later step are shown to `tap` (steps then run part by part); empty removes it.
    void set_tap(TapFn tap) { tap_ = std::move(tap); }
    // With a timer, every later step runs part by part with its phases timed into `totals` (Phase::Count doubles).
    void set_phase_timer(PhaseTimer* timer, double* totals) { phases_ = timer; phase_totals_ = totals; }

    DecoderModel& model;
    CacheManager& cache;
    Workspace workspace;
    bool cuda_graphs;
    int max_positions;
    bool has_fused() const { return fused_ != nullptr; }
    void disable_fused() { fused_.reset(); }
    FusedDecodeStack* fused() { return fused_.get(); }
    // counters
    uint64_t steps = 0, graph_steps = 0, fused_steps = 0, eager_steps = 0, tokens_run = 0, graphs_captured = 0;

private:
    using ShapeKey = std::tuple<int, int, int, int>;        // requests, tokens, wanted rows, bucket of the longest portion
    struct CapturedStep {
        DeviceBuffer layout;
        size_t layout_ints = 0;
        cudaGraphExec_t exec = nullptr;
        Rows logits;
        uint64_t generation = 0;
        uint64_t launches = 0;
        uint64_t last_used = 0;
    };
    struct Layout {
        StepContext ctx;
        std::vector<std::pair<RequestId, int>> out_rows;
    };

    ShapeKey shape_key(const std::vector<StepEntry>& entries, const std::vector<int64_t>& q_len) const;
    bool worth_capturing(const std::vector<StepEntry>& entries, const std::vector<int64_t>& q_len);
    Rows graph_step(const std::vector<StepEntry>& entries, const std::vector<int>& rows, const std::vector<int64_t>& q_len,
                    const DeviceTokens* dt, Layout* layout);
    void lay_out(const std::vector<StepEntry>& entries, const std::vector<int>& rows, const std::vector<int64_t>& q_len,
                 const DeviceTokens* dt, CapturedStep* fixed, int max_q_len, Layout* out);
    void drop_graph(CapturedStep& g);

    std::unique_ptr<FusedDecodeStack> fused_;
    std::map<ShapeKey, CapturedStep> graphs_;
    std::map<ShapeKey, int> seen_;
    PinnedBuffer host_[2];
    std::unique_ptr<Event> copied_[2];
    DeviceBuffer dev_;
    int turn_ = 0;
    TapFn tap_;
    PhaseTimer* phases_ = nullptr;
    double* phase_totals_ = nullptr;
    bool model_capturable_ = false;
};

}  // namespace liyab
