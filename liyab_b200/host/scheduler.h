// The scheduler above the step function: it admits requests, cuts prompts into
// portions under a token budget, decodes, finishes and frees.
//
// One central loop owns the GPU (the reference has no central loop: every call
// runs on its caller's thread and a leader batches pending passes,
// src/core/engine.cpp:1483-1540, 1842-2041; what is kept of it is what a pass may
// hold: prompt portions of some sequences beside single decode tokens of others,
// engine.cpp:2017-2030, and the finishing rules of the generation loop,
// engine.cpp:4351-4393).
//
// Decisions, all made on the host from the cache manager's accounting, so they
// run and are tested without a GPU:
//
// * Every unfinished request has `tokens` (prompt + generated so far) of which
//   `n_computed` are in the cache; it always has at least one token pending.  A
//   request whose pending tokens all fit a step gets a new token sampled at the
//   end of that step.
// * A step's token budget (`max_batched_tokens`) is spent first on requests with
//   one pending token (decoding), then on running requests in the middle of a
//   prompt, then on newly admitted ones; the last portion is cut to what is left
//   of the budget, down to a single token.
// * A waiting request is admitted, first come first served, while fewer than
//   `max_requests` are running and the free pages, after what the step already
//   plans to take, would hold its whole prompt plus one token.
// * When pages run out for the tokens that running requests need, the most
//   recently admitted running request is preempted: its pages are given back and
//   it returns to the front of the waiting queue, to be recomputed later from its
//   prompt and the tokens it had generated (its random draws are indexed by
//   position in its own stream, so it continues exactly as if never preempted).
//   A request that is alone and still cannot get a page can never finish: it ends
//   with CONTEXT_FULL.  (The reference fails the pass and clears that sequence's
//   context, src/core/transformer.cpp:6652-6654, src/core/engine.cpp:3878-3882.)
// * A request finishes on its end-of-sequence token (unless told to ignore it),
//   at `max_tokens`, when its sequence fills the model's positions, when its
//   callback returns false, or when cancelled; its pages and state slot are freed
//   at once.  The last sampled token is returned but never run, as in the
//   reference (engine.cpp:4388-4393).
// * A step is accounted for in two halves, so that the host can run one step ahead of
//   the GPU: `begin_step` (right after the step is launched) advances every request and
//   appends a placeholder for each token the step will sample; `finish_step` (when the
//   sampled ids have arrived) puts the real tokens in, calls callbacks and finishes
//   requests.  Between the two, the next step may already be planned and launched with
//   the placeholders standing for tokens that are still on the device.  What the length
//   limits decide is known at `begin_step`; what depends on a token's value (end of
//   sequence, a callback's verdict) is decided at `finish_step`, one step later, so a
//   request may have run one token too many; that token is dropped.  `update` is both
//   halves at once.
#pragma once

#include <deque>
#include <functional>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "cache.h"
#include "sampling.h"

namespace liyab {

constexpr int32_t kPlaceholder = -1;     // stands in a request's tokens for an id sampled by a step whose result is not back yet

enum class RequestState { Waiting, Running, Finished };
enum class FinishReason { None = 0, Eos = 1, Length = 2, Context = 3, Stopped = 4, Cancelled = 5, Failed = 6 };
const char* finish_reason_name(FinishReason r);

struct Request {
    RequestId id = 0;
    std::vector<int32_t> prompt;
    SamplingParams params;
    std::function<bool(int32_t)> callback;          // called with each new token; false stops
    RequestState state = RequestState::Waiting;
    std::vector<int32_t> tokens;                    // prompt + generated
    int64_t n_computed = 0;                         // tokens already in the cache
    FinishReason finish_reason = FinishReason::None;
    std::optional<Error> error;
    bool cancelled = false;
    int preemptions = 0;
    uint64_t seed = 0, stream = 0;
    int64_t admitted_at = -1;
    int sample_slot = -1;                           // where the step in flight will put this request's token

    int64_t generated_count() const { return static_cast<int64_t>(tokens.size() - prompt.size()); }
    int64_t pending() const { return static_cast<int64_t>(tokens.size()) - n_computed; }
    // The draw for this request's next generated token.
    double next_uniform() const { return uniform_draw(seed, stream, static_cast<uint64_t>(generated_count())); }
};

struct PlannedEntry {
    Request* request = nullptr;
    int64_t start = 0;          // first token of the portion (index into request->tokens)
    int64_t count = 0;
    bool sample = false;        // the portion ends the known tokens: a new token is sampled after it
    int64_t token_index = -1;   // where in request->tokens the sampled token goes (set by begin_step)
    FinishReason ends = FinishReason::None;      // the length limit that this very token reaches, if any (set by begin_step)
};

struct StepPlan {
    std::vector<PlannedEntry> entries;
    std::vector<Request*> preempted;
    int64_t n_tokens() const;
};

struct SchedulerStats {
    uint64_t steps = 0, batched_tokens = 0, prefill_tokens = 0, decode_tokens = 0, preemptions = 0, finished = 0;
    int peak_running = 0;
    // Steps by the number of tokens they batched: 1, 2-8, 9-32, 33-128, 129-512, 513-2048, more.
    uint64_t histogram[7] = {0, 0, 0, 0, 0, 0, 0};
};

class Scheduler {
public:
    Scheduler(CacheManager& cache, int64_t max_positions, int max_batched_tokens, int max_requests, std::optional<int64_t> eos_token_id);

    void add(Request* request);                     // the caller owns the request and keeps it alive until it finishes
    bool has_work() const { return !waiting.empty() || !running.empty(); }
    void cancel(RequestId id);
    void cancel_all();
    // The next step, and (in `finished`) the requests that ended while planning (cancelled, or that can never fit).
    StepPlan plan(std::vector<Request*>* finished);
    void begin_step(StepPlan& plan);
    std::vector<Request*> finish_step(StepPlan& plan, const std::vector<int32_t>& sampled);
    std::vector<Request*> update(StepPlan& plan, const std::vector<int32_t>& sampled);
    // Ends a request from outside a step (an engine failure).
    void fail(Request* r, const Error& error);

    CacheManager& cache;
    int64_t max_positions;
    int max_batched_tokens;
    int max_requests;
    std::optional<int64_t> eos_token_id;
    std::deque<Request*> waiting;
    std::vector<Request*> running;
    SchedulerStats stats;

private:
    void finish(Request* r, FinishReason reason, std::optional<Error> error = std::nullopt);
    void preempt(Request* r);
    bool fits(const std::vector<std::pair<Request*, int64_t>>& wants) const;

    int64_t admissions_ = 0;
    uint64_t streams_ = 0;
};

}  // namespace liyab
