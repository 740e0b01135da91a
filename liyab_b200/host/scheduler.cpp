#include "scheduler.h"

#include <algorithm>

namespace liyab {

const char* finish_reason_name(FinishReason r) {
    switch (r) {
        case FinishReason::None: return "unfinished";
        case FinishReason::Eos: return "eos";
        case FinishReason::Length: return "length";
        case FinishReason::Context: return "context";
        case FinishReason::Stopped: return "stopped";
        case FinishReason::Cancelled: return "cancelled";
        case FinishReason::Failed: return "error";
    }
    return "?";
}

int64_t StepPlan::n_tokens() const {
    int64_t n = 0;
    for (const auto& e : entries) n += e.count;
    return n;
}

Scheduler::Scheduler(CacheManager& cache_, int64_t max_positions_, int max_batched_tokens_, int max_requests_,
                     std::optional<int64_t> eos)
    : cache(cache_), max_positions(max_positions_), max_batched_tokens(max_batched_tokens_),
      max_requests(std::min(max_requests_, cache_.max_requests)), eos_token_id(eos) {
    if (max_batched_tokens <= 0 || max_requests_ <= 0) throw invalid_argument("max_batched_tokens and max_requests must be positive");
}

void Scheduler::add(Request* r) {
    r->params.validate();
    if (r->prompt.empty()) throw invalid_argument("request {} has an empty prompt", r->id);
    if (static_cast<int64_t>(r->prompt.size()) > max_positions)
        throw make_error(Code::ContextFull, "request {}: a prompt of {} tokens does not fit {} positions", r->id, r->prompt.size(), max_positions);
    r->tokens = r->prompt;
    r->n_computed = 0;
    r->state = RequestState::Waiting;
    r->finish_reason = FinishReason::None;
    r->seed = r->params.resolved_seed();
    r->stream = streams_++;
    waiting.push_back(r);
}

void Scheduler::cancel(RequestId id) {
    for (Request* r : running)
        if (r->id == id) r->cancelled = true;
    for (Request* r : waiting)
        if (r->id == id) r->cancelled = true;
}

void Scheduler::cancel_all() {
    for (Request* r : running) r->cancelled = true;
    for (Request* r : waiting) r->cancelled = true;
}

void Scheduler::finish(Request* r, FinishReason reason, std::optional<Error> error) {
    if (r->state == RequestState::Finished) {
        r->finish_reason = reason;
        return;
    }
    if (r->state == RequestState::Running) {
        running.erase(std::find(running.begin(), running.end(), r));
        cache.close(r->id);
    } else {
        const auto it = std::find(waiting.begin(), waiting.end(), r);
        if (it != waiting.end()) waiting.erase(it);
    }
    r->state = RequestState::Finished;
    r->finish_reason = reason;
    r->error = std::move(error);
    ++stats.finished;
}

void Scheduler::fail(Request* r, const Error& error) {
    if (!r->tokens.empty() && r->tokens.back() == kPlaceholder) r->tokens.pop_back();
    finish(r, FinishReason::Failed, error);
}

void Scheduler::preempt(Request* r) {
    running.erase(std::find(running.begin(), running.end(), r));
    cache.close(r->id);
    r->state = RequestState::Waiting;
    r->n_computed = 0;
    ++r->preemptions;
    waiting.push_front(r);
    ++stats.preemptions;
}

bool Scheduler::fits(const std::vector<std::pair<Request*, int64_t>>& wants) const {
    if (wants.empty()) return true;
    std::vector<int> rows;
    std::vector<int64_t> n;
    for (const auto& [r, count] : wants) {
        rows.push_back(cache.row_of(r->id));
        n.push_back(count);
    }
    return cache.can_reserve_rows(rows, n);
}

StepPlan Scheduler::plan(std::vector<Request*>* finished) {
    {
        std::vector<Request*> gone;
        for (Request* r : running)
            if (r->cancelled) gone.push_back(r);
        for (Request* r : waiting)
            if (r->cancelled) gone.push_back(r);
        for (Request* r : gone) {
            finish(r, FinishReason::Cancelled);
            if (finished != nullptr) finished->push_back(r);
        }
    }
    StepPlan plan;
    std::vector<std::pair<Request*, int64_t>> wants;
    int64_t budget = max_batched_tokens;
    while (true) {
        budget = max_batched_tokens;
        plan.entries.clear();
        wants.clear();
        std::vector<Request*> order;
        for (Request* r : running)
            if (r->pending() == 1) order.push_back(r);
        for (Request* r : running)
            if (r->pending() > 1) order.push_back(r);
        for (Request* r : order) {
            if (budget == 0) break;
            const int64_t n = std::min(r->pending(), budget);
            plan.entries.push_back({r, r->n_computed, n, n == r->pending()});
            wants.push_back({r, n});
            budget -= n;
        }
        if (fits(wants)) break;
        // Pages ran out for what running requests need: the most recently admitted one makes room.
        Request* victim = *std::max_element(running.begin(), running.end(),
                                            [](const Request* a, const Request* b) { return a->admitted_at < b->admitted_at; });
        if (running.size() == 1) {
            std::string free_text;
            for (const int f : cache.free_pages()) free_text += (free_text.empty() ? "" : ", ") + std::to_string(f);
            finish(victim, FinishReason::Failed,
                   make_error(Code::ContextFull, "request {} needs more pages than the cache has ({} tokens, {} pages free)", victim->id,
                              victim->n_computed + victim->pending(), free_text));
            if (finished != nullptr) finished->push_back(victim);
        } else {
            preempt(victim);
            plan.preempted.push_back(victim);
        }
    }
    // Admission: first come first served, only what fits whole.
    while (!waiting.empty() && static_cast<int>(running.size()) < max_requests && budget > 0 && plan.preempted.empty()) {
        Request* r = waiting.front();
        const int64_t n_tokens = static_cast<int64_t>(r->tokens.size());
        const int64_t whole = (std::min(n_tokens + 1, max_positions) + cache.page_size - 1) / cache.page_size;
        int64_t total_pages = whole;
        if (!cache.groups.empty()) {
            total_pages = cache.groups[0].pool.num_pages();
            for (const auto& g : cache.groups) total_pages = std::min<int64_t>(total_pages, g.pool.num_pages());
        }
        if (whole > total_pages) {
            finish(r, FinishReason::Failed,
                   make_error(Code::ContextFull, "request {}: {} tokens need {} pages, the cache has {}", r->id, n_tokens, whole, total_pages));
            if (finished != nullptr) finished->push_back(r);
            continue;
        }
        cache.open(r->id);
        const int64_t n = std::min(r->pending(), budget);
        auto probe = wants;
        probe.push_back({r, n_tokens < max_positions ? n_tokens + 1 : n_tokens});
        if (!fits(probe)) {
            cache.close(r->id);
            break;
        }
        waiting.pop_front();
        r->state = RequestState::Running;
        r->admitted_at = admissions_++;
        running.push_back(r);
        plan.entries.push_back({r, r->n_computed, n, n == r->pending()});
        wants.push_back({r, n});
        budget -= n;
    }
    stats.peak_running = std::max(stats.peak_running, static_cast<int>(running.size()));
    return plan;
}

void Scheduler::begin_step(StepPlan& plan) {
    ++stats.steps;
    const int64_t n = plan.n_tokens();
    stats.batched_tokens += static_cast<uint64_t>(n);
    const int bucket = n <= 1 ? 0 : n <= 8 ? 1 : n <= 32 ? 2 : n <= 128 ? 3 : n <= 512 ? 4 : n <= 2048 ? 5 : 6;
    ++stats.histogram[bucket];
    for (auto& e : plan.entries) {
        Request* r = e.request;
        r->n_computed += e.count;
        if (e.count == 1 && r->n_computed > static_cast<int64_t>(r->prompt.size())) ++stats.decode_tokens;
        else stats.prefill_tokens += static_cast<uint64_t>(e.count);
        if (!e.sample) continue;
        r->tokens.push_back(kPlaceholder);
        e.token_index = static_cast<int64_t>(r->tokens.size()) - 1;
        if (r->generated_count() >= r->params.max_tokens) e.ends = FinishReason::Length;
        else if (static_cast<int64_t>(r->tokens.size()) > max_positions) e.ends = FinishReason::Context;   // no position left to run the new token at
        if (e.ends != FinishReason::None) finish(r, e.ends);
    }
}

std::vector<Request*> Scheduler::finish_step(StepPlan& plan, const std::vector<int32_t>& sampled) {
    std::vector<Request*> done;
    size_t next = 0;
    for (auto& e : plan.entries) {
        if (!e.sample) continue;
        if (next >= sampled.size()) throw internal_error("a step sampled {} tokens, its plan wanted more", sampled.size());
        const int32_t token = sampled[next++];
        Request* r = e.request;
        if (e.token_index >= static_cast<int64_t>(r->tokens.size())) continue;      // the request ended on an earlier token; this one was one too many
        if (r->state == RequestState::Finished && r->finish_reason == FinishReason::Failed) continue;
        r->tokens[static_cast<size_t>(e.token_index)] = token;
        bool keep_going = true;
        if (r->callback) keep_going = r->callback(token);
        FinishReason reason = FinishReason::None;
        if (!r->params.ignore_eos && eos_token_id && token == *eos_token_id) reason = FinishReason::Eos;
        else if (e.ends != FinishReason::None) reason = e.ends;       // this token reached a length limit (known since begin_step)
        else if (!keep_going) reason = FinishReason::Stopped;
        else if (r->cancelled) reason = FinishReason::Cancelled;
        if (reason != FinishReason::None) {
            r->tokens.resize(static_cast<size_t>(e.token_index) + 1);       // drops a placeholder of the step after this one, if any
            finish(r, reason);
            done.push_back(r);
        }
    }
    return done;
}

std::vector<Request*> Scheduler::update(StepPlan& plan, const std::vector<int32_t>& sampled) {
    begin_step(plan);
    return finish_step(plan, sampled);
}

}  // namespace liyab
