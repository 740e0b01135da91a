#include "step.h"

#include <algorithm>
#include <cstring>
#include <set>

#include "kernels.h"
#include "log.h"

namespace liyab {

Stepper::Stepper(DecoderModel& model_, CacheManager& cache_, const StepperOptions& o)
    : model(model_), cache(cache_), cuda_graphs(o.cuda_graphs),
      max_positions(static_cast<int>(std::min<int64_t>(o.max_positions > 0 ? o.max_positions : model_.max_positions(), model_.max_positions()))) {
    if (o.max_step_tokens > 0) workspace.reserve_rows(o.max_step_tokens);
    if (o.max_logit_rows > 0 && model.runtime.stream != nullptr) {
        // The head's buffers at their final size, so that captured steps keep their addresses.
        workspace.get("head.normed", o.max_logit_rows, model.spec.hidden(), model.runtime.dtype, false);
        workspace.get("logits", o.max_logit_rows, model.spec.vocab_size(), DType::F32, false);
    }
    cache.stream = model.runtime.stream;
    model_capturable_ = model.capturable();
    // Decode steps of a few tokens go to the one-kernel path where the model is made of standard parts.
    if (o.fused_decode) fused_ = FusedDecodeStack::try_build(model, cache);
}

Stepper::~Stepper() {
    for (auto& kv : graphs_) drop_graph(kv.second);
}

void Stepper::drop_graph(CapturedStep& g) {
    if (g.exec != nullptr) cudaGraphExecDestroy(g.exec);
    g.exec = nullptr;
}

void Stepper::validate(const std::vector<StepEntry>& entries, const DeviceTokens* dt, std::vector<int>* rows,
                       std::vector<int64_t>* q_len) const {
    if (entries.empty()) throw invalid_argument("a step needs at least one entry");
    const size_t S = entries.size();
    rows->resize(S);
    q_len->resize(S);
    const int64_t vocab = model.spec.vocab_size();
    if (dt != nullptr && dt->index.size() != S) throw invalid_argument("device tokens must name one source per entry");
    std::set<int> seen;
    for (size_t i = 0; i < S; ++i) {
        const StepEntry& e = entries[i];
        (*rows)[i] = cache.row_of(e.request);
        if (!seen.insert((*rows)[i]).second) throw invalid_argument("request {} appears twice in one step", e.request);
        if (e.n_tokens <= 0) throw invalid_argument("request {} brings no tokens", e.request);
        (*q_len)[i] = e.n_tokens;
        const bool on_device = dt != nullptr && dt->index[i] >= 0;
        if (on_device && e.n_tokens != 1) throw invalid_argument("a token can stay on the device only as the single token of its request");
        if (!on_device)
            for (int t = 0; t < e.n_tokens; ++t)
                if (e.tokens[t] < 0 || e.tokens[t] >= vocab)
                    throw invalid_argument("request {} has a token id outside [0, {})", e.request, vocab);
        const int64_t reach = cache.length_of_row[static_cast<size_t>((*rows)[i])] + e.n_tokens;
        if (reach > max_positions)
            throw make_error(Code::ContextFull, "request {} would reach {} tokens; the model has {} positions", e.request, reach, max_positions);
        for (int w = 0; w < e.n_want; ++w)
            if (e.want[w] < 0 || e.want[w] >= e.n_tokens)
                throw invalid_argument("request {} wants logits at {}, outside its {} tokens", e.request, e.want[w], e.n_tokens);
    }
}

StepOutput Stepper::step(const std::vector<StepEntry>& entries, const DeviceTokens* dt) {
    std::vector<int> rows;
    std::vector<int64_t> q_len;
    validate(entries, dt, &rows, &q_len);
    cache.reserve_rows(rows, q_len);         // all or nothing: throws OutOfPages and takes no page
    Layout layout;
    Rows logits;
    try {
        bool decode = true;
        int64_t tokens = 0;
        for (size_t i = 0; i < entries.size(); ++i) {
            decode = decode && q_len[i] == 1 && entries[i].n_want == 1;
            tokens += q_len[i];
        }
        const bool tapped = static_cast<bool>(tap_) || phases_ != nullptr;
        if (decode && !tapped && fused_ != nullptr && fused_->accepts(static_cast<int>(entries.size()))) {
            lay_out(entries, rows, q_len, dt, nullptr, 0, &layout);
            logits = fused_->run(layout.ctx);
            ++fused_steps;
        } else if (cuda_graphs && !tapped && model_capturable_ && (decode || worth_capturing(entries, q_len))) {
            logits = graph_step(entries, rows, q_len, dt, &layout);
        } else {
            lay_out(entries, rows, q_len, dt, nullptr, 0, &layout);
            if (tap_) layout.ctx.tap_fn = &tap_;
            if (phases_ != nullptr) {
                phases_->begin_step();
                layout.ctx.phases = phases_;
            }
            logits = model.forward(layout.ctx);
            if (phases_ != nullptr) phases_->end_step(model.runtime.stream, phase_totals_);
            ++eager_steps;
        }
        tokens_run += static_cast<uint64_t>(tokens);
    } catch (...) {
        cache.rollback_rows(rows);           // the step did not happen: every position as it was
        throw;
    }
    cache.commit_rows(rows, q_len);
    ++steps;
    return StepOutput{logits, std::move(layout.out_rows)};
}

Stepper::ShapeKey Stepper::shape_key(const std::vector<StepEntry>& entries, const std::vector<int64_t>& q_len) const {
    int T = 0, R = 0;
    int64_t longest = 0;
    for (size_t i = 0; i < entries.size(); ++i) {
        T += static_cast<int>(q_len[i]);
        R += entries[i].n_want;
        longest = std::max(longest, q_len[i]);
    }
    const int S = static_cast<int>(entries.size());
    return {S, T, R, T != S ? static_cast<int>((longest + 63) / 64 * 64) : 1};
}

bool Stepper::worth_capturing(const std::vector<StepEntry>& entries, const std::vector<int64_t>& q_len) {
    // A step with prompt portions is captured when its shape comes up for the third time (capturing costs
    // about as much as an eager step) and the scratch buffers are sized so that they will not move.
    const ShapeKey key = shape_key(entries, q_len);
    if (std::get<1>(key) > workspace.min_rows()) return false;
    if (graphs_.count(key)) return true;
    if (seen_.size() > 4096) seen_.clear();
    return ++seen_[key] >= 3;
}

Rows Stepper::graph_step(const std::vector<StepEntry>& entries, const std::vector<int>& rows, const std::vector<int64_t>& q_len,
                         const DeviceTokens* dt, Layout* layout) {
    // A graph fits every step with the same number of requests, tokens and wanted rows whose longest portion
    // falls into the same bucket of 64 tokens; everything else about the step (tokens, positions, where portions
    // start, block tables, slots) is data the graph reads from its own layout buffer.
    const ShapeKey key = shape_key(entries, q_len);
    const int bucket = std::get<3>(key);
    CapturedStep& g = graphs_[key];
    g.last_used = steps;
    cudaStream_t stream = model.runtime.stream;
    if (g.exec != nullptr && g.generation == workspace.generation()) {
        lay_out(entries, rows, q_len, dt, &g, bucket, layout);
        LIYAB_CUDA(cudaGraphLaunch(g.exec, stream));
        kernels::launches.fetch_add(g.launches, std::memory_order_relaxed);
        ++graph_steps;
        return Rows{g.logits.data, g.logits.dtype, std::get<2>(key), g.logits.cols, g.logits.stride};
    }
    // First step of this shape (or buffers moved since): run it part by part on the graph's own layout buffer,
    // which gives this step's result and creates every scratch buffer; then record the same launches for the
    // steps to come.  Recording runs nothing, so the step's tokens are computed exactly once.
    drop_graph(g);
    lay_out(entries, rows, q_len, dt, &g, bucket, layout);
    const Rows logits = model.forward(layout->ctx);
    ++eager_steps;
    const uint64_t generation = workspace.generation();
    const uint64_t before = kernels::launches.load();
    cudaGraph_t graph = nullptr;
    LIYAB_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    try {
        g.logits = model.forward(layout->ctx);
    } catch (...) {
        cudaStreamEndCapture(stream, &graph);
        if (graph != nullptr) cudaGraphDestroy(graph);
        graphs_.erase(key);
        throw;
    }
    LIYAB_CUDA(cudaStreamEndCapture(stream, &graph));
    g.launches = kernels::launches.load() - before;
    kernels::launches.store(before);             // recorded, not launched
    const bool moved = workspace.generation() != generation;
    cudaError_t err = moved ? cudaSuccess : cudaGraphInstantiate(&g.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (moved || err != cudaSuccess) {
        g.exec = nullptr;
        graphs_.erase(key);
        if (moved) throw internal_error("a scratch buffer was created while a step was being recorded");
        cuda_check(err, "cudaGraphInstantiate");
    }
    g.generation = generation;
    ++graphs_captured;
    if (graphs_.size() > 48) {                   // keep the most recently used shapes
        auto oldest = graphs_.end();
        for (auto it = graphs_.begin(); it != graphs_.end(); ++it)
            if (it->first != key && (oldest == graphs_.end() || it->second.last_used < oldest->second.last_used)) oldest = it;
        if (oldest != graphs_.end()) {
            drop_graph(oldest->second);
            graphs_.erase(oldest);
        }
    }
    return logits;
}

void Stepper::lay_out(const std::vector<StepEntry>& entries, const std::vector<int>& rows, const std::vector<int64_t>& q_len,
                      const DeviceTokens* dt, CapturedStep* fixed, int max_q_len, Layout* out) {
    const int S = static_cast<int>(entries.size());
    const int G = static_cast<int>(cache.groups.size());
    int T = 0, R = 0;
    for (int i = 0; i < S; ++i) { T += static_cast<int>(q_len[static_cast<size_t>(i)]); R += entries[static_cast<size_t>(i)].n_want; }
    // Block tables: the widest of the step's requests, or (for a captured step) widths that never change.
    std::vector<int> widths(static_cast<size_t>(G), 0);
    std::vector<std::vector<int32_t>> tables(static_cast<size_t>(G));
    for (int g = 0; g < G; ++g) {
        if (fixed != nullptr) widths[static_cast<size_t>(g)] = (max_positions + cache.page_size - 1) / cache.page_size;
        tables[static_cast<size_t>(g)] = cache.table_rows(g, rows, &widths[static_cast<size_t>(g)]);
    }
    const bool with_map = dt != nullptr || fixed != nullptr;         // a captured step keeps room for the map
    // Sizes of the pieces, each starting on a 16-byte boundary.
    std::vector<size_t> sizes{static_cast<size_t>(T), static_cast<size_t>(T), static_cast<size_t>(T), static_cast<size_t>(S + 1),
                              static_cast<size_t>(S), static_cast<size_t>(S), static_cast<size_t>(R)};
    for (int g = 0; g < G; ++g) sizes.push_back(static_cast<size_t>(S) * static_cast<size_t>(widths[static_cast<size_t>(g)]));
    for (int g = 0; g < G; ++g) sizes.push_back(static_cast<size_t>(T));
    if (with_map) sizes.push_back(static_cast<size_t>(T));
    std::vector<size_t> offsets;
    size_t total = 0;
    for (const size_t n : sizes) { offsets.push_back(total); total += (n + 3) / 4 * 4; }

    turn_ = 1 - turn_;
    PinnedBuffer& hostbuf = host_[turn_];
    if (hostbuf.bytes() < total * 4) {
        hostbuf = PinnedBuffer(std::max<size_t>(total, 4096) * 4 * 2);
        copied_[turn_] = std::make_unique<Event>();
    } else {
        copied_[turn_]->synchronize();       // rewritten only after the copy that last read it has finished
    }
    int32_t* host = static_cast<int32_t*>(hostbuf.data());
    int32_t* dev = nullptr;
    if (fixed != nullptr) {
        if (fixed->layout.data() == nullptr) {
            fixed->layout = DeviceBuffer(total * 4);
            fixed->layout_ints = total;
        }
        if (fixed->layout_ints != total) throw internal_error("a captured step's layout changed size");
        dev = static_cast<int32_t*>(fixed->layout.data());
    } else {
        if (dev_.bytes() < total * 4) dev_ = DeviceBuffer(std::max<size_t>(total, 4096) * 4 * 2);
        dev = static_cast<int32_t*>(dev_.data());
    }

    StepContext& ctx = out->ctx;
    ctx = StepContext{};
    int32_t* h_tokens = host + offsets[0];
    int32_t* h_pos = host + offsets[1];
    int32_t* h_seq = host + offsets[2];
    int32_t* h_qstart = host + offsets[3];
    int32_t* h_npast = host + offsets[4];
    int32_t* h_slots = host + offsets[5];
    int32_t* h_logit = host + offsets[6];
    out->out_rows.clear();
    out->out_rows.reserve(static_cast<size_t>(R));
    ctx.host_q_start.resize(static_cast<size_t>(S + 1));
    ctx.host_n_past.resize(static_cast<size_t>(S));
    ctx.host_state_slots.assign(rows.begin(), rows.end());
    int at = 0, r = 0, longest = 0, max_kv = 0;
    for (int i = 0; i < S; ++i) {
        const StepEntry& e = entries[static_cast<size_t>(i)];
        const int row = rows[static_cast<size_t>(i)];
        const int past = static_cast<int>(cache.length_of_row[static_cast<size_t>(row)]);
        const bool on_device = dt != nullptr && dt->index[static_cast<size_t>(i)] >= 0;
        h_qstart[i] = at;
        h_npast[i] = past;
        h_slots[i] = row;
        ctx.host_q_start[static_cast<size_t>(i)] = at;
        ctx.host_n_past[static_cast<size_t>(i)] = past;
        for (int t = 0; t < e.n_tokens; ++t) {
            h_tokens[at + t] = on_device ? 0 : e.tokens[t];
            h_pos[at + t] = past + t;
            h_seq[at + t] = i;
            for (int g = 0; g < G; ++g) host[offsets[static_cast<size_t>(7 + G + g)] + static_cast<size_t>(at + t)] = cache.slot_of(g, row, past + t);
        }
        if (with_map) {
            int32_t* h_map = host + offsets[static_cast<size_t>(7 + 2 * G)];
            for (int t = 0; t < e.n_tokens; ++t) h_map[at + t] = -1;
            if (on_device) h_map[at] = dt->index[static_cast<size_t>(i)];
        }
        for (int w = 0; w < e.n_want; ++w) {
            h_logit[r++] = at + e.want[w];
            out->out_rows.emplace_back(e.request, e.want[w]);
        }
        longest = std::max(longest, e.n_tokens);
        max_kv = std::max(max_kv, past + e.n_tokens);
        at += e.n_tokens;
    }
    h_qstart[S] = at;
    ctx.host_q_start[static_cast<size_t>(S)] = at;
    for (int g = 0; g < G; ++g)
        std::memcpy(host + offsets[static_cast<size_t>(7 + g)], tables[static_cast<size_t>(g)].data(), tables[static_cast<size_t>(g)].size() * 4);

    cudaStream_t stream = model.runtime.stream;
    LIYAB_CUDA(cudaMemcpyAsync(dev, host, total * 4, cudaMemcpyHostToDevice, stream));
    copied_[turn_]->record(stream);
    if (dt != nullptr) kernels::gather_tokens(stream, dev + offsets[0], dt->source, dev + offsets[static_cast<size_t>(7 + 2 * G)], T);

    ctx.runtime = model.runtime;
    ctx.workspace = &workspace;
    ctx.cache = &cache;
    ctx.n_tokens = T;
    ctx.n_seq = S;
    ctx.tokens = dev + offsets[0];
    ctx.positions = dev + offsets[1];
    ctx.tok_seq = dev + offsets[2];
    ctx.q_start = dev + offsets[3];
    ctx.n_past = dev + offsets[4];
    ctx.state_slots = dev + offsets[5];
    ctx.logit_rows = dev + offsets[6];
    ctx.n_logit_rows = R;
    for (int g = 0; g < G; ++g)
        ctx.groups.push_back(GroupView{&cache.groups[static_cast<size_t>(g)], dev + offsets[static_cast<size_t>(7 + g)],
                                       widths[static_cast<size_t>(g)], dev + offsets[static_cast<size_t>(7 + G + g)]});
    ctx.max_q_len = max_q_len > 0 ? max_q_len : longest;
    ctx.max_kv_len = max_kv;
    ctx.decode_only = T == S;
    ctx.max_positions = max_positions;
}

}  // namespace liyab
