#include "decoder.h"

#include <set>

#include "kernels.h"

namespace liyab {
namespace {

void add_decls(std::vector<ParamDecl>& out, const std::string& prefix, const std::vector<ParamDecl>& decls) {
    for (const auto& d : decls) out.push_back({prefix + d.name, d.shape, d.kind});
}

std::vector<ParamDecl> slot_parameters(const SlotSpec& s) {
    switch (s.role) {
        case Role::Norm: return norms().get(s.part.kind).parameters(s.part);
        case Role::Mixer: return mixers().get(s.part.kind).parameters(s.part);
        case Role::FeedForward: return feed_forwards().get(s.part.kind).parameters(s.part);
    }
    return {};
}

std::shared_ptr<Part> build_slot(const SlotSpec& s, const Params& p, const Runtime& rt) {
    switch (s.role) {
        case Role::Norm: return norms().get(s.part.kind).build(s.part, p, rt);
        case Role::Mixer: return mixers().get(s.part.kind).build(s.part, p, rt);
        case Role::FeedForward: return feed_forwards().get(s.part.kind).build(s.part, p, rt);
    }
    return nullptr;
}

}  // namespace

std::vector<ParamDecl> parameter_shapes(const ModelSpec& spec) {
    register_builtin_parts();
    std::vector<ParamDecl> out;
    out.push_back({"embedding.weight", {spec.embedding.vocab_size, spec.embedding.size}, ParamKind::Table});
    add_decls(out, "position.", positions().get(spec.position.kind).parameters(spec.position));
    for (size_t i = 0; i < spec.layers.size(); ++i)
        for (const auto& slot : spec.layers[i].slots) add_decls(out, std::format("layers.{}.{}.", i, slot.name), slot_parameters(slot));
    add_decls(out, "final_norm.", norms().get(spec.final_norm.kind).parameters(spec.final_norm));
    if (!spec.head.tied) out.push_back({"head.weight", {spec.head.vocab_size, spec.head.size}, ParamKind::Matrix});
    if (spec.head.bias) out.push_back({"head.bias", {spec.head.vocab_size}, ParamKind::Vector});
    return out;
}

DecoderModel::DecoderModel(ModelSpec spec_, const Params& params, Runtime runtime_) : spec(std::move(spec_)), runtime(runtime_) {
    register_builtin_parts();
    std::string problems;
    for (const auto& d : parameter_shapes(spec)) {
        const Tensor* t = params.find(d.name);
        if (t == nullptr) problems += std::format("{}missing parameter '{}'", problems.empty() ? "" : "; ", d.name);
        else if (t->shape != d.shape)
            problems += std::format("{}parameter '{}' has shape {}, expected {}", problems.empty() ? "" : "; ", d.name, shape_text(t->shape),
                                    shape_text(d.shape));
        else params_.add(d.name, *t);
    }
    if (!problems.empty()) throw invalid_model("{}", problems);
    if (spec.head.soft_cap < 0) throw invalid_model("head.soft_cap {} is negative", spec.head.soft_cap);
    embedding = params_.at("embedding.weight");
    position = positions().get(spec.position.kind).build(spec.position, params_.sub("position."), runtime);
    for (size_t i = 0; i < spec.layers.size(); ++i) {
        Layer layer;
        const Params lp = params_.sub(std::format("layers.{}.", i));
        for (const auto& slot : spec.layers[i].slots) layer.parts.by_name[slot.name] = build_slot(slot, lp.sub(slot.name + "."), runtime);
        layer.block = arrangements().get(spec.layers[i].arrangement).build(spec.layers[i], layer.parts, runtime);
        layers.push_back(std::move(layer));
    }
    final_norm = norms().get(spec.final_norm.kind).build(spec.final_norm, params_.sub("final_norm."), runtime);
    head_weight = spec.head.tied ? embedding : params_.at("head.weight");
    if (spec.head.bias) head_bias = static_cast<const float*>(params_.at("head.bias").data);
    const int n = static_cast<int>(spec.run_order.size());
    for (int i = 0; i < n; ++i) {
        const RunEntry& e = spec.run_order[static_cast<size_t>(i)];
        if (e.layer < 0 || e.layer >= static_cast<int>(layers.size()) || e.cache < 0 || e.cache >= n)
            throw invalid_model("run order entry {} names layer {} / cache {} out of range", i, e.layer, e.cache);
        if (e.cache != i && spec.run_order[static_cast<size_t>(e.cache)].cache != e.cache)
            throw invalid_model("run order entry {} reads the cache of entry {}, which keeps none", i, e.cache);
        if (e.cache > i) throw invalid_model("run order entry {} reads the cache of a later entry {}", i, e.cache);
    }
    kv_needs();      // checks that entries sharing a cache agree on its shape
}

Mixer* DecoderModel::mixer_of(const RunEntry& e) const {
    const auto ms = layers[static_cast<size_t>(e.layer)].block->mixers();
    return ms.empty() ? nullptr : ms.front();
}

std::map<int, KvNeed> DecoderModel::kv_needs() const {
    std::map<int, KvNeed> out;
    const int n = static_cast<int>(spec.run_order.size());
    for (int i = 0; i < n; ++i) {
        const RunEntry& e = spec.run_order[static_cast<size_t>(i)];
        if (e.cache != i) continue;
        Mixer* m = mixer_of(e);
        if (m == nullptr) continue;
        if (const auto need = m->kv_need()) out[i] = *need;
    }
    for (int i = 0; i < n; ++i) {
        const RunEntry& e = spec.run_order[static_cast<size_t>(i)];
        if (e.cache == i) continue;
        Mixer* m = mixer_of(e);
        const auto mine = m != nullptr ? m->kv_need() : std::nullopt;
        const auto it = out.find(e.cache);
        if (mine && (it == out.end() || !(it->second == *mine)))
            throw invalid_model("run order entry {} reads the cache of entry {}, whose keys and values have another shape or window", i, e.cache);
    }
    return out;
}

std::map<int, StateNeed> DecoderModel::state_needs() const {
    std::map<int, StateNeed> out;
    for (size_t i = 0; i < spec.run_order.size(); ++i) {
        Mixer* m = mixer_of(spec.run_order[i]);
        if (m == nullptr) continue;
        if (const auto need = m->state_need()) out[static_cast<int>(i)] = *need;
    }
    return out;
}

int64_t DecoderModel::max_positions() const { return std::min(spec.max_positions, position->max_positions()); }

size_t DecoderModel::weight_bytes() const {
    std::set<const void*> seen;
    size_t total = 0;
    for (const auto& [name, t] : params_.all())
        if (seen.insert(t.data).second) total += t.bytes();
    return total;
}

bool DecoderModel::capturable() const {
    if (!position->capturable() || !final_norm->capturable()) return false;
    for (const auto& l : layers)
        if (!l.block->capturable()) return false;
    return true;
}

Rows DecoderModel::forward(StepContext& ctx) {
    const int T = ctx.n_tokens;
    const int64_t width = spec.hidden();
    Workspace& ws = *ctx.workspace;
    const Rows x = ws.get("residual", T, width, DType::F32);
    ctx.phase(Phase::Embed);
    position->embed(ctx, embedding, static_cast<float>(spec.embedding.scale), x);
    ctx.tap("embed", x);
    for (size_t i = 0; i < spec.run_order.size(); ++i) {
        const RunEntry& e = spec.run_order[i];
        layers[static_cast<size_t>(e.layer)].block->forward(ctx, x, CacheUnit{e.cache, e.cache == static_cast<int>(i)});
    }
    const int R = ctx.n_logit_rows;
    if (R == 0) return Rows{nullptr, DType::F32, 0, spec.vocab_size(), spec.vocab_size()};
    // The head's buffers are sized by the rows whose logits are wanted, not by the step's tokens.
    ctx.phase(Phase::Head);
    const Rows y = ws.get("head.normed", R, width, runtime.dtype, false);
    final_norm->forward(ctx, x, y, R, ctx.logit_rows);
    ctx.tap("final_norm", y);
    const Rows logits = ws.get("logits", R, spec.vocab_size(), DType::F32, false);
    kernels::linear(runtime, &ws, y, head_weight, head_bias, logits, R, kernels::kNone, nullptr);
    if (spec.head.logit_scale != 1.0 || spec.head.soft_cap > 0.0)
        kernels::scale_softcap(ctx.stream(), logits.f32(), static_cast<int64_t>(R) * spec.vocab_size(), static_cast<float>(spec.head.logit_scale),
                               static_cast<float>(spec.head.soft_cap));
    return logits;
}

}  // namespace liyab
