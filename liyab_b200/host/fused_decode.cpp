#include "fused_decode.h"

#include <cstring>

#include "../csrc/api.h"
#include "builtin_parts.h"

namespace liyab {
namespace {

// One layer as the kernel reads it (csrc/decode_stack.cu, StackLayer): 13 pointers, 3 floats, 6 ints, padding.
struct LayerRecord {
    const void* ptr[13];
    float eps1, eps2, scale;
    int32_t n_head, n_kv_head, head_dim, inner, activation, window;
    int32_t pad;
};
static_assert(sizeof(LayerRecord) == 13 * 8 + 3 * 4 + 6 * 4 + 4, "the layer record is packed without holes");

}  // namespace

std::unique_ptr<FusedDecodeStack> FusedDecodeStack::try_build(const DecoderModel& model, const CacheManager& cache) {
    using namespace builtin;
    const ModelSpec& spec = model.spec;
    if (model.runtime.dtype != DType::BF16 || cache.groups.size() != 1 || !cache.states.needs.empty()) return nullptr;
    const auto* learned = dynamic_cast<const LearnedAbsolutePosition*>(model.position.get());
    if (learned == nullptr && dynamic_cast<const NoPosition*>(model.position.get()) == nullptr) return nullptr;
    const auto* lnf = dynamic_cast<const LayerNorm*>(model.final_norm.get());
    if (lnf == nullptr || spec.head.logit_scale != 1.0 || spec.head.soft_cap != 0.0) return nullptr;
    const int ps = cache.page_size;
    if ((ps & (ps - 1)) != 0 || ps < 16 || spec.hidden() % 8 != 0) return nullptr;      // the attention phase takes its 16-key tiles from one page
    if (lb_decode_stack_layer_bytes() != static_cast<int>(sizeof(LayerRecord))) return nullptr;

    std::unique_ptr<FusedDecodeStack> s(new FusedDecodeStack());
    s->model_ = &model;
    s->cache_ = &cache;
    s->max_k_ = static_cast<int>(spec.hidden());
    std::vector<LayerRecord> records;
    for (size_t i = 0; i < spec.run_order.size(); ++i) {
        const RunEntry& e = spec.run_order[i];
        if (e.cache != static_cast<int>(i)) return nullptr;
        const auto* block = dynamic_cast<const PreNormBlock*>(model.layers[static_cast<size_t>(e.layer)].block.get());
        if (block == nullptr) return nullptr;
        const auto* n1 = dynamic_cast<const LayerNorm*>(&block->mixer_norm);
        const auto* n2 = dynamic_cast<const LayerNorm*>(&block->ff_norm);
        const auto* at = dynamic_cast<const CausalSelfAttention*>(&block->mixer);
        const auto* ff = dynamic_cast<const DenseFeedForward*>(&block->feed_forward);
        if (n1 == nullptr || n2 == nullptr || at == nullptr || ff == nullptr) return nullptr;
        const auto& a = at->shape;
        if ((a.head_dim != 64 && a.head_dim != 128) || (s->head_dim_ != 0 && s->head_dim_ != a.head_dim) || ff->inner % 8 != 0) return nullptr;
        if (a.n_head / a.n_kv_head > 16) return nullptr;       // the query heads of a key/value head are the 16 rows of a tile
        if (at->hidden != spec.hidden()) return nullptr;
        s->head_dim_ = a.head_dim;
        const int qd = a.n_head * a.head_dim;
        s->max_qd_ = std::max(s->max_qd_, qd);
        s->max_inner_ = std::max(s->max_inner_, static_cast<int>(ff->inner));
        s->max_heads_ = std::max(s->max_heads_, a.n_head);
        s->max_kv_heads_ = std::max(s->max_kv_heads_, a.n_kv_head);
        s->max_k_ = std::max({s->max_k_, qd, static_cast<int>(ff->inner)});
        LayerRecord r{};
        const void* ptrs[13] = {n1->weight_, n1->bias_, n2->weight_, n2->bias_, at->qkv.weight.data, at->qkv.bias, at->out.weight.data,
                                at->out.bias, ff->up.weight.data, ff->up.bias, ff->down.weight.data, ff->down.bias,
                                cache.groups[0].unit_storage(static_cast<int>(i))};
        std::memcpy(r.ptr, ptrs, sizeof ptrs);
        r.eps1 = n1->eps_;
        r.eps2 = n2->eps_;
        r.scale = a.scale;
        r.n_head = a.n_head;
        r.n_kv_head = a.n_kv_head;
        r.head_dim = a.head_dim;
        r.inner = static_cast<int32_t>(ff->inner);
        r.activation = ff->activation;
        r.window = a.window;
        records.push_back(r);
    }
    if (s->head_dim_ == 0) return nullptr;
    s->n_layers_ = static_cast<int>(records.size());
    const size_t act = static_cast<size_t>(kMaxTokens) * (static_cast<size_t>((s->max_k_ + 63) / 64 * 64) + 32) * 2 + 8 * 8 * 128 * 4;
    const size_t smem = std::max<size_t>(act, 200 * 1024) + 64 + 16 + 16 + 256 + records.size() * sizeof(LayerRecord);
    if (smem > 227 * 1024) return nullptr;

    s->pos_table_ = learned != nullptr ? learned->table_.data : nullptr;
    s->lnf_w_ = lnf->weight_;
    s->lnf_b_ = lnf->bias_;
    s->lnf_eps_ = lnf->eps_;
    const size_t T = kMaxTokens;
    s->layers_ = DeviceBuffer(records.size() * sizeof(LayerRecord));
    LIYAB_CUDA(cudaMemcpy(s->layers_.data(), records.data(), records.size() * sizeof(LayerRecord), cudaMemcpyHostToDevice));
    s->x_ = DeviceBuffer(T * static_cast<size_t>(spec.hidden()) * 4);
    s->q_ = DeviceBuffer(T * static_cast<size_t>(s->max_qd_) * 2);
    s->att_ = DeviceBuffer(T * static_cast<size_t>(s->max_qd_) * 2);
    s->inner_ = DeviceBuffer(T * static_cast<size_t>(s->max_inner_) * 2);
    s->logits_ = DeviceBuffer(T * static_cast<size_t>(spec.vocab_size()) * 4);
    s->partial_ = DeviceBuffer(T * static_cast<size_t>(s->max_heads_) * 64 * static_cast<size_t>(s->head_dim_ + 2) * 4);
    s->counters_ = DeviceBuffer(T * static_cast<size_t>(s->max_heads_) * 4, true);
    s->barrier_ = DeviceBuffer(8, true);         // two counters, used by alternate launches
    return s;
}

bool FusedDecodeStack::accepts(int n_tokens) const {
    return n_tokens >= 1 && n_tokens <= kMaxTokens && n_tokens * max_kv_heads_ <= model_->runtime.sm_count;
}

void FusedDecodeStack::splits(int n_tokens, int* n_splits, int* unit_warps) const {
    // (key ranges per (token, key/value head), warps per work item): a function of the batch's shape only.
    // A range merged across blocks costs a round of atomics and reloads, so from 64 pairs on a pair is one item,
    // served by a whole block (eight warps) while there are blocks enough for that, else by half a block; fewer
    // pairs are split until every half block has an item.
    const int pairs = n_tokens * max_kv_heads_, n_sm = model_->runtime.sm_count;
    if (pairs >= 64) {
        *n_splits = 1;
        *unit_warps = pairs <= n_sm ? 8 : 4;
        return;
    }
    *n_splits = std::max(1, std::min(8, (2 * n_sm) / pairs));      // more ranges only lengthen the last group's merge
    *unit_warps = 4;
}

void FusedDecodeStack::record_stamps(bool on) {
    stamps_ = on ? DeviceBuffer(kStamps * sizeof(uint64_t), true) : DeviceBuffer();
}

std::vector<uint64_t> FusedDecodeStack::stamps() const {
    std::vector<uint64_t> out(stamps_.data() != nullptr ? kStamps : 0);
    if (!out.empty()) LIYAB_CUDA(cudaMemcpy(out.data(), stamps_.data(), out.size() * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    return out;
}

Rows FusedDecodeStack::run(StepContext& ctx) {
    const ModelSpec& spec = model_->spec;
    const int B = ctx.n_tokens;
    const GroupView& view = ctx.groups.at(0);
    int n_splits = 1, unit_warps = 4;
    splits(B, &n_splits, &unit_warps);
    unsigned* barrier = static_cast<unsigned*>(barrier_.data()) + (launches_ & 1);
    kernels::check(lb_decode_stack(layers_.data(), n_layers_, B, static_cast<int>(spec.hidden()), static_cast<int>(spec.vocab_size()),
                                   model_->embedding.data, pos_table_, static_cast<float>(spec.embedding.scale), lnf_w_, lnf_b_, lnf_eps_,
                                   model_->head_weight.data, model_->head_bias, ctx.tokens, ctx.positions, view.block_table,
                                   view.table_width, view.slot_mapping, cache_->page_size, static_cast<float*>(x_.data()), q_.data(),
                                   att_.data(), inner_.data(), static_cast<float*>(partial_.data()), static_cast<int*>(counters_.data()),
                                   static_cast<float*>(logits_.data()), barrier, max_k_, head_dim_, n_splits, unit_warps,
                                   static_cast<unsigned long long*>(stamps_.data()), ctx.stream()),
                   "decode_stack");
    ++launches_;
    return Rows{logits_.data(), DType::F32, B, spec.vocab_size(), spec.vocab_size()};
}

}  // namespace liyab
