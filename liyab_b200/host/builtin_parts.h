// The library's own parts: LayerNorm, learned absolute positions (and none),
// causal self-attention over the paged cache, the dense feed-forward and the
// pre-norm arrangement.  Every size and constant is an option of the part's spec;
// no part knows which model it is in.  The classes are declared here (not hidden in
// their source file) so that the one-kernel decode step can recognise a model made
// of nothing else by exact type and read the parts' own parameters.
#pragma once

#include <cmath>

#include "kernels.h"
#include "parts.h"

namespace liyab::builtin {


inline int64_t need_int(const PartSpec& s, const char* key, int64_t lo = 1) {
    const Json* v = s.options.find(key);
    if (v == nullptr || !v->is_int() || v->as_int() < lo)
        throw invalid_model("{}: option '{}' must be an integer >= {}", s.kind, key, lo);
    return v->as_int();
}

inline const float* f32_or_null(const Tensor* t) { return t == nullptr ? nullptr : static_cast<const float*>(t->data); }

// A matrix [out, in] in the compute type with an optional float32 bias: y = act(x W^T + b) (+ residual).
// The product runs on the tensor-core kernels when the operands are bfloat16 and the sizes suit them, else on the
// 32-bit units; all fuse bias, activation and the residual sum into their epilogue, in the reference's order
// (bias, activation, residual: src/core/transformer.cpp:111-118, 4903-4912, 5526-5532).
struct Linear {
    Tensor weight;
    const float* bias = nullptr;

    Linear() = default;
    Linear(const Params& p, const std::string& prefix, const char* what) {
        weight = p.at(prefix + "weight");
        if (weight.shape.size() != 2) throw invalid_model("{}: weight must be a matrix, got shape {}", what, shape_text(weight.shape));
        if (const Tensor* b = p.find(prefix + "bias")) {
            if (b->shape != std::vector<int64_t>{weight.dim(0)} || b->dtype != DType::F32)
                throw invalid_model("{}: bias has shape {}, expected [{}] of float32", what, shape_text(b->shape), weight.dim(0));
            bias = static_cast<const float*>(b->data);
        }
    }
    static void declare(std::vector<ParamDecl>& out, const std::string& prefix, int64_t out_features, int64_t in_features, bool bias) {
        out.push_back({prefix + "weight", {out_features, in_features}, ParamKind::Matrix});
        if (bias) out.push_back({prefix + "bias", {out_features}, ParamKind::Vector});
    }
    void forward(StepContext& ctx, const Rows& a, const Rows& out, int m, int act = kernels::kNone, const Rows* residual = nullptr) const {
        kernels::linear(ctx.runtime, ctx.workspace, a, weight, bias, out, m, act, residual);
    }
};

// ---- LayerNorm with 32-bit statistics (reference: src/core/transformer.cpp:77-106) ----------------

class LayerNorm final : public Norm {
public:
    LayerNorm(const PartSpec& s, const Params& p) : eps_(static_cast<float>(s.options.get_number("eps", 1e-5))) {
        weight_ = f32_or_null(&p.at("weight"));
        bias_ = f32_or_null(p.find("bias"));
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t size = need_int(s, "size");
        std::vector<ParamDecl> out{{"weight", {size}, ParamKind::Vector}};
        if (s.options.get_bool("bias", true)) out.push_back({"bias", {size}, ParamKind::Vector});
        return out;
    }
    bool capturable() const override { return true; }
    void forward(StepContext& ctx, const Rows& x, const Rows& out, int n_rows, const int32_t* rows) override {
        kernels::layernorm(ctx.stream(), x, rows, weight_, bias_, out, n_rows, eps_);
    }
    std::optional<NormRecipe> recipe() const override { return NormRecipe{weight_, bias_, eps_}; }
    const float* weight_ = nullptr;
    const float* bias_ = nullptr;
    float eps_;
};

// ---- position encodings that act where the tokens are embedded -------------------------------------
// `learned_absolute` adds a row of a learned table for each token's position (reference: add_positions,
// src/core/transformer.cpp:2791-2808); the gather of the embedding row and this sum are one kernel.  `none`
// embeds only.  An encoding that acts inside the mixer instead (a rotation of queries and keys, a bias on
// scores) registers with an `embed` that embeds only, and its mixer reads the step context's positions.

class LearnedAbsolutePosition final : public PositionEncoding {
public:
    LearnedAbsolutePosition(const PartSpec& s, const Params& p) : table_(p.at("weight")), max_(need_int(s, "max_positions")) {}
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        return {{"weight", {need_int(s, "max_positions"), need_int(s, "size")}, ParamKind::Table}};
    }
    bool capturable() const override { return true; }
    int64_t max_positions() const override { return max_; }
    void embed(StepContext& ctx, const Tensor& table, float scale, const Rows& x) override {
        kernels::embed_positions(ctx.stream(), ctx.tokens, ctx.positions, table, &table_, x, ctx.n_tokens, scale);
    }
    Tensor table_;
    int64_t max_;
};

class NoPosition final : public PositionEncoding {
public:
    explicit NoPosition(const PartSpec& s) : max_(s.options.get_int("max_positions", int64_t{1} << 30)) {}
    bool capturable() const override { return true; }
    int64_t max_positions() const override { return max_; }
    void embed(StepContext& ctx, const Tensor& table, float scale, const Rows& x) override {
        kernels::embed_positions(ctx.stream(), ctx.tokens, ctx.positions, table, nullptr, x, ctx.n_tokens, scale);
    }
    int64_t max_;
};

// ---- causal self-attention over the paged cache, one fused projection of queries, keys and values -----
// Sizes and constants are the spec's: heads, key/value heads, head size, the factor on the scores and the
// window.  The step's keys and values are written to the unit's pages first; attention then reads every key,
// old and new, from the pages, so a token's result does not depend on how its sequence was cut into steps.
// Reference: attention_mixer (src/core/transformer.cpp:3035-3142): fused projection and split [q | k | v]
// (:2657-2673), biases (:3089-3101), store_kv (:2875-2890), attention (:2130-2453), output projection (:3139-3140).

class CausalSelfAttention final : public Mixer {
public:
    CausalSelfAttention(const PartSpec& s, const Params& p) {
        hidden = need_int(s, "hidden");
        shape.n_head = static_cast<int>(need_int(s, "n_head"));
        shape.n_kv_head = static_cast<int>(s.options.get_int("n_kv_head", shape.n_head));
        shape.head_dim = static_cast<int>(need_int(s, "head_dim"));
        shape.scale = static_cast<float>(s.options.get_number("scale", 1.0 / std::sqrt(static_cast<double>(shape.head_dim))));
        shape.window = static_cast<int>(s.options.get_int("window", 0));
        if (shape.n_kv_head <= 0 || shape.n_head % shape.n_kv_head != 0)
            throw invalid_model("attention: n_head {} is not a multiple of n_kv_head {}", shape.n_head, shape.n_kv_head);
        if (shape.window < 0) throw invalid_model("attention: window {} is negative", shape.window);
        q_dim = shape.n_head * shape.head_dim;
        kv_dim = shape.n_kv_head * shape.head_dim;
        qkv = Linear(p, "qkv.", "attention.qkv");
        out = Linear(p, "out.", "attention.out");
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t hidden = need_int(s, "hidden"), n_head = need_int(s, "n_head"), hd = need_int(s, "head_dim");
        const int64_t n_kv = s.options.get_int("n_kv_head", n_head);
        const bool bias = s.options.get_bool("bias", true);
        std::vector<ParamDecl> out;
        Linear::declare(out, "qkv.", (n_head + 2 * n_kv) * hd, hidden, bias);
        Linear::declare(out, "out.", hidden, n_head * hd, bias);
        return out;
    }
    bool capturable() const override { return true; }
    std::optional<KvNeed> kv_need() const override { return KvNeed{shape.n_kv_head, shape.head_dim, shape.window}; }

    // A step of up to 16 tokens in bfloat16 with rows of up to 1024 values: the projection normalises the rows inside
    // its kernel (and fills the cache from its epilogue), so the LayerNorm before the mixer is not launched.
    bool forward_from(StepContext& ctx, const Rows& x_in, const NormRecipe& norm, const Rows& x, CacheUnit unit) override {
        const int T = ctx.n_tokens;
        if (!unit.write || !kernels::gemm_rows_normed_supports(ctx.runtime, x_in, qkv.weight, T)) return false;
        const Rows qkv_out = ctx.workspace->get("attn.qkv", T, q_dim + 2 * kv_dim, ctx.runtime.dtype);
        const GroupView* view = nullptr;
        void* cache = ctx.kv(unit.read, &view);
        kernels::AttentionShape a = shape;
        a.page_size = view->group->page_size;
        const kernels::KvDestination dest{cache, view->slot_mapping, q_dim, a.n_kv_head, a.head_dim, a.page_size};
        kernels::gemm_rows_normed(ctx.stream(), x_in, norm.gain, norm.offset, norm.eps, qkv.weight, qkv.bias, qkv_out, T, kernels::kNone,
                                  nullptr, &dest);
        attend_and_project(ctx, qkv_out, cache, *view, a, x);
        return true;
    }

    void forward(StepContext& ctx, const Rows& h, const Rows& x, CacheUnit unit) override {
        const int T = ctx.n_tokens;
        const DType dt = ctx.runtime.dtype;
        Workspace& ws = *ctx.workspace;
        const Rows qkv_out = ws.get("attn.qkv", T, q_dim + 2 * kv_dim, dt);
        const GroupView* view = nullptr;
        void* cache = ctx.kv(unit.read, &view);
        kernels::AttentionShape a = shape;
        a.page_size = view->group->page_size;
        const kernels::KvDestination dest{cache, view->slot_mapping, q_dim, a.n_kv_head, a.head_dim, a.page_size};
        const Tensor& w = qkv.weight;
        if (unit.write && dt == DType::BF16 && kernels::gemm_rows_takes(T, static_cast<int>(w.dim(0)), static_cast<int>(w.dim(1)), ctx.runtime.sm_count) && kernels::gemm_rows_supports(h, w, T)) {
            // A step of a few dozen tokens: the projection's epilogue also puts the new keys and values into their pages.
            kernels::gemm_rows(ctx.stream(), h, w, qkv.bias, qkv_out, T, kernels::kNone, nullptr, &dest);
        } else if (unit.write && dt == DType::BF16 && T > 64 && kernels::gemm_persistent_tile(h, w, qkv_out, T, nullptr) > 0 &&
                   kernels::gemm_persistent_kv_supports(w, qkv_out, dest)) {
            // Many tokens: the same from the tensor-core product's epilogue (only the queries go to `qkv_out`).
            kernels::gemm_persistent(ctx.stream(), h, w, qkv.bias, qkv_out, T, kernels::kNone, nullptr, &dest);
        } else if (unit.write && dt == DType::BF16 && kernels::linear_with_cache(ctx.runtime, &ws, h, w, qkv.bias, qkv_out, T, dest)) {
            // Few tokens, K split over blocks: the split product's second half filled the cache as well.
        } else {
            qkv.forward(ctx, h, qkv_out, T);
            if (unit.write)
                kernels::kv_append(ctx.stream(), qkv_out.columns(q_dim, kv_dim), qkv_out.columns(q_dim + kv_dim, kv_dim),
                                   view->slot_mapping, cache, dt, T, a.n_kv_head, a.head_dim, a.page_size);
        }
        attend_and_project(ctx, qkv_out, cache, *view, a, x);
    }

private:
    void attend_and_project(StepContext& ctx, const Rows& qkv_out, void* cache, const GroupView& view, const kernels::AttentionShape& a,
                            const Rows& x) {
        const int T = ctx.n_tokens;
        const Rows q = qkv_out.columns(0, q_dim);
        const Rows att = ctx.workspace->get("attn.out", T, q_dim, ctx.runtime.dtype);
        attend(ctx, q, cache, view, att, a);
        ctx.tap("attention", att);
        out.forward(ctx, att, x, T, kernels::kNone, &x);
    }

    // Chooses the attention kernel.  bfloat16: a split-key decode kernel for steps of single tokens (on the
    // tensor cores where that one takes the shape, else scalar), the tensor-core prefill kernel for steps with
    // prompt portions, where they take the shape.  Else the generic kernel; all of the 32-bit engine runs on it,
    // so that there a position's result has the same bits however the work was cut.
    void attend(StepContext& ctx, const Rows& q, void* cache, const GroupView& view, const Rows& att, const kernels::AttentionShape& a) {
        const int T = ctx.n_tokens;
        const int n_pages = view.group->pool.num_pages();
        if (ctx.runtime.dtype == DType::BF16 && ctx.decode_only) {
            const bool tensor = kernels::decode_mma_supports(a), scalar = kernels::decode_scalar_supports(a);
            if (tensor || scalar) {
                const int splits = kernels::decode_splits(T, a.n_kv_head, ctx.max_positions, tensor);
                float* partial = nullptr;
                int* counters = nullptr;
                if (splits > 1) {
                    partial = static_cast<float*>(ctx.workspace->flat("attn.decode.partial",
                                                                      static_cast<int64_t>(T) * a.n_head * splits * (a.head_dim + 2), DType::F32));
                    counters = static_cast<int*>(ctx.workspace->flat("attn.decode.counters", static_cast<int64_t>(T) * a.n_kv_head, DType::I32, true));
                }
                kernels::decode_attention(ctx.stream(), tensor, q, cache, n_pages, ctx.positions, view.block_table, view.table_width,
                                          att, partial, counters, T, a, splits);
                return;
            }
        }
        if (ctx.runtime.dtype == DType::BF16 && kernels::prefill_supports(a)) {
            kernels::prefill_attention(ctx.runtime, q, T, cache, n_pages, ctx.q_start, ctx.n_past, view.block_table, view.table_width,
                                       att, ctx.n_seq, ctx.max_q_len, a);
            return;
        }
        kernels::attention_generic(ctx.stream(), ctx.runtime.dtype, q, cache, ctx.tok_seq, ctx.positions, view.block_table,
                                   view.table_width, att, T, a);
    }

public:
    kernels::AttentionShape shape;
    int64_t hidden = 0;
    int q_dim = 0, kv_dim = 0;
    Linear qkv, out;
};

// ---- the dense, ungated feed-forward: down(act(up(x))) ----------------------------------------------
// Reference: dense_ffn, ungated branch (src/core/transformer.cpp:4903-4913) with the activations of :125-142.
// Bias and activation ride in the first product's epilogue, bias and the residual sum in the second's.

class DenseFeedForward final : public FeedForward {
public:
    DenseFeedForward(const PartSpec& s, const Params& p) {
        inner = need_int(s, "inner");
        activation = kernels::activation_from_name(s.options.get_string("activation", "gelu_tanh"));
        up = Linear(p, "up.", "feed_forward.up");
        down = Linear(p, "down.", "feed_forward.down");
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t hidden = need_int(s, "hidden"), inner = need_int(s, "inner");
        const bool bias = s.options.get_bool("bias", true);
        std::vector<ParamDecl> out;
        Linear::declare(out, "up.", inner, hidden, bias);
        Linear::declare(out, "down.", hidden, inner, bias);
        return out;
    }
    bool capturable() const override { return true; }
    void forward(StepContext& ctx, const Rows& h, const Rows& x) override {
        const int T = ctx.n_tokens;
        const Rows mid = ctx.workspace->get("ff.inner", T, inner, ctx.runtime.dtype);
        up.forward(ctx, h, mid, T, activation);
        down.forward(ctx, mid, x, T, kernels::kNone, &x);
    }
    // As the attention's: the up projection of a few tokens normalises the rows inside its kernel.
    bool forward_from(StepContext& ctx, const Rows& x_in, const NormRecipe& norm, const Rows& x) override {
        const int T = ctx.n_tokens;
        if (!kernels::gemm_rows_normed_supports(ctx.runtime, x_in, up.weight, T)) return false;
        const Rows mid = ctx.workspace->get("ff.inner", T, inner, ctx.runtime.dtype);
        kernels::gemm_rows_normed(ctx.stream(), x_in, norm.gain, norm.offset, norm.eps, up.weight, up.bias, mid, T, activation, nullptr, nullptr);
        down.forward(ctx, mid, x, T, kernels::kNone, &x);
        return true;
    }
    int64_t inner = 0;
    int activation = 0;
    Linear up, down;
};

// ---- how a layer's parts are arranged around the residual stream ---------------------------------------
// `pre_norm`: x += mixer(norm(x)); x += feed_forward(norm(x)), the reference's run_block for this architecture
// (src/core/transformer.cpp:5574-5577, 5633-5637, 5647, 5663-5666, 5684-5685, 5692).  The residual stream stays
// float32 in every mode; the normalised input of a part is in the compute type.  Slots: mixer_norm (norm), mixer,
// ff_norm (norm), feed_forward.

class PreNormBlock final : public Arrangement {
public:
    PreNormBlock(const LayerSpec& spec, const LayerParts& parts)
        : mixer_norm(parts.get<Norm>("mixer_norm")), mixer(parts.get<Mixer>("mixer")), ff_norm(parts.get<Norm>("ff_norm")),
          feed_forward(parts.get<FeedForward>("feed_forward")), keep_(parts) {
        if (spec.slots.size() != 4) throw invalid_model("arrangement 'pre_norm' takes the slots mixer_norm, mixer, ff_norm and feed_forward only");
    }
    bool capturable() const override {
        return mixer_norm.capturable() && mixer.capturable() && ff_norm.capturable() && feed_forward.capturable();
    }
    std::vector<Mixer*> mixers() const override { return {&mixer}; }
    void forward(StepContext& ctx, const Rows& x, CacheUnit unit) override {
        const int T = ctx.n_tokens;
        const Rows h = ctx.workspace->get("block.normed", T, x.cols, ctx.runtime.dtype);
        // A norm that has a recipe offers it, with the rows as they are, to the part after it; where that part
        // declines (or a test wants to see the norm's output), the norm runs by itself as usual.
        const std::optional<NormRecipe> first = ctx.tap_fn == nullptr ? mixer_norm.recipe() : std::nullopt;
        ctx.phase(Phase::Mixer);
        if (!(first && mixer.forward_from(ctx, x, *first, x, unit))) {
            ctx.phase(Phase::Norm);
            mixer_norm.forward(ctx, x, h, T, nullptr);
            ctx.tap("mixer_norm", h);
            ctx.phase(Phase::Mixer);
            mixer.forward(ctx, h, x, unit);
        }
        ctx.tap("mixer", x);
        const std::optional<NormRecipe> second = ctx.tap_fn == nullptr ? ff_norm.recipe() : std::nullopt;
        ctx.phase(Phase::FeedForward);
        if (!(second && feed_forward.forward_from(ctx, x, *second, x))) {
            ctx.phase(Phase::Norm);
            ff_norm.forward(ctx, x, h, T, nullptr);
            ctx.tap("ff_norm", h);
            ctx.phase(Phase::FeedForward);
            feed_forward.forward(ctx, h, x);
        }
        ctx.tap("feed_forward", x);
    }
    Norm& mixer_norm;
    Mixer& mixer;
    Norm& ff_norm;
    FeedForward& feed_forward;

private:
    LayerParts keep_;
};


}  // namespace liyab::builtin
