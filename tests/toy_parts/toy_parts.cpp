// Toy parts and a toy architecture, defined in the tests and registered with the framework from outside it (a
// plug-in built against the host's headers): a mixer with state of its own, a feed-forward with routing, a position
// encoding without a table, a norm without a mean, two arrangements of a block (side by side; with a third norm) and
// an architecture with its own config.json keys.  None of the framework's files knows about any of them.
#include <cuda_runtime_api.h>

#include <cmath>

#include "arch.h"
#include "kernels.h"
#include "parts.h"

extern "C" {
void toy_running_mean(const void* h, int bf16, int64_t h_stride, void* means, int64_t m_stride, float* state, const int32_t* q_start,
                      const int32_t* slots, int n_seq, int hidden, int write, int only_seq, cudaStream_t s);
void toy_rms(const float* x, const int32_t* rows, const float* weight, void* out, int bf16, int n_rows, int width, float eps, cudaStream_t s);
void toy_sinusoid(float* x, const int32_t* positions, int n_tokens, int width, float base, cudaStream_t s);
void toy_routed_ff(const void* h, int bf16, int64_t h_stride, float* x, int64_t x_stride, const void* router, const void* up, const void* down,
                   int n_tokens, int experts, int inner, int hidden, int top, cudaStream_t s);
}

using namespace liyab;

namespace {

// out_t = W . mean(h_0 .. h_t): the state is the running sum and the count.  With the option "host_loop" the
// mixer walks the requests on the host (it reads the host copy of the layout), which a captured graph would
// freeze: it then says that it cannot be captured.
class RunningMeanMixer final : public Mixer {
public:
    RunningMeanMixer(const PartSpec& s, const Params& p) : hidden_(s.options.at("hidden").as_int()), host_loop_(s.options.get_bool("host_loop", false)), w_(p.at("w")) {}
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t h = s.options.at("hidden").as_int();
        return {{"w", {h, h}, ParamKind::Matrix}};
    }
    bool capturable() const override { return !host_loop_; }
    std::optional<StateNeed> state_need() const override { return StateNeed{{hidden_ + 1}, DType::F32}; }
    void forward(StepContext& ctx, const Rows& h, const Rows& x, CacheUnit unit) override {
        const int T = ctx.n_tokens, bf16 = h.dtype == DType::BF16;
        const Rows means = ctx.workspace->get("toy.means", T, hidden_, h.dtype);
        float* state = static_cast<float*>(ctx.state(unit.read));
        if (host_loop_) {
            for (int i = 0; i < ctx.n_seq; ++i)
                if (ctx.host_q_start[static_cast<size_t>(i) + 1] > ctx.host_q_start[static_cast<size_t>(i)])
                    toy_running_mean(h.data, bf16, h.stride, means.data, means.stride, state, ctx.q_start, ctx.state_slots, ctx.n_seq,
                                     static_cast<int>(hidden_), unit.write, i, ctx.stream());
        } else {
            toy_running_mean(h.data, bf16, h.stride, means.data, means.stride, state, ctx.q_start, ctx.state_slots, ctx.n_seq,
                             static_cast<int>(hidden_), unit.write, -1, ctx.stream());
        }
        kernels::linear(ctx.runtime, ctx.workspace, means, w_, nullptr, x, T, kernels::kNone, &x);
    }

private:
    int64_t hidden_;
    bool host_loop_;
    Tensor w_;
};

class RoutedFeedForward final : public FeedForward {
public:
    RoutedFeedForward(const PartSpec& s, const Params& p)
        : experts_(static_cast<int>(s.options.at("experts").as_int())), inner_(static_cast<int>(s.options.at("inner").as_int())),
          hidden_(static_cast<int>(s.options.at("hidden").as_int())), top_(static_cast<int>(s.options.at("top").as_int())),
          router_(p.at("router")), up_(p.at("up")), down_(p.at("down")) {
        if (top_ < 1 || top_ > experts_ || top_ > 8) throw invalid_model("toy_routed: top {} of {} experts", top_, experts_);
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t E = s.options.at("experts").as_int(), I = s.options.at("inner").as_int(), H = s.options.at("hidden").as_int();
        return {{"router", {E, H}, ParamKind::Matrix}, {"up", {E * I, H}, ParamKind::Matrix}, {"down", {E * H, I}, ParamKind::Matrix}};
    }
    bool capturable() const override { return true; }
    void forward(StepContext& ctx, const Rows& h, const Rows& x) override {
        toy_routed_ff(h.data, h.dtype == DType::BF16, h.stride, x.f32(), x.stride, router_.data, up_.data, down_.data, ctx.n_tokens, experts_, inner_,
                      hidden_, top_, ctx.stream());
    }

private:
    int experts_, inner_, hidden_, top_;
    Tensor router_, up_, down_;
};

// sin / cos of the position at geometric frequencies, added to the embedding; nothing learned.
class SinusoidPosition final : public PositionEncoding {
public:
    explicit SinusoidPosition(const PartSpec& s) : base_(static_cast<float>(s.options.at("base").as_number())) {}
    bool capturable() const override { return true; }
    int64_t max_positions() const override { return int64_t{1} << 20; }
    void embed(StepContext& ctx, const Tensor& table, float scale, const Rows& x) override {
        kernels::embed_positions(ctx.stream(), ctx.tokens, ctx.positions, table, nullptr, x, ctx.n_tokens, scale);
        toy_sinusoid(x.f32(), ctx.positions, ctx.n_tokens, static_cast<int>(x.cols), base_, ctx.stream());
    }

private:
    float base_;
};

class RmsNorm final : public Norm {
public:
    RmsNorm(const PartSpec& s, const Params& p) : eps_(static_cast<float>(s.options.at("eps").as_number())), weight_(static_cast<const float*>(p.at("weight").data)) {}
    static std::vector<ParamDecl> parameters(const PartSpec& s) { return {{"weight", {s.options.at("hidden").as_int()}, ParamKind::Vector}}; }
    bool capturable() const override { return true; }
    void forward(StepContext& ctx, const Rows& x, const Rows& out, int n_rows, const int32_t* rows) override {
        toy_rms(x.f32(), rows, weight_, out.data, out.dtype == DType::BF16, n_rows, static_cast<int>(x.cols), eps_, ctx.stream());
    }

private:
    float eps_;
    const float* weight_;
};

// x += mixer(norm(x)) + feed_forward(norm(x)): both parts read the same normalised input.  Three slots.
class SideBySideBlock final : public Arrangement {
public:
    explicit SideBySideBlock(const LayerParts& parts)
        : norm_(parts.get<Norm>("norm")), mixer_(parts.get<Mixer>("mixer")), ff_(parts.get<FeedForward>("feed_forward")), keep_(parts) {}
    bool capturable() const override { return norm_.capturable() && mixer_.capturable() && ff_.capturable(); }
    std::vector<Mixer*> mixers() const override { return {&mixer_}; }
    void forward(StepContext& ctx, const Rows& x, CacheUnit unit) override {
        const Rows h = ctx.workspace->get("block.normed", ctx.n_tokens, x.cols, ctx.runtime.dtype);
        norm_.forward(ctx, x, h, ctx.n_tokens, nullptr);
        mixer_.forward(ctx, h, x, unit);
        ff_.forward(ctx, h, x);
    }

private:
    Norm& norm_;
    Mixer& mixer_;
    FeedForward& ff_;
    LayerParts keep_;
};

// The pre-norm block with a third norm over the stream at its end: x += mixer(n1(x)); x += ff(n2(x)); x = n3(x).  Five slots.
class ThirdNormBlock final : public Arrangement {
public:
    explicit ThirdNormBlock(const LayerParts& parts)
        : n1_(parts.get<Norm>("mixer_norm")), mixer_(parts.get<Mixer>("mixer")), n2_(parts.get<Norm>("ff_norm")),
          ff_(parts.get<FeedForward>("feed_forward")), n3_(parts.get<Norm>("out_norm")), keep_(parts) {}
    bool capturable() const override { return n1_.capturable() && mixer_.capturable() && n2_.capturable() && ff_.capturable() && n3_.capturable(); }
    std::vector<Mixer*> mixers() const override { return {&mixer_}; }
    void forward(StepContext& ctx, const Rows& x, CacheUnit unit) override {
        const int T = ctx.n_tokens;
        const Rows h = ctx.workspace->get("block.normed", T, x.cols, ctx.runtime.dtype);
        n1_.forward(ctx, x, h, T, nullptr);
        mixer_.forward(ctx, h, x, unit);
        n2_.forward(ctx, x, h, T, nullptr);
        ff_.forward(ctx, h, x);
        const Rows y = ctx.workspace->get("block.renormed", T, x.cols, DType::F32);
        n3_.forward(ctx, x, y, T, nullptr);
        LIYAB_CUDA(cudaMemcpyAsync(x.data, y.data, static_cast<size_t>(T) * static_cast<size_t>(x.cols) * 4, cudaMemcpyDeviceToDevice, ctx.stream()));
    }

private:
    Norm& n1_;
    Mixer& mixer_;
    Norm& n2_;
    FeedForward& ff_;
    Norm& n3_;
    LayerParts keep_;
};

// An architecture with config.json keys of its own: {"model_type": "toy_stack", "width", "depth", "vocab", "positions",
// "host_loop"}; layers alternate between attention and the running-mean mixer.
class ToyStackConfig final : public ArchitectureConfig {
public:
    explicit ToyStackConfig(const Json& raw) : raw_(raw) {
        for (const char* key : {"width", "depth", "vocab", "positions"})
            if (!raw.contains(key) || !raw.at(key).is_int() || raw.at(key).as_int() <= 0) throw invalid_model("missing or invalid {} in config.json", key);
    }
    Json to_json() const override { return raw_; }
    ModelSpec model_spec() const override {
        const int64_t H = raw_.at("width").as_int(), L = raw_.at("depth").as_int(), V = raw_.at("vocab").as_int(), P = raw_.at("positions").as_int();
        ModelSpec m;
        m.architecture = "toy_stack";
        m.embedding = {V, H, 1.0};
        m.position = {"learned_absolute", Json::object().set("size", H).set("max_positions", P)};
        const PartSpec norm{"layernorm", Json::object().set("size", H).set("eps", 1e-5)};
        for (int64_t i = 0; i < L; ++i) {
            LayerSpec l;
            l.arrangement = "pre_norm";
            l.slots.push_back({"mixer_norm", Role::Norm, norm});
            if (i % 2 == 0)
                l.slots.push_back({"mixer", Role::Mixer, {"attention", Json::object().set("hidden", H).set("n_head", 2).set("n_kv_head", 1).set("head_dim", H / 2).set("scale", 0.25)}});
            else
                l.slots.push_back({"mixer", Role::Mixer, {"toy_running_mean", Json::object().set("hidden", H).set("host_loop", raw_.get_bool("host_loop", false))}});
            l.slots.push_back({"ff_norm", Role::Norm, norm});
            l.slots.push_back({"feed_forward", Role::FeedForward, {"dense", Json::object().set("hidden", H).set("inner", 2 * H).set("activation", "gelu_tanh")}});
            m.layers.push_back(l);
            m.run_order.push_back({static_cast<int>(i), static_cast<int>(i)});
        }
        m.final_norm = norm;
        m.head = {V, H, true, false, 1.0, 0.0};
        m.max_positions = P;
        return m;
    }
    CheckpointMap checkpoint_map() const override {
        CheckpointMap out;
        for (const auto& d : parameter_shapes_of(model_spec())) {
            const bool gain = d.name.size() >= 11 && d.name.compare(d.name.size() - 11, 11, "norm.weight") == 0;
            out.push_back({d.name, CheckpointTensor::one("toy." + d.name, d.shape, d.kind, "none", gain ? 1.0 : 0.0, 0.3)});
        }
        return out;
    }
    static std::vector<ParamDecl> parameter_shapes_of(const ModelSpec& spec);

private:
    Json raw_;
};

}  // namespace

namespace liyab {
std::vector<ParamDecl> parameter_shapes(const ModelSpec& spec);      // decoder.h
}
std::vector<ParamDecl> ToyStackConfig::parameter_shapes_of(const ModelSpec& spec) { return liyab::parameter_shapes(spec); }

extern "C" int liyab_b200_plugin_init(void) {
    mixers().add("toy_running_mean", {RunningMeanMixer::parameters, [](const PartSpec& s, const Params& p, const Runtime&) { return std::make_shared<RunningMeanMixer>(s, p); }});
    feed_forwards().add("toy_routed", {RoutedFeedForward::parameters, [](const PartSpec& s, const Params& p, const Runtime&) { return std::make_shared<RoutedFeedForward>(s, p); }});
    positions().add("toy_sinusoid", {[](const PartSpec&) { return std::vector<ParamDecl>{}; },
                                     [](const PartSpec& s, const Params&, const Runtime&) { return std::make_shared<SinusoidPosition>(s); }});
    norms().add("toy_rms", {RmsNorm::parameters, [](const PartSpec& s, const Params& p, const Runtime&) { return std::make_shared<RmsNorm>(s, p); }});
    arrangements().add("toy_side_by_side", {[](const LayerSpec&, const LayerParts& parts, const Runtime&) { return std::make_shared<SideBySideBlock>(parts); }});
    arrangements().add("toy_third_norm", {[](const LayerSpec&, const LayerParts& parts, const Runtime&) { return std::make_shared<ThirdNormBlock>(parts); }});
    register_architecture({"toy_stack", {}, [](const Json& raw) -> std::unique_ptr<ArchitectureConfig> { return std::make_unique<ToyStackConfig>(raw); }});
    return 0;
}
