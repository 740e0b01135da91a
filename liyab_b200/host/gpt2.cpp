#include "gpt2.h"

#include <cmath>
#include <map>

namespace liyab {
namespace {

const std::map<std::string, std::string>& activations() {
    static const std::map<std::string, std::string> m{
        {"gelu_new", "gelu_tanh"}, {"gelu_pytorch_tanh", "gelu_tanh"}, {"gelu_fast", "gelu_tanh"}, {"gelu", "gelu_erf"}};
    return m;
}

int64_t int_key(const Json& raw, const char* key, std::initializer_list<const char*> aliases = {}, std::optional<int64_t> fallback = {},
                int64_t lo = 1, int64_t hi = int64_t{1} << 24) {
    const Json* v = raw.find(key);
    for (const char* a : aliases)
        if (v == nullptr || v->is_null()) v = raw.find(a);
    if (v == nullptr || v->is_null()) {
        if (fallback) return *fallback;
        throw invalid_model("missing or invalid {} in config.json (got nothing, need an integer in [{}, {}])", key, lo, hi);
    }
    if (!v->is_int() || v->as_int() < lo || v->as_int() > hi)
        throw invalid_model("missing or invalid {} in config.json (got {}, need an integer in [{}, {}])", key, v->dump(), lo, hi);
    return v->as_int();
}

bool bool_key(const Json& raw, const char* key, bool fallback) {
    const Json* v = raw.find(key);
    if (v == nullptr || v->is_null()) return fallback;
    if (!v->is_bool()) throw invalid_model("invalid {} in config.json (got {}, need true or false)", key, v->dump());
    return v->as_bool();
}

}  // namespace

std::unique_ptr<GPT2Config> GPT2Config::parse(const Json& raw) {
    auto c = std::make_unique<GPT2Config>();
    c->n_layer = int_key(raw, "n_layer", {"num_hidden_layers"});
    c->n_embd = int_key(raw, "n_embd", {"hidden_size"});
    c->n_head = int_key(raw, "n_head", {"num_attention_heads"});
    if (c->n_embd % c->n_head != 0)
        throw invalid_model("invalid head dimensions: n_embd {} is not a multiple of n_head {}", c->n_embd, c->n_head);
    c->n_inner = int_key(raw, "n_inner", {}, 4 * c->n_embd);
    c->n_positions = int_key(raw, "n_positions", {"n_ctx", "max_position_embeddings"});
    c->vocab_size = int_key(raw, "vocab_size");
    if (const Json* eps = raw.find("layer_norm_epsilon"); eps != nullptr && !eps->is_null()) {
        if (!eps->is_number() || !std::isfinite(eps->as_number()) || eps->as_number() < 0)
            throw invalid_model("invalid layer_norm_epsilon in config.json (got {}, need a finite number >= 0)", eps->dump());
        c->layer_norm_epsilon = eps->as_number();
    }
    if (const Json* act = raw.find("activation_function"); act != nullptr && !act->is_null()) {
        if (!act->is_string() || !activations().count(act->as_string())) {
            std::string known;
            for (const auto& kv : activations()) known += (known.empty() ? "" : ", ") + kv.first;
            throw unsupported("activation_function {} is not supported; supported: {}", act->dump(), known);
        }
        c->activation_function = act->as_string();
    }
    // reorder_and_upcast_attn only changes where the layer factor is applied in half precision; scores are
    // computed in 32-bit here either way.
    bool_key(raw, "reorder_and_upcast_attn", false);
    if (const Json* x = raw.find("add_cross_attention"); x != nullptr && x->is_bool() && x->as_bool())
        throw unsupported("add_cross_attention is not supported");
    for (const char* key : {"eos_token_id", "bos_token_id"}) {
        const Json* v = raw.find(key);
        if (v == nullptr || v->is_null()) continue;
        if (!v->is_int() || v->as_int() < 0 || v->as_int() >= c->vocab_size)
            throw invalid_model("invalid {} in config.json (got {}, need an id below vocab_size {})", key, v->dump(), c->vocab_size);
        (std::string(key) == "eos_token_id" ? c->eos_token_id : c->bos_token_id) = v->as_int();
    }
    c->scale_attn_weights = bool_key(raw, "scale_attn_weights", true);
    c->scale_attn_by_inverse_layer_idx = bool_key(raw, "scale_attn_by_inverse_layer_idx", false);
    c->tie_word_embeddings = bool_key(raw, "tie_word_embeddings", true);
    return c;
}

double GPT2Config::attention_scale(int64_t layer) const {
    double scale = scale_attn_weights ? 1.0 / std::sqrt(static_cast<double>(head_dim())) : 1.0;
    if (scale_attn_by_inverse_layer_idx) scale /= static_cast<double>(layer + 1);
    return scale;
}

Json GPT2Config::to_json() const {
    Json j = Json::object();
    j.set("model_type", "gpt2").set("architectures", Json::array().push("GPT2LMHeadModel"));
    j.set("n_layer", n_layer).set("n_embd", n_embd).set("n_head", n_head).set("n_inner", n_inner);
    j.set("n_positions", n_positions).set("vocab_size", vocab_size).set("layer_norm_epsilon", layer_norm_epsilon);
    j.set("activation_function", activation_function).set("scale_attn_weights", scale_attn_weights);
    j.set("scale_attn_by_inverse_layer_idx", scale_attn_by_inverse_layer_idx).set("tie_word_embeddings", tie_word_embeddings);
    j.set("eos_token_id", eos_token_id ? Json(*eos_token_id) : Json(nullptr));
    j.set("bos_token_id", bos_token_id ? Json(*bos_token_id) : Json(nullptr));
    return j;
}

ModelSpec GPT2Config::model_spec() const {
    const int64_t d = n_embd;
    ModelSpec m;
    m.architecture = "gpt2";
    m.embedding = {vocab_size, d, 1.0};
    m.position = {"learned_absolute", Json::object().set("size", d).set("max_positions", n_positions)};
    const PartSpec norm{"layernorm", Json::object().set("size", d).set("eps", layer_norm_epsilon).set("bias", true)};
    for (int64_t i = 0; i < n_layer; ++i) {
        LayerSpec l;
        l.arrangement = "pre_norm";
        l.slots.push_back({"mixer_norm", Role::Norm, norm});
        l.slots.push_back({"mixer", Role::Mixer,
                           {"attention", Json::object().set("hidden", d).set("n_head", n_head).set("n_kv_head", n_head)
                                             .set("head_dim", head_dim()).set("scale", attention_scale(i)).set("window", 0).set("bias", true)}});
        l.slots.push_back({"ff_norm", Role::Norm, norm});
        l.slots.push_back({"feed_forward", Role::FeedForward,
                           {"dense", Json::object().set("hidden", d).set("inner", n_inner)
                                         .set("activation", activations().at(activation_function)).set("bias", true)}});
        m.layers.push_back(std::move(l));
        m.run_order.push_back({static_cast<int>(i), static_cast<int>(i)});
    }
    m.final_norm = norm;
    m.head = {vocab_size, d, tie_word_embeddings, false, 1.0, 0.0};
    m.max_positions = n_positions;
    m.eos_token_id = eos_token_id;
    return m;
}

CheckpointMap GPT2Config::checkpoint_map() const {
    // GPT-2's projections are stored [in, out] (the converter the reference relies on transposes them:
    // docs/validation/models-stage1/converter-classic.patch:11-22); the engine keeps every matrix [out, in].
    const int64_t d = n_embd, ff = n_inner, L = n_layer;
    const double proj_std = 0.02 / std::sqrt(2.0 * static_cast<double>(L));
    using K = ParamKind;
    CheckpointMap m;
    m.push_back({"embedding.weight", CheckpointTensor::one("wte.weight", {vocab_size, d}, K::Table)});
    m.push_back({"position.weight", CheckpointTensor::one("wpe.weight", {n_positions, d}, K::Table)});
    m.push_back({"final_norm.weight", CheckpointTensor::one("ln_f.weight", {d}, K::Vector, "none", 1.0, 0.1)});
    m.push_back({"final_norm.bias", CheckpointTensor::one("ln_f.bias", {d}, K::Vector)});
    if (!tie_word_embeddings) m.push_back({"head.weight", CheckpointTensor::one("lm_head.weight", {vocab_size, d})});
    for (int64_t i = 0; i < L; ++i) {
        const std::string p = std::format("layers.{}.", i), h = std::format("h.{}.", i);
        m.push_back({p + "mixer_norm.weight", CheckpointTensor::one(h + "ln_1.weight", {d}, K::Vector, "none", 1.0, 0.1)});
        m.push_back({p + "mixer_norm.bias", CheckpointTensor::one(h + "ln_1.bias", {d}, K::Vector)});
        m.push_back({p + "mixer.qkv.weight", CheckpointTensor::one(h + "attn.c_attn.weight", {d, 3 * d}, K::Matrix, "transpose")});
        m.push_back({p + "mixer.qkv.bias", CheckpointTensor::one(h + "attn.c_attn.bias", {3 * d}, K::Vector)});
        m.push_back({p + "mixer.out.weight", CheckpointTensor::one(h + "attn.c_proj.weight", {d, d}, K::Matrix, "transpose", 0.0, proj_std)});
        m.push_back({p + "mixer.out.bias", CheckpointTensor::one(h + "attn.c_proj.bias", {d}, K::Vector)});
        m.push_back({p + "ff_norm.weight", CheckpointTensor::one(h + "ln_2.weight", {d}, K::Vector, "none", 1.0, 0.1)});
        m.push_back({p + "ff_norm.bias", CheckpointTensor::one(h + "ln_2.bias", {d}, K::Vector)});
        m.push_back({p + "feed_forward.up.weight", CheckpointTensor::one(h + "mlp.c_fc.weight", {d, ff}, K::Matrix, "transpose")});
        m.push_back({p + "feed_forward.up.bias", CheckpointTensor::one(h + "mlp.c_fc.bias", {ff}, K::Vector)});
        m.push_back({p + "feed_forward.down.weight", CheckpointTensor::one(h + "mlp.c_proj.weight", {ff, d}, K::Matrix, "transpose", 0.0, proj_std)});
        m.push_back({p + "feed_forward.down.bias", CheckpointTensor::one(h + "mlp.c_proj.bias", {d}, K::Vector)});
    }
    return m;
}

std::vector<std::string> GPT2Config::ignored_tensors() const {
    // Tensors a GPT-2 file may hold that carry no weights: the causal-mask buffers (dropped by the converter,
    // converter-classic.patch:14-19) and a stored copy of the tied head.
    std::vector<std::string> pats{R"(h\.\d+\.attn\.bias)", R"(h\.\d+\.attn\.masked_bias)"};
    if (tie_word_embeddings) pats.push_back(R"(lm_head\.weight)");
    return pats;
}

void register_gpt2() {
    register_architecture({"gpt2", {"GPT2LMHeadModel", "GPT2Model"}, [](const Json& raw) -> std::unique_ptr<ArchitectureConfig> {
                               return GPT2Config::parse(raw);
                           }});
}

}  // namespace liyab
