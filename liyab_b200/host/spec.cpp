#include "spec.h"

namespace liyab {

Json PartSpec::to_json() const {
    Json j = Json::object();
    j.set("kind", kind);
    for (const auto& m : options.members()) j.set(m.first, m.second);
    return j;
}

PartSpec PartSpec::from_json(const Json& j, const std::string& what) {
    if (!j.is_object() || !j.contains("kind") || !j.at("kind").is_string())
        throw invalid_model("{} must be an object with a string 'kind'", what);
    PartSpec p;
    p.kind = j.at("kind").as_string();
    for (const auto& m : j.members())
        if (m.first != "kind") p.options.set(m.first, m.second);
    return p;
}

const char* role_name(Role r) {
    switch (r) {
        case Role::Norm: return "norm";
        case Role::Mixer: return "mixer";
        case Role::FeedForward: return "feed_forward";
    }
    return "?";
}

Role role_from_name(const std::string& name) {
    if (name == "norm") return Role::Norm;
    if (name == "mixer") return Role::Mixer;
    if (name == "feed_forward") return Role::FeedForward;
    throw invalid_model("unknown slot role '{}' (norm, mixer or feed_forward)", name);
}

const SlotSpec* LayerSpec::find(const std::string& name) const {
    for (const auto& s : slots)
        if (s.name == name) return &s;
    return nullptr;
}

const SlotSpec& LayerSpec::slot(const std::string& name) const {
    const SlotSpec* s = find(name);
    if (s == nullptr) throw invalid_model("arrangement '{}' needs a slot named '{}'", arrangement, name);
    return *s;
}

Json ModelSpec::to_json() const {
    Json j = Json::object();
    j.set("architecture", architecture);
    j.set("embedding", Json::object().set("vocab_size", embedding.vocab_size).set("size", embedding.size).set("scale", embedding.scale));
    j.set("position", position.to_json());
    Json ls = Json::array();
    for (const auto& l : layers) {
        Json lj = Json::object();
        lj.set("arrangement", l.arrangement);
        if (l.options.size()) lj.set("options", l.options);
        Json slots = Json::array();
        for (const auto& s : l.slots)
            slots.push(Json::object().set("name", s.name).set("role", role_name(s.role)).set("part", s.part.to_json()));
        lj.set("slots", slots);
        ls.push(lj);
    }
    j.set("layers", ls);
    Json ro = Json::array();
    for (const auto& e : run_order) ro.push(Json::object().set("layer", e.layer).set("cache", e.cache));
    j.set("run_order", ro);
    j.set("final_norm", final_norm.to_json());
    j.set("head", Json::object().set("vocab_size", head.vocab_size).set("size", head.size).set("tied", head.tied)
                       .set("bias", head.bias).set("logit_scale", head.logit_scale).set("soft_cap", head.soft_cap));
    j.set("max_positions", max_positions);
    j.set("eos_token_id", eos_token_id ? Json(*eos_token_id) : Json(nullptr));
    return j;
}

ModelSpec ModelSpec::from_json(const Json& j) {
    if (!j.is_object()) throw invalid_model("a model description must be a JSON object");
    ModelSpec s;
    try {
        s.architecture = j.get_string("architecture", "spec");
        const Json& e = j.at("embedding");
        s.embedding = {e.at("vocab_size").as_int(), e.at("size").as_int(), e.get_number("scale", 1.0)};
        s.position = PartSpec::from_json(j.at("position"), "position");
        int li = 0;
        for (const auto& lj : j.at("layers").items()) {
            LayerSpec l;
            l.arrangement = lj.at("arrangement").as_string();
            if (const Json* o = lj.find("options")) l.options = *o;
            for (const auto& sj : lj.at("slots").items()) {
                SlotSpec slot;
                slot.name = sj.at("name").as_string();
                slot.role = role_from_name(sj.at("role").as_string());
                slot.part = PartSpec::from_json(sj.at("part"), std::format("layers[{}].{}", li, slot.name));
                if (l.find(slot.name) != nullptr) throw invalid_model("layers[{}] names the slot '{}' twice", li, slot.name);
                l.slots.push_back(std::move(slot));
            }
            s.layers.push_back(std::move(l));
            ++li;
        }
        for (const auto& r : j.at("run_order").items())
            s.run_order.push_back({static_cast<int>(r.at("layer").as_int()), static_cast<int>(r.at("cache").as_int())});
        s.final_norm = PartSpec::from_json(j.at("final_norm"), "final_norm");
        const Json& h = j.at("head");
        s.head = {h.at("vocab_size").as_int(), h.at("size").as_int(), h.get_bool("tied", true), h.get_bool("bias", false),
                  h.get_number("logit_scale", 1.0), h.get_number("soft_cap", 0.0)};
        s.max_positions = j.at("max_positions").as_int();
        if (const Json* eos = j.find("eos_token_id"); eos != nullptr && !eos->is_null()) s.eos_token_id = eos->as_int();
    } catch (const Error& err) {
        if (err.code() == Code::InvalidModel) throw;
        throw invalid_model("malformed model description: {}", err.message());
    }
    return s;
}

const char* param_kind_name(ParamKind k) {
    switch (k) {
        case ParamKind::Matrix: return "matrix";
        case ParamKind::Table: return "table";
        case ParamKind::Vector: return "vector";
        case ParamKind::Index: return "index";
    }
    return "?";
}

ParamKind param_kind_from_name(const std::string& name) {
    if (name == "matrix") return ParamKind::Matrix;
    if (name == "table") return ParamKind::Table;
    if (name == "vector") return ParamKind::Vector;
    if (name == "index") return ParamKind::Index;
    throw invalid_model("unknown parameter kind '{}' (matrix, table, vector or index)", name);
}

Json CheckpointTensor::to_json() const {
    Json j = Json::object();
    Json src = Json::array();
    for (const auto& s : sources) src.push(Json::object().set("name", s.name).set("shape", Json::array_of(s.shape)));
    j.set("sources", src);
    j.set("transform", transform);
    if (sources.size() > 1) j.set("concat_axis", concat_axis);
    if (slice_axis >= 0) j.set("slice", Json::object().set("axis", slice_axis).set("begin", slice_begin).set("end", slice_end));
    j.set("kind", param_kind_name(kind));
    j.set("init", Json::array().push(init_mean).push(init_std));
    return j;
}

CheckpointTensor CheckpointTensor::from_json(const Json& j, const std::string& what) {
    CheckpointTensor t;
    try {
        for (const auto& s : j.at("sources").items()) t.sources.push_back({s.at("name").as_string(), s.at("shape").int_list()});
        if (t.sources.empty()) throw invalid_model("{} names no tensor of the file", what);
        t.transform = j.get_string("transform", "none");
        t.concat_axis = static_cast<int>(j.get_int("concat_axis", 0));
        if (const Json* s = j.find("slice")) {
            t.slice_axis = static_cast<int>(s->at("axis").as_int());
            t.slice_begin = s->at("begin").as_int();
            t.slice_end = s->at("end").as_int();
        }
        t.kind = param_kind_from_name(j.get_string("kind", "matrix"));
        if (const Json* init = j.find("init")) {
            t.init_mean = init->items().at(0).as_number();
            t.init_std = init->items().at(1).as_number();
        }
    } catch (const Error& err) {
        if (err.code() == Code::InvalidModel) throw;
        throw invalid_model("malformed checkpoint entry for {}: {}", what, err.message());
    }
    return t;
}

std::string shape_text(const std::vector<int64_t>& shape) {
    std::string s = "[";
    for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
    return s + "]";
}

int64_t shape_numel(const std::vector<int64_t>& shape) {
    int64_t n = 1;
    for (const int64_t d : shape) n *= d;
    return n;
}

}  // namespace liyab
