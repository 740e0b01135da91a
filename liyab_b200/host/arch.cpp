#include "arch.h"

#include <algorithm>
#include <cstdlib>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>

#include "decoder.h"
#include "parts.h"

namespace liyab {
namespace {

std::map<std::string, Architecture>& table() {
    static std::map<std::string, Architecture> t;
    return t;
}

// A model given wholly as data: config.json holds the `ModelSpec` itself under "spec" and, optionally, under
// "checkpoint" the map from parameter paths to the file's tensors (absent: every parameter is stored under its
// own path with its own shape).  This is what "a layer list and a run order are data" means taken to the end; the
// tests use it for models put together from toy parts.
class SpecConfig final : public ArchitectureConfig {
public:
    explicit SpecConfig(const Json& raw) : raw_(raw) {
        const Json* s = raw.find("spec");
        if (s == nullptr) throw invalid_model("missing spec in config.json (model_type liyab_spec needs the model description)");
        spec_ = ModelSpec::from_json(*s);
        if (const Json* c = raw.find("checkpoint"))
            for (const auto& m : c->members()) checkpoint_.push_back({m.first, CheckpointTensor::from_json(m.second, m.first)});
        init_std_ = raw.get_number("init_std", 0.05);
    }
    Json to_json() const override { return raw_; }
    ModelSpec model_spec() const override { return spec_; }
    CheckpointMap checkpoint_map() const override {
        if (!checkpoint_.empty()) return checkpoint_;
        CheckpointMap out;
        for (const auto& d : parameter_shapes(spec_)) {
            const bool gain = d.name.size() >= 11 && d.name.compare(d.name.size() - 11, 11, "norm.weight") == 0;
            out.push_back({d.name, CheckpointTensor::one(d.name, d.shape, d.kind, "none", gain ? 1.0 : 0.0, init_std_)});
        }
        return out;
    }

private:
    Json raw_;
    ModelSpec spec_;
    CheckpointMap checkpoint_;
    double init_std_;
};

}  // namespace

void register_gpt2();      // gpt2.cpp

void register_architecture(Architecture arch) { table()[arch.name] = std::move(arch); }

void register_builtin_architectures() {
    static std::once_flag once;
    std::call_once(once, [] {
        register_gpt2();
        register_architecture({"liyab_spec", {}, [](const Json& raw) { return std::make_unique<SpecConfig>(raw); }});
    });
    // Plug-ins named by the environment (paths separated by ':') are loaded once, so that the programs can run
    // models made of parts from outside the library.
    static std::once_flag plugins;
    std::call_once(plugins, [] {
        const char* env = std::getenv("LIYAB_B200_PLUGINS");
        if (env == nullptr) return;
        std::string list = env;
        size_t at = 0;
        while (at <= list.size()) {
            const size_t end = std::min(list.find(':', at), list.size());
            if (end > at) load_plugin(list.substr(at, end - at));
            at = end + 1;
        }
    });
}

std::vector<std::string> supported_architectures() {
    register_builtin_architectures();
    std::vector<std::string> out;
    for (const auto& kv : table()) out.push_back(kv.first);
    return out;
}

const Architecture& find_architecture(const Json& config) {
    register_builtin_architectures();
    if (!config.is_object()) throw invalid_model("config.json does not hold a JSON object");
    const Json* name = config.find("model_type");
    if (name != nullptr && name->is_string()) {
        const auto it = table().find(name->as_string());
        if (it != table().end()) return it->second;
    }
    std::string shown = name != nullptr && name->is_string() ? name->as_string() : "";
    if (const Json* classes = config.find("architectures"); classes != nullptr && classes->is_array()) {
        for (const auto& cls : classes->items()) {
            if (!cls.is_string()) continue;
            for (const auto& kv : table())
                if (std::find(kv.second.class_names.begin(), kv.second.class_names.end(), cls.as_string()) != kv.second.class_names.end())
                    return kv.second;
            if (shown.empty()) shown = cls.as_string();
        }
    }
    std::string known;
    for (const auto& n : supported_architectures()) known += (known.empty() ? "" : ", ") + n;
    throw unsupported("architecture '{}' is not supported; supported: {}", shown.empty() ? "nothing" : shown, known);
}

std::unique_ptr<ArchitectureConfig> parse_config(const Json& config) { return find_architecture(config).parse(config); }

std::string read_text_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw make_error(Code::Io, "cannot read {}", path);
    std::ostringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

std::unique_ptr<ArchitectureConfig> read_config(const std::string& model_dir) {
    const std::string path = model_dir + "/config.json";
    const std::string text = read_text_file(path);
    Json raw;
    try {
        raw = Json::parse(text, path);
    } catch (const Error& e) {
        throw invalid_model("{}", e.message());
    }
    if (!raw.is_object()) throw invalid_model("{} does not hold a JSON object", path);
    return parse_config(raw);
}

}  // namespace liyab
