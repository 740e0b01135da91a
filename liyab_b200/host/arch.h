// The one registry from an architecture's name to its configuration and model.
//
// The reference keeps a table of `ArchSpec` rows keyed by `general.architecture`
// and answers an unknown name with `Unsupported` plus the list of names it knows
// (src/compat/architecture.cpp:19-426, 578-585).  Here a row is an `Architecture`
// whose `parse` turns the object of config.json into a typed configuration; that
// configuration yields the `ModelSpec` and the map from parameters to the tensor
// names of the model file.  Nothing else is particular to an architecture:
// loader, cache manager, step, scheduler, replay and command line work from the spec.
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "json.h"
#include "spec.h"

namespace liyab {

// What every architecture's typed configuration offers the framework.
class ArchitectureConfig {
public:
    virtual ~ArchitectureConfig() = default;
    virtual Json to_json() const = 0;                       // in the keys of the architecture's own config.json
    virtual ModelSpec model_spec() const = 0;
    virtual CheckpointMap checkpoint_map() const = 0;
    // Regular expressions of tensors a file may hold that carry no weights.
    virtual std::vector<std::string> ignored_tensors() const { return {}; }
    // Prefixes a file may put before every tensor name.
    virtual std::vector<std::string> name_prefixes() const { return {""}; }
};

struct Architecture {
    std::string name;                                       // config.json "model_type"
    std::vector<std::string> class_names;                   // config.json "architectures" entries
    std::function<std::unique_ptr<ArchitectureConfig>(const Json&)> parse;
};

void register_architecture(Architecture arch);
void register_builtin_architectures();                      // idempotent
std::vector<std::string> supported_architectures();
// Chooses the row by `model_type`, else by the first of `architectures`; UNSUPPORTED with the known names otherwise.
const Architecture& find_architecture(const Json& config);
std::unique_ptr<ArchitectureConfig> parse_config(const Json& config);
std::unique_ptr<ArchitectureConfig> read_config(const std::string& model_dir);

std::string read_text_file(const std::string& path);       // IO_ERROR when it cannot be read

}  // namespace liyab
