// Typed descriptions of a model, part by part.
//
// A model is data before it is code: an architecture's configuration is turned
// into a `ModelSpec`: a list of `LayerSpec`s and a `run_order` that says which
// layer runs when and whose cache it reads.  A layer is an arrangement (by kind)
// and an ordered list of named slots; a slot has a role (norm, mixer or
// feed-forward) and a `PartSpec`, the part's kind with its own sizes and
// constants.  The parts registry (parts.h) maps each kind to the class that
// implements it, so a layer's parts are chosen layer by layer and no part knows
// the model it is in.  Everything here can be written to and read from JSON.
//
// The reference keeps the same split: `ModelConfig` holds the global facts and a
// `BlockPlan` per block holds n_head, n_head_kv, n_ff, head_dim, attn_scale, the
// mixer and the feed-forward kind (src/compat/architecture.h:282-380, 452-630).
#pragma once

#include <cstdint>
#include <map>
#include <optional>
#include <string>
#include <vector>

#include "json.h"

namespace liyab {

// `kind` selects the implementation; `options` are the part's sizes and constants.
struct PartSpec {
    std::string kind;
    Json options = Json::object();

    Json to_json() const;
    static PartSpec from_json(const Json& j, const std::string& what);
};

enum class Role { Norm, Mixer, FeedForward };
const char* role_name(Role r);
Role role_from_name(const std::string& name);

struct SlotSpec {
    std::string name;        // the slot's name inside its layer, and the prefix of its parameters
    Role role;
    PartSpec part;
};

// One block: which parts, and how they are arranged around the residual stream.
struct LayerSpec {
    std::string arrangement;             // e.g. "pre_norm"
    Json options = Json::object();       // constants of the arrangement itself
    std::vector<SlotSpec> slots;

    const SlotSpec* find(const std::string& name) const;
    const SlotSpec& slot(const std::string& name) const;      // INVALID_MODEL when absent
};

// One entry of the run order.  `layer` indexes ModelSpec::layers (a layer may be
// named twice: its weights are then used twice).  `cache` names the cache unit
// this run of the layer reads; when it equals the entry's own index in the run
// order the entry also writes that unit, otherwise it reads the keys and values
// that the entry numbered `cache` wrote (and writes none of its own).
struct RunEntry {
    int layer = 0;
    int cache = 0;
};

struct EmbeddingSpec {
    int64_t vocab_size = 0;
    int64_t size = 0;
    double scale = 1.0;
};

// The projection to the vocabulary; `tied` reuses the embedding table.  After the
// product: + bias, * logit_scale, then soft_cap * tanh(x / soft_cap) when soft_cap > 0
// (the reference's finish_logits and apply_final_softcap; both neutral for gpt2).
struct HeadSpec {
    int64_t vocab_size = 0;
    int64_t size = 0;
    bool tied = true;
    bool bias = false;
    double logit_scale = 1.0;
    double soft_cap = 0.0;
};

struct ModelSpec {
    std::string architecture;
    EmbeddingSpec embedding;
    PartSpec position;
    std::vector<LayerSpec> layers;
    std::vector<RunEntry> run_order;
    PartSpec final_norm;
    HeadSpec head;
    int64_t max_positions = 0;
    std::optional<int64_t> eos_token_id;

    int64_t vocab_size() const { return embedding.vocab_size; }
    int64_t hidden() const { return embedding.size; }
    Json to_json() const;
    static ModelSpec from_json(const Json& j);
};

// How a parameter is stored in reduced precision: matrices and tables are kept in
// the compute type, vectors (norm gains, biases) always in 32-bit, index tables in int32.
enum class ParamKind { Matrix, Table, Vector, Index };
const char* param_kind_name(ParamKind k);
ParamKind param_kind_from_name(const std::string& name);

struct ParamDecl {
    std::string name;
    std::vector<int64_t> shape;
    ParamKind kind = ParamKind::Matrix;
};

// Where a parameter lives in the model file.  `sources` are tensors of the file
// (each with the shape it has there).  After reading, `transform` ("none" or
// "transpose", for matrices stored [in, out]) is applied to every source; several
// sources are joined along `concat_axis` (separate q, k, v matrices becoming one
// fused projection); then, when `slice_axis` >= 0, rows [slice_begin, slice_end)
// of that axis are kept (one half of a fused [gate | up]).  `init` is (mean, std)
// for the random-weights mode.
struct CheckpointSource {
    std::string name;
    std::vector<int64_t> shape;
};
struct CheckpointTensor {
    std::vector<CheckpointSource> sources;
    std::string transform = "none";
    int concat_axis = 0;
    int slice_axis = -1;
    int64_t slice_begin = 0, slice_end = 0;
    ParamKind kind = ParamKind::Matrix;
    double init_mean = 0.0, init_std = 0.02;

    static CheckpointTensor one(std::string name, std::vector<int64_t> shape, ParamKind kind = ParamKind::Matrix,
                                std::string transform = "none", double mean = 0.0, double std = 0.02) {
        CheckpointTensor t;
        t.sources.push_back({std::move(name), std::move(shape)});
        t.kind = kind;
        t.transform = std::move(transform);
        t.init_mean = mean;
        t.init_std = std;
        return t;
    }
    Json to_json() const;
    static CheckpointTensor from_json(const Json& j, const std::string& what);
};

// Parameter path ("layers.3.mixer.qkv.weight") -> where it comes from, in a fixed order.
using CheckpointMap = std::vector<std::pair<std::string, CheckpointTensor>>;

std::string shape_text(const std::vector<int64_t>& shape);
int64_t shape_numel(const std::vector<int64_t>& shape);

}  // namespace liyab
