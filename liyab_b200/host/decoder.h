// A decoder put together from a `ModelSpec`: embedding, position encoding, the
// layers in their run order, final norm and the head.
//
// Nothing here is particular to an architecture: the spec says which parts every
// layer has, the registries say which class implements each kind, and the
// parameters arrive as {path: tensor} with paths made of the part's place
// ("layers.3.mixer.qkv.weight").  The forward pass follows the reference's
// (embed -> add_positions -> every block -> final norm and head on the wanted rows
// only: src/core/transformer.cpp:6589-6769).
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "parts.h"
#include "spec.h"

namespace liyab {

// Every parameter the model needs, from the parts' own declarations, with full paths.
std::vector<ParamDecl> parameter_shapes(const ModelSpec& spec);

class DecoderModel {
public:
    DecoderModel(ModelSpec spec, const Params& params, Runtime runtime);

    ModelSpec spec;
    Runtime runtime;
    Tensor embedding;
    std::shared_ptr<PositionEncoding> position;
    struct Layer {
        LayerParts parts;
        std::shared_ptr<Arrangement> block;
    };
    std::vector<Layer> layers;
    std::shared_ptr<Norm> final_norm;
    Tensor head_weight;
    const float* head_bias = nullptr;

    // -- what the cache manager has to provide
    std::map<int, KvNeed> kv_needs() const;          // cache units (run-order entries that write keys and values)
    std::map<int, StateNeed> state_needs() const;
    int64_t max_positions() const;
    size_t weight_bytes() const;                     // bytes of all parameters, a tied table counted once
    bool capturable() const;                         // every part may be captured into a CUDA graph

    // Runs the step's tokens; returns logits [R, vocab] float32 at ctx.logit_rows (rows == 0 when R = 0).
    Rows forward(StepContext& ctx);

private:
    Mixer* mixer_of(const RunEntry& e) const;
    Params params_;
};

}  // namespace liyab
