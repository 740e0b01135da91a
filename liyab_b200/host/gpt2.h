// GPT-2: a dense pre-LayerNorm decoder with learned absolute positions, fused
// query/key/value attention, an ungated GELU feed-forward and a tied output head.
//
// The reference's row for it fixes LayerNorm, the tanh GELU and "no rotary"
// (src/compat/architecture.cpp:81-88); sizes come from the file's metadata
// (architecture.cpp:588-600, 699-708, 799-805, 975-985, 994-998, 1012-1022).  Here
// the same facts are read from the keys of GPT-2's own config.json.  Two options
// of that file have no counterpart in the reference and are wired onto the
// per-layer attention scale: `scale_attn_weights` and
// `scale_attn_by_inverse_layer_idx`; and `activation_function` may name the exact
// (erf) GELU, which the reference implements beside the tanh form
// (src/core/transformer.cpp:125-142).
#pragma once

#include <optional>

#include "arch.h"

namespace liyab {

struct GPT2Config final : public ArchitectureConfig {
    int64_t n_layer = 0, n_embd = 0, n_head = 0, n_inner = 0, n_positions = 0, vocab_size = 0;
    double layer_norm_epsilon = 1e-5;
    std::string activation_function = "gelu_new";
    bool scale_attn_weights = true;
    bool scale_attn_by_inverse_layer_idx = false;
    bool tie_word_embeddings = true;
    std::optional<int64_t> eos_token_id, bos_token_id;

    static std::unique_ptr<GPT2Config> parse(const Json& raw);
    int64_t head_dim() const { return n_embd / n_head; }
    // 1/sqrt(head_dim) computed as the reference does (architecture.cpp:975-985), divided by (layer + 1) when
    // the configuration asks for it.
    double attention_scale(int64_t layer) const;

    Json to_json() const override;
    ModelSpec model_spec() const override;
    CheckpointMap checkpoint_map() const override;
    std::vector<std::string> ignored_tensors() const override;
    std::vector<std::string> name_prefixes() const override { return {"", "transformer."}; }
};

}  // namespace liyab
