#include "builtin_parts.h"

#include <mutex>

namespace liyab {

using namespace builtin;

void register_builtin_parts() {
    static std::once_flag once;
    std::call_once(once, [] {
        norms().add("layernorm", {LayerNorm::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                      return std::make_shared<LayerNorm>(s, p);
                                  }});
        positions().add("learned_absolute", {LearnedAbsolutePosition::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                                 return std::make_shared<LearnedAbsolutePosition>(s, p);
                                             }});
        positions().add("none", {[](const PartSpec&) { return std::vector<ParamDecl>{}; },
                                 [](const PartSpec& s, const Params&, const Runtime&) { return std::make_shared<NoPosition>(s); }});
        mixers().add("attention", {CausalSelfAttention::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                       return std::make_shared<CausalSelfAttention>(s, p);
                                   }});
        feed_forwards().add("dense", {DenseFeedForward::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                          return std::make_shared<DenseFeedForward>(s, p);
                                      }});
        arrangements().add("pre_norm", {[](const LayerSpec& l, const LayerParts& parts, const Runtime&) {
                               return std::make_shared<PreNormBlock>(l, parts);
                           }});
    });
}

}  // namespace liyab
