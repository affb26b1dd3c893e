#include "builtin_parts.h"
#include "parallel_parts.h"
#include "gated_parts.h"
#include "state_parts.h"

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
        norms().add("rms_norm", {GroupedRmsNorm::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                     return std::make_shared<GroupedRmsNorm>(s, p);
                                 }});
        shifts().add("lerp_previous", {LerpShift::parameters, [](const PartSpec& s, const Params& p, const Runtime& rt) {
                                           return std::make_shared<LerpShift>(s, p, rt);
                                       }});
        mixers().add("latent_attention", {LatentAttention::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                              return std::make_shared<LatentAttention>(s, p);
                                          }});
        token_inputs().add("gated_side", {GatedTokenSide::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                              return std::make_shared<GatedTokenSide>(s, p);
                                          }});
        mixers().add("gated_attention", {GatedAttention::parameters, [](const PartSpec& s, const Params& p, const Runtime& rt) {
                                             return std::make_shared<GatedAttention>(s, p, rt);
                                         }});
        mixers().add("matrix_memory", {MatrixMemory::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                           return std::make_shared<MatrixMemory>(s, p);
                                       }});
        mixers().add("branch_sum", {BranchSum::parameters, [](const PartSpec& s, const Params& p, const Runtime& rt) {
                                        return std::make_shared<BranchSum>(s, p, rt);
                                    }});
        feed_forwards().add("gated", {GatedFeedForward::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                          return std::make_shared<GatedFeedForward>(s, p);
                                      }});
        feed_forwards().add("routed", {RoutedExperts::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                           return std::make_shared<RoutedExperts>(s, p);
                                       }});
        positions().add("sinusoid", {SinusoidPosition::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                         return std::make_shared<SinusoidPosition>(s, p);
                                     }});
        mixers().add("state_space", {StateSpaceMixer::parameters, [](const PartSpec& s, const Params& p, const Runtime&) {
                                         return std::make_shared<StateSpaceMixer>(s, p);
                                     }});
        arrangements().add("parallel", {[](const LayerSpec& l, const LayerParts& parts, const Runtime&) {
                               return std::make_shared<ParallelBlock>(l, parts);
                           }});
        arrangements().add("sublayer_norm", {[](const LayerSpec& l, const LayerParts& parts, const Runtime&) {
                               return std::make_shared<SublayerNormBlock>(l, parts);
                           }});
        arrangements().add("pre_norm", {[](const LayerSpec& l, const LayerParts& parts, const Runtime&) {
                               return std::make_shared<PreNormBlock>(l, parts);
                           }});
    });
}

}  // namespace liyab
