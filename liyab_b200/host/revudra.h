// Revudra: a decoder whose sublayers read the residual stream as it is and whose outputs pass an RMS norm before they join it,
// x += m norm(mixer(x)); x += m norm(feed_forward(x)).  The embedded row is scaled by a constant; the logits too.  A layer's
// mixer is one of three: softmax attention under a sliding window (grouped key/value heads, queries and keys normed over the
// whole projection and rotated in part, a sink a head in the softmax's divisor, values blended with those of the first such
// layer, a sigmoid gate element by element); a matrix memory per head with a fixed decay whose queries, keys and values pass
// SiLU, all heads normed together and gated; attention whose keys and values are maps of a cached latent row beside one rotated
// key part shared by the heads (queries through a normed latent of their own, pairs rotated side by side, causal, a sink and a
// sigmoid gate a head).  The feed-forward is dense with the square of relu, a set of small gated experts chosen by a table over
// the token ids (equal weights), or absent.  No position table; the head is a matrix of its own.
//
// config.json: {"architecture": "Revudra", "vocab", "width", "norm": {"eps"}, "residual_mult", "embedding": {"scale"}, "logit_scale",
// "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"base", "dims"},
// "v_mix"}} | {"type": "lightning", "mixer": {"heads", "dim", "vdim", "decay": [..]}} | {"type": "latent_attention", "mixer":
// {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot": {"base", "dims"}}}, each with "mlp": {"kind": "dense",
// "ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}} | null]}.
// Tensors: embed, head, final.norm, and per layer l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*.
#pragma once

#include "arch.h"

namespace liyab {

struct RevudraConfig final : public ArchitectureConfig {
    enum class Mixer { Attention, Lightning, Latent };
    struct Layer {
        Mixer mixer = Mixer::Attention;
        int64_t heads = 0, dim = 0, vdim = 0;
        // attention under a window
        int64_t kv_heads = 0, window = 0;
        bool v_mix = false;
        // attention of both kinds
        int64_t rot_dims = 0;
        double rot_base = 10000.0, scale = 1.0;
        // latent attention
        int64_t rot_dim = 0, kv_rank = 0, q_rank = 0;
        // matrix memory
        std::vector<double> decay;
        // feed-forward: ff > 0 dense; experts > 0 chosen by table; neither: none
        int64_t ff = 0, experts = 0, top = 0, expert_ff = 0;
    };
    int64_t vocab = 0, width = 0;
    double norm_eps = 1e-6, residual_mult = 1.0, embedding_scale = 1.0, logit_scale = 1.0;
    int64_t max_positions = int64_t{1} << 17;        // the design has no limit of its own; the engine's tables need one
    std::vector<Layer> layers;
    Json raw;

    static std::unique_ptr<RevudraConfig> parse(const Json& raw);
    Json to_json() const override { return raw; }
    ModelSpec model_spec() const override;
    CheckpointMap checkpoint_map() const override;
    std::vector<std::string> ignored_tensors() const override;

private:
    // The first layer whose values the later ones blend with; -1: no layer blends.
    int value_source() const;
};

}  // namespace liyab
