// Viresun: a decoder of pre-norm blocks, x += mixer(norm(x)); x += feed_forward(norm(x)), whose norms have one gain for all
// coordinates (stored as a single number).  The embedded row gets a sinusoid of its position and passes the model's norm.  A
// block's mixer is either softmax attention under a sliding window (queries and keys over their root mean square without a
// gain, a temperature on the queries that grows with the logarithm of the position, a learned penalty on the scores that grows
// with the logarithm of the distance, no rotation) or a state space per head with an input-dependent step (a short causal
// convolution, a matrix state that decays and takes outer products, a gated group norm).  The feed-forward is dense and gated
// (relu), a mixture of small experts chosen by a router with a bias (softmax over the chosen, capped gate), or absent.  A layer
// may use another layer's weights with a cache or state of its own.  The head is a matrix of its own.
//
// config.json: {"architecture": "Viresun", "vocab", "width", "norm": {"eps"}, "layers": [{"type": "attention", "mixer": {"heads",
// "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "q_temp": {"coef", "every"}}, "mlp": ..} | {"type": "mamba2", "mixer":
// {"heads", "vdim", "state", "groups", "conv", "norm_groups"}, "mlp": ..}, each optionally with "weights_of": j], "mlp": {"kind":
// "dense", "ff"} | {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}} | null}.
// Tensors: embed, embed.norm, head, final.norm, and per layer with weights of its own l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*.
#pragma once

#include "arch.h"

namespace liyab {

struct ViresunConfig final : public ArchitectureConfig {
    struct Layer {
        bool state_space = false;
        int64_t weights_of = -1;          // the layer whose tensors this one uses (resolved to a layer with tensors of its own); -1: its own
        // attention
        int64_t heads = 0, kv_heads = 0, dim = 0, vdim = 0, window = 0, temp_every = 0;
        double scale = 1.0, temp_coef = 0.0;
        // state space (heads and vdim as above)
        int64_t n_state = 0, groups = 1, taps = 1, norm_groups = 1;
        // feed-forward: ff > 0 dense; experts > 0 routed; neither: none
        int64_t ff = 0, experts = 0, top = 0, expert_ff = 0;
        double limit = 0.0;
    };
    // Constants that the design fixes.
    static constexpr double kSinusoidBase = 10000.0;
    static constexpr double kExpertGateAlpha = 1.702;

    int64_t vocab = 0, width = 0;
    double norm_eps = 1e-6;
    int64_t max_positions = int64_t{1} << 17;        // the design has no limit of its own; the engine's tables need one
    std::vector<Layer> layers;
    Json raw;

    static std::unique_ptr<ViresunConfig> parse(const Json& raw);
    Json to_json() const override { return raw; }
    ModelSpec model_spec() const override;
    CheckpointMap checkpoint_map() const override;
    std::vector<std::string> ignored_tensors() const override;

private:
    // The place of config layer i among the layers that have tensors of their own (the model spec lists only those).
    std::vector<int> spec_index() const;
};

}  // namespace liyab
