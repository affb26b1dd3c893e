#include "viresun.h"

#include <cmath>

#include "config_keys.h"

namespace liyab {

std::unique_ptr<ViresunConfig> ViresunConfig::parse(const Json& raw) {
    auto c = std::make_unique<ViresunConfig>();
    c->raw = raw;
    c->vocab = int_in(raw, "vocab", "", 1);
    c->width = int_in(raw, "width", "", 1);
    c->norm_eps = number_in(object_in(raw, "norm", ""), "eps", "norm.");
    if (c->norm_eps < 0) throw invalid_model("invalid norm.eps {} in config.json", c->norm_eps);
    if (optional_in(raw, "max_positions") != nullptr) c->max_positions = int_in(raw, "max_positions", "", 1);
    const Json* layers = raw.find("layers");
    if (layers == nullptr || !layers->is_array() || layers->size() == 0) throw invalid_model("missing or invalid layers in config.json (need a list of layers)");
    const int64_t L = static_cast<int64_t>(layers->size());
    for (int64_t i = 0; i < L; ++i) {
        const Json& lj = (*layers)[static_cast<size_t>(i)];
        const std::string where = std::format("layers[{}].", i);
        if (!lj.is_object()) throw invalid_model("invalid {} in config.json (need an object)", where);
        Layer l;
        if (optional_in(lj, "weights_of") != nullptr) {
            l.weights_of = int_in(lj, "weights_of", where, 0, L - 1);
            if (l.weights_of == i) throw invalid_model("invalid {}weights_of in config.json: layer {} names itself", where, i);
        }
        const std::string type = lj.get_string("type", "");
        const Json& m = object_in(lj, "mixer", where);
        const std::string mw = where + "mixer.";
        l.heads = int_in(m, "heads", mw, 1, 65535);
        if (type == "attention") {
            l.kv_heads = m.contains("kv_heads") ? int_in(m, "kv_heads", mw, 1, l.heads) : l.heads;
            if (l.heads % l.kv_heads != 0) throw invalid_model("invalid {}kv_heads in config.json: {} heads do not split over {}", mw, l.heads, l.kv_heads);
            l.dim = int_in(m, "dim", mw, 1);
            l.vdim = m.contains("vdim") ? int_in(m, "vdim", mw, 1) : l.dim;
            l.scale = m.contains("scale") ? number_in(m, "scale", mw) : 1.0 / std::sqrt(static_cast<double>(l.dim));
            if (const Json* mask = optional_in(m, "mask")) l.window = int_in(*mask, "size", mw + "mask.", 1);
            if (const Json* t = optional_in(m, "q_temp")) {
                l.temp_coef = number_in(*t, "coef", mw + "q_temp.");
                l.temp_every = int_in(*t, "every", mw + "q_temp.", 1);
            }
        } else if (type == "mamba2") {
            l.state_space = true;
            l.vdim = int_in(m, "vdim", mw, 1);
            l.n_state = int_in(m, "state", mw, 1);
            l.groups = m.contains("groups") ? int_in(m, "groups", mw, 1, l.heads) : 1;
            if (l.heads % l.groups != 0) throw invalid_model("invalid {}groups in config.json: {} heads do not split over {}", mw, l.heads, l.groups);
            l.taps = m.contains("conv") ? int_in(m, "conv", mw, 1, 64) : 1;
            l.norm_groups = m.contains("norm_groups") ? int_in(m, "norm_groups", mw, 1) : 1;
            if ((l.heads * l.vdim) % l.norm_groups != 0)
                throw invalid_model("invalid {}norm_groups in config.json: {} values do not split into {} equal parts", mw, l.heads * l.vdim, l.norm_groups);
        } else {
            throw unsupported("{}type '{}' is not supported; supported: attention, mamba2", where, type);
        }
        if (const Json* mlp = optional_in(lj, "mlp")) {
            const std::string kind = mlp->get_string("kind", ""), fw = where + "mlp.";
            if (kind == "dense") {
                l.ff = int_in(*mlp, "ff", fw, 1);
            } else if (kind == "moe") {
                const Json& router = object_in(*mlp, "router", fw);
                l.experts = int_in(router, "experts", fw + "router.", 1, 4096);
                l.top = int_in(router, "top", fw + "router.", 1, l.experts);
                const Json& expert = object_in(*mlp, "expert", fw);
                l.expert_ff = int_in(expert, "ff", fw + "expert.", 1);
                l.limit = number_in(expert, "limit", fw + "expert.");
                if (!(l.limit > 0)) throw invalid_model("invalid {}expert.limit in config.json (need a positive number)", fw);
            } else {
                throw unsupported("{}kind '{}' is not supported; supported: dense, moe", fw, kind);
            }
        }
        c->layers.push_back(std::move(l));
    }
    // Every `weights_of` is resolved to a layer with tensors of its own.
    for (int64_t i = 0; i < L; ++i) {
        int64_t j = c->layers[static_cast<size_t>(i)].weights_of, hops = 0;
        while (j >= 0 && c->layers[static_cast<size_t>(j)].weights_of >= 0) {
            j = c->layers[static_cast<size_t>(j)].weights_of;
            if (++hops > L) throw invalid_model("invalid layers[{}].weights_of in config.json: the layers' weights_of run in a circle", i);
        }
        if (j >= 0) {
            Layer resolved = c->layers[static_cast<size_t>(j)];
            resolved.weights_of = j;
            c->layers[static_cast<size_t>(i)] = std::move(resolved);
        }
    }
    return c;
}

std::vector<int> ViresunConfig::spec_index() const {
    std::vector<int> at(layers.size(), -1);
    int n = 0;
    for (size_t i = 0; i < layers.size(); ++i)
        if (layers[i].weights_of < 0) at[i] = n++;
    for (size_t i = 0; i < layers.size(); ++i)
        if (layers[i].weights_of >= 0) at[i] = at[static_cast<size_t>(layers[i].weights_of)];
    return at;
}

ModelSpec ViresunConfig::model_spec() const {
    ModelSpec m;
    m.architecture = "viresun";
    m.embedding = {vocab, width, 1.0};
    m.position = {"sinusoid", Json::object().set("size", width).set("base", kSinusoidBase).set("norm", true).set("eps", norm_eps).set("max_positions", max_positions)};
    const PartSpec norm{"rms_norm", Json::object().set("size", width).set("groups", 1).set("eps", norm_eps)};
    for (const Layer& c : layers) {
        if (c.weights_of >= 0) continue;
        LayerSpec l;
        l.arrangement = "pre_norm";
        l.slots.push_back({"mixer_norm", Role::Norm, norm});
        if (c.state_space) {
            l.slots.push_back({"mixer", Role::Mixer,
                               {"state_space", Json::object().set("hidden", width).set("n_head", c.heads).set("vdim", c.vdim).set("n_state", c.n_state)
                                                   .set("groups", c.groups).set("taps", c.taps).set("norm_groups", c.norm_groups).set("eps", norm_eps)}});
        } else {
            l.slots.push_back({"mixer", Role::Mixer,
                               {"gated_attention", Json::object().set("hidden", width).set("n_head", c.heads).set("n_kv_head", c.kv_heads).set("dim", c.dim)
                                                       .set("vdim", c.vdim).set("scale", c.scale).set("window", c.window).set("qk_norm", true).set("qk_gain", false)
                                                       .set("bias", false).set("gate", "none").set("eps", norm_eps).set("q_temp_coef", c.temp_coef)
                                                       .set("q_temp_every", c.temp_every).set("distance_bias", true)}});
        }
        if (c.ff > 0 || c.experts > 0) {
            l.slots.push_back({"ff_norm", Role::Norm, norm});
            if (c.ff > 0)
                l.slots.push_back({"feed_forward", Role::FeedForward, {"gated", Json::object().set("hidden", width).set("inner", c.ff).set("activation", "relu")}});
            else
                l.slots.push_back({"feed_forward", Role::FeedForward,
                                   {"routed", Json::object().set("hidden", width).set("experts", c.experts).set("top", c.top).set("inner", c.expert_ff)
                                                  .set("activation", "capped").set("gate_alpha", kExpertGateAlpha).set("gate_limit", c.limit).set("score", "softmax")
                                                  .set("renormalise", true).set("weight_on", "output").set("router_bias", true).set("shared_inner", 0)}});
        }
        m.layers.push_back(std::move(l));
    }
    // Every layer of the configuration is a run with a cache unit or state of its own; one that uses another's weights names that layer.
    const std::vector<int> at = spec_index();
    for (size_t i = 0; i < layers.size(); ++i) m.run_order.push_back({at[i], static_cast<int>(i), -1});
    m.final_norm = norm;
    m.head = {vocab, width, false, false, 1.0, 0.0};
    m.max_positions = max_positions;
    return m;
}

CheckpointMap ViresunConfig::checkpoint_map() const {
    using K = ParamKind;
    CheckpointMap m;
    const double w_std = 1.0 / std::sqrt(static_cast<double>(width));
    m.push_back({"embedding.weight", CheckpointTensor::one("embed", {vocab, width}, K::Table, "none", 0.0, 1.0)});
    m.push_back({"position.norm.weight", CheckpointTensor::repeated("embed.norm", width, K::Vector, 1.0, 0.1)});
    m.push_back({"head.weight", CheckpointTensor::one("head", {vocab, width}, K::Matrix, "none", 0.0, w_std)});
    m.push_back({"final_norm.weight", CheckpointTensor::repeated("final.norm", width, K::Vector, 1.0, 0.1)});
    const std::vector<int> at = spec_index();
    for (size_t i = 0; i < layers.size(); ++i) {
        const Layer& c = layers[i];
        if (c.weights_of >= 0) continue;
        const std::string p = std::format("layers.{}.", at[i]), f = std::format("l{}.", i);
        m.push_back({p + "mixer_norm.weight", CheckpointTensor::repeated(f + "norm1", width, K::Vector, 1.0, 0.1)});
        if (c.state_space) {
            const int64_t inner = c.heads * c.vdim, channels = inner + 2 * c.groups * c.n_state;
            m.push_back({p + "mixer.proj.weight", CheckpointTensor::one(f + "mix.in", {inner + channels + c.heads, width}, K::Matrix, "none", 0.0, w_std)});
            m.push_back({p + "mixer.conv.weight", CheckpointTensor::one(f + "mix.conv", {channels, c.taps}, K::Vector, "none", 0.0, 1.0 / std::sqrt(static_cast<double>(c.taps)))});
            m.push_back({p + "mixer.conv.bias", CheckpointTensor::one(f + "mix.conv.b", {channels}, K::Vector, "none", 0.0, 0.1)});
            m.push_back({p + "mixer.dt_bias", CheckpointTensor::one(f + "mix.dt_bias", {c.heads}, K::Vector, "none", -2.0, 0.7)});
            m.push_back({p + "mixer.a_log", CheckpointTensor::one(f + "mix.A_log", {c.heads}, K::Vector, "none", -1.0, 0.7)});
            m.push_back({p + "mixer.skip", CheckpointTensor::one(f + "mix.D", {c.heads}, K::Vector, "none", 1.0, 0.1)});
            m.push_back({p + "mixer.norm.weight", CheckpointTensor::one(f + "mix.norm", {inner}, K::Vector, "none", 1.0, 0.1)});
            m.push_back({p + "mixer.out.weight", CheckpointTensor::one(f + "mix.o", {width, inner}, K::Matrix, "none", 0.0, 1.0 / std::sqrt(static_cast<double>(inner)))});
        } else {
            const int64_t QD = c.heads * c.dim, KD = c.kv_heads * c.dim, VD = c.kv_heads * c.vdim, OD = c.heads * c.vdim;
            m.push_back({p + "mixer.proj.weight", joined({{f + "mix.q", {QD, width}}, {f + "mix.k", {KD, width}}, {f + "mix.v", {VD, width}}}, K::Matrix, w_std)});
            // r1 around one, r2 a small positive number: 1 + r2 d stays positive.
            m.push_back({p + "mixer.distance", joined({{f + "mix.r1", {c.heads}}, {f + "mix.r2", {c.heads}}}, K::Vector, 0.02, 0.25)});
            m.push_back({p + "mixer.out.weight", CheckpointTensor::one(f + "mix.o", {width, OD}, K::Matrix, "none", 0.0, 1.0 / std::sqrt(static_cast<double>(OD)))});
        }
        if (c.ff > 0 || c.experts > 0) m.push_back({p + "ff_norm.weight", CheckpointTensor::repeated(f + "norm2", width, K::Vector, 1.0, 0.1)});
        if (c.ff > 0) {
            m.push_back({p + "feed_forward.gate_up.weight", joined({{f + "mlp.gate", {c.ff, width}}, {f + "mlp.up", {c.ff, width}}}, K::Matrix, w_std)});
            m.push_back({p + "feed_forward.down.weight", CheckpointTensor::one(f + "mlp.down", {width, c.ff}, K::Matrix, "none", 0.0, 1.0 / std::sqrt(static_cast<double>(c.ff)))});
        } else if (c.experts > 0) {
            m.push_back({p + "feed_forward.router.weight", CheckpointTensor::one(f + "mlp.router", {c.experts, width}, K::Matrix, "none", 0.0, w_std)});
            m.push_back({p + "feed_forward.router.bias", CheckpointTensor::one(f + "mlp.router.b", {c.experts}, K::Vector, "none", 0.0, 0.5)});
            std::vector<CheckpointSource> gate_up, down;
            for (int64_t e = 0; e < c.experts; ++e) {
                const std::string ef = std::format("{}mlp.e{}.", f, e);
                gate_up.push_back({ef + "gate", {c.expert_ff, width}});
                gate_up.push_back({ef + "up", {c.expert_ff, width}});
                down.push_back({ef + "down", {width, c.expert_ff}});
            }
            m.push_back({p + "feed_forward.experts.gate_up.weight", joined(std::move(gate_up), K::Matrix, w_std)});
            m.push_back({p + "feed_forward.experts.down.weight", joined(std::move(down), K::Matrix, 1.0 / std::sqrt(static_cast<double>(c.expert_ff)))});
        }
    }
    return m;
}

// A block without a feed-forward may still carry the gain of the norm before it.
std::vector<std::string> ViresunConfig::ignored_tensors() const {
    std::vector<std::string> out;
    for (size_t i = 0; i < layers.size(); ++i)
        if (layers[i].weights_of < 0 && layers[i].ff == 0 && layers[i].experts == 0) out.push_back(std::format("l{}\\.norm2", i));
    return out;
}

void register_viresun() {
    register_architecture({"viresun", {"Viresun", "ViresunForCausalLM"}, [](const Json& raw) -> std::unique_ptr<ArchitectureConfig> {
                               return ViresunConfig::parse(raw);
                           }});
}

}  // namespace liyab
