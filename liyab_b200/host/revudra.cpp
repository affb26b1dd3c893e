#include "revudra.h"

#include <cmath>

#include "config_keys.h"

namespace liyab {

std::unique_ptr<RevudraConfig> RevudraConfig::parse(const Json& raw) {
    auto c = std::make_unique<RevudraConfig>();
    c->raw = raw;
    c->vocab = int_in(raw, "vocab", "", 1);
    c->width = int_in(raw, "width", "", 1);
    c->norm_eps = number_in(object_in(raw, "norm", ""), "eps", "norm.");
    if (c->norm_eps < 0) throw invalid_model("invalid norm.eps {} in config.json", c->norm_eps);
    if (optional_in(raw, "residual_mult") != nullptr) c->residual_mult = number_in(raw, "residual_mult", "");
    if (const Json* e = optional_in(raw, "embedding")) c->embedding_scale = number_in(*e, "scale", "embedding.");
    if (optional_in(raw, "logit_scale") != nullptr) c->logit_scale = number_in(raw, "logit_scale", "");
    if (optional_in(raw, "max_positions") != nullptr) c->max_positions = int_in(raw, "max_positions", "", 1);
    const Json* layers = raw.find("layers");
    if (layers == nullptr || !layers->is_array() || layers->size() == 0) throw invalid_model("missing or invalid layers in config.json (need a list of layers)");
    int64_t blended = -1;       // n_kv_head x vdim of the layers that blend values
    for (size_t i = 0; i < layers->size(); ++i) {
        const Json& lj = (*layers)[i];
        const std::string where = std::format("layers[{}].", i);
        if (!lj.is_object()) throw invalid_model("invalid {} in config.json (need an object)", where);
        Layer l;
        const std::string type = lj.get_string("type", "");
        const Json& m = object_in(lj, "mixer", where);
        const std::string mw = where + "mixer.";
        l.heads = int_in(m, "heads", mw, 1, 65535);
        l.dim = int_in(m, "dim", mw, 1);
        l.vdim = m.contains("vdim") ? int_in(m, "vdim", mw, 1) : l.dim;
        auto rotation = [&](int64_t most) {
            if (const Json* r = optional_in(m, "rot")) {
                l.rot_dims = int_in(*r, "dims", mw + "rot.", 0, most);
                if (l.rot_dims % 2 != 0) throw invalid_model("invalid {}rot.dims in config.json: {} values cannot be rotated in pairs", mw, l.rot_dims);
                l.rot_base = number_in(*r, "base", mw + "rot.");
                if (!(l.rot_base > 0)) throw invalid_model("invalid {}rot.base in config.json (need a positive number)", mw);
            }
        };
        if (type == "attention") {
            l.mixer = Mixer::Attention;
            l.kv_heads = m.contains("kv_heads") ? int_in(m, "kv_heads", mw, 1, l.heads) : l.heads;
            if (l.heads % l.kv_heads != 0) throw invalid_model("invalid {}kv_heads in config.json: {} heads do not split over {}", mw, l.heads, l.kv_heads);
            l.scale = m.contains("scale") ? number_in(m, "scale", mw) : 1.0 / std::sqrt(static_cast<double>(l.dim));
            if (const Json* mask = optional_in(m, "mask")) l.window = int_in(*mask, "size", mw + "mask.", 1);
            rotation(l.dim);
            if (const Json* v = optional_in(m, "v_mix")) {
                if (!v->is_bool()) throw invalid_model("invalid {}v_mix in config.json (need true or false)", mw);
                l.v_mix = v->as_bool();
            }
            if (l.v_mix) {
                if (blended >= 0 && blended != l.kv_heads * l.vdim)
                    throw invalid_model("invalid {}v_mix in config.json: this layer has {} values a token, the first such layer {}", mw, l.kv_heads * l.vdim, blended);
                blended = l.kv_heads * l.vdim;
            }
        } else if (type == "lightning") {
            l.mixer = Mixer::Lightning;
            const Json* d = m.find("decay");
            if (d == nullptr || !d->is_array() || d->size() != static_cast<size_t>(l.heads))
                throw invalid_model("missing or invalid {}decay in config.json (need one number a head)", mw);
            for (const auto& v : d->items()) {
                if (!v.is_number() || !std::isfinite(v.as_number())) throw invalid_model("invalid {}decay in config.json (need finite numbers)", mw);
                l.decay.push_back(v.as_number());
            }
        } else if (type == "latent_attention") {
            l.mixer = Mixer::Latent;
            l.rot_dim = int_in(m, "rot_dim", mw, 0);
            l.kv_rank = int_in(m, "kv_rank", mw, 1);
            l.q_rank = int_in(m, "q_rank", mw, 1);
            l.scale = m.contains("scale") ? number_in(m, "scale", mw) : 1.0 / std::sqrt(static_cast<double>(l.dim + l.rot_dim));
            l.rot_dims = l.rot_dim - l.rot_dim % 2;          // the whole rotated part unless `rot.dims` says less
            rotation(l.rot_dim);
        } else {
            throw unsupported("{}type '{}' is not supported; supported: attention, lightning, latent_attention", where, type);
        }
        if (const Json* mlp = optional_in(lj, "mlp")) {
            const std::string kind = mlp->get_string("kind", ""), fw = where + "mlp.";
            if (kind == "dense") {
                l.ff = int_in(*mlp, "ff", fw, 1);
            } else if (kind == "moe") {
                const Json& router = object_in(*mlp, "router", fw);
                l.experts = int_in(router, "experts", fw + "router.", 1, 4096);
                l.top = int_in(router, "top", fw + "router.", 1, l.experts);
                l.expert_ff = int_in(object_in(*mlp, "expert", fw), "ff", fw + "expert.", 1);
            } else {
                throw unsupported("{}kind '{}' is not supported; supported: dense, moe", fw, kind);
            }
        }
        c->layers.push_back(std::move(l));
    }
    return c;
}

int RevudraConfig::value_source() const {
    int first = -1, count = 0;
    for (size_t i = 0; i < layers.size(); ++i)
        if (layers[i].mixer == Mixer::Attention && layers[i].v_mix) {
            if (first < 0) first = static_cast<int>(i);
            ++count;
        }
    return count > 1 ? first : -1;       // a lone such layer has nothing to give its values to
}

ModelSpec RevudraConfig::model_spec() const {
    ModelSpec m;
    m.architecture = "revudra";
    m.embedding = {vocab, width, embedding_scale};
    m.position = {"none", Json::object().set("max_positions", max_positions)};
    const PartSpec norm{"rms_norm", Json::object().set("size", width).set("groups", 1).set("eps", norm_eps)};
    const int source = value_source();
    for (size_t i = 0; i < layers.size(); ++i) {
        const Layer& c = layers[i];
        LayerSpec l;
        l.arrangement = "sublayer_norm";
        l.options = Json::object().set("residual_scale", residual_mult);
        if (c.mixer == Mixer::Attention) {
            const bool blends = source >= 0 && c.v_mix;
            l.slots.push_back({"mixer", Role::Mixer,
                               {"gated_attention", Json::object().set("hidden", width).set("n_head", c.heads).set("n_kv_head", c.kv_heads).set("dim", c.dim)
                                                       .set("vdim", c.vdim).set("scale", c.scale).set("window", c.window).set("qk_norm", true)
                                                       .set("qk_norm_over", "projection").set("bias", false).set("gate", "sigmoid").set("eps", norm_eps)
                                                       .set("rot_dims", c.rot_dims).set("rot_base", c.rot_base).set("sink", true)
                                                       .set("value_blend", !blends ? "none" : static_cast<int>(i) == source ? "source" : "blend")}});
        } else if (c.mixer == Mixer::Lightning) {
            Json decay = Json::array();
            for (const double d : c.decay) decay.push(d);
            l.slots.push_back({"mixer", Role::Mixer,
                               {"matrix_memory", Json::object().set("hidden", width).set("n_head", c.heads).set("dim", c.dim).set("vdim", c.vdim)
                                                     .set("recurrence", "fixed_decay").set("decay", decay).set("rot_dims", 0).set("qkv_activation", "silu")
                                                     .set("head_norm", true).set("norm_over", "all").set("norm_gain", true).set("gate", "sigmoid").set("eps", norm_eps)}});
        } else {
            l.slots.push_back({"mixer", Role::Mixer,
                               {"latent_attention", Json::object().set("hidden", width).set("n_head", c.heads).set("dim", c.dim).set("rot_dim", c.rot_dim)
                                                        .set("rot_dims", c.rot_dims).set("rot_base", c.rot_base).set("rot_layout", "interleaved").set("vdim", c.vdim)
                                                        .set("kv_rank", c.kv_rank).set("q_rank", c.q_rank).set("window", 0).set("scale", c.scale).set("eps", norm_eps)
                                                        .set("own_latent", true).set("sink", true).set("head_gate", true)}});
        }
        l.slots.push_back({"mixer_norm", Role::Norm, norm});
        if (c.ff > 0 || c.experts > 0) {
            if (c.ff > 0)
                l.slots.push_back({"feed_forward", Role::FeedForward,
                                   {"dense", Json::object().set("hidden", width).set("inner", c.ff).set("activation", "relu2").set("bias", false)}});
            else
                l.slots.push_back({"feed_forward", Role::FeedForward,
                                   {"routed", Json::object().set("hidden", width).set("experts", c.experts).set("top", c.top).set("inner", c.expert_ff)
                                                  .set("activation", "silu").set("route", "table").set("vocab", vocab).set("weight_on", "output").set("shared_inner", 0)}});
            l.slots.push_back({"ff_norm", Role::Norm, norm});
        }
        m.layers.push_back(std::move(l));
        m.run_order.push_back({static_cast<int>(i), static_cast<int>(i), -1});
    }
    m.final_norm = norm;
    m.head = {vocab, width, false, false, logit_scale, 0.0};
    m.max_positions = max_positions;
    return m;
}

CheckpointMap RevudraConfig::checkpoint_map() const {
    using K = ParamKind;
    CheckpointMap m;
    const double w_std = 1.0 / std::sqrt(static_cast<double>(width));
    auto inv_sqrt = [](int64_t n) { return 1.0 / std::sqrt(static_cast<double>(n)); };
    m.push_back({"embedding.weight", CheckpointTensor::one("embed", {vocab, width}, K::Table, "none", 0.0, 1.0)});
    m.push_back({"head.weight", CheckpointTensor::one("head", {vocab, width}, K::Matrix, "none", 0.0, w_std)});
    m.push_back({"final_norm.weight", CheckpointTensor::one("final.norm", {width}, K::Vector, "none", 1.0, 0.1)});
    const int source = value_source();
    for (size_t i = 0; i < layers.size(); ++i) {
        const Layer& c = layers[i];
        const std::string p = std::format("layers.{}.", i), f = std::format("l{}.", i);
        m.push_back({p + "mixer_norm.weight", CheckpointTensor::one(f + "norm1", {width}, K::Vector, "none", 1.0, 0.1)});
        const int64_t OD = c.heads * c.vdim;
        if (c.mixer == Mixer::Attention) {
            const int64_t QD = c.heads * c.dim, KD = c.kv_heads * c.dim, VD = c.kv_heads * c.vdim;
            m.push_back({p + "mixer.proj.weight",
                         joined({{f + "mix.q", {QD, width}}, {f + "mix.k", {KD, width}}, {f + "mix.v", {VD, width}}, {f + "mix.g", {OD, width}}}, K::Matrix, w_std)});
            m.push_back({p + "mixer.q_norm.weight", CheckpointTensor::one(f + "mix.q.norm", {QD}, K::Vector, "none", 1.0, 0.1)});
            m.push_back({p + "mixer.k_norm.weight", CheckpointTensor::one(f + "mix.k.norm", {KD}, K::Vector, "none", 1.0, 0.1)});
            m.push_back({p + "mixer.sink", CheckpointTensor::one(f + "mix.sink", {c.heads}, K::Vector, "none", 0.0, 1.0)});
            if (source >= 0 && c.v_mix && static_cast<int>(i) != source) m.push_back({p + "mixer.blend", CheckpointTensor::repeated(f + "mix.vmix", 1, K::Vector, 0.5, 0.1)});
        } else if (c.mixer == Mixer::Lightning) {
            const int64_t QD = c.heads * c.dim;
            m.push_back({p + "mixer.proj.weight",
                         joined({{f + "mix.q", {QD, width}}, {f + "mix.k", {QD, width}}, {f + "mix.v", {OD, width}}, {f + "mix.g", {OD, width}}}, K::Matrix, w_std)});
            m.push_back({p + "mixer.norm.weight", CheckpointTensor::one(f + "mix.norm", {OD}, K::Vector, "none", 1.0, 0.1)});
        } else {
            const int64_t QD = c.heads * (c.dim + c.rot_dim), row = c.kv_rank + c.rot_dim;
            m.push_back({p + "mixer.proj.weight", joined({{f + "mix.dq", {c.q_rank, width}}, {f + "mix.dkv", {row, width}}, {f + "mix.g", {c.heads, width}}}, K::Matrix, w_std)});
            m.push_back({p + "mixer.q_norm.weight", CheckpointTensor::one(f + "mix.dq.norm", {c.q_rank}, K::Vector, "none", 1.0, 0.1)});
            m.push_back({p + "mixer.q_up.weight", CheckpointTensor::one(f + "mix.uq", {QD, c.q_rank}, K::Matrix, "none", 0.0, inv_sqrt(c.q_rank))});
            m.push_back({p + "mixer.latent_norm.weight", CheckpointTensor::one(f + "mix.dkv.norm", {c.kv_rank}, K::Vector, "none", 1.0, 0.1)});
            m.push_back({p + "mixer.uk.weight", CheckpointTensor::one(f + "mix.uk", {c.heads * c.dim, c.kv_rank}, K::Matrix, "none", 0.0, inv_sqrt(c.kv_rank))});
            m.push_back({p + "mixer.uv.weight", CheckpointTensor::one(f + "mix.uv", {OD, c.kv_rank}, K::Matrix, "none", 0.0, inv_sqrt(c.kv_rank))});
            m.push_back({p + "mixer.sink", CheckpointTensor::one(f + "mix.sink", {c.heads}, K::Vector, "none", 0.0, 1.0)});
        }
        m.push_back({p + "mixer.out.weight", CheckpointTensor::one(f + "mix.o", {width, OD}, K::Matrix, "none", 0.0, inv_sqrt(OD))});
        if (c.ff > 0 || c.experts > 0) m.push_back({p + "ff_norm.weight", CheckpointTensor::one(f + "norm2", {width}, K::Vector, "none", 1.0, 0.1)});
        if (c.ff > 0) {
            m.push_back({p + "feed_forward.up.weight", CheckpointTensor::one(f + "mlp.up", {c.ff, width}, K::Matrix, "none", 0.0, w_std)});
            m.push_back({p + "feed_forward.down.weight", CheckpointTensor::one(f + "mlp.down", {width, c.ff}, K::Matrix, "none", 0.0, inv_sqrt(c.ff))});
        } else if (c.experts > 0) {
            m.push_back({p + "feed_forward.table", CheckpointTensor::one(f + "mlp.table", {vocab, c.top}, K::Index, "none", 0.0, static_cast<double>(c.experts))});
            std::vector<CheckpointSource> gate_up, down;
            for (int64_t e = 0; e < c.experts; ++e) {
                const std::string ef = std::format("{}mlp.e{}.", f, e);
                gate_up.push_back({ef + "gate", {c.expert_ff, width}});
                gate_up.push_back({ef + "up", {c.expert_ff, width}});
                down.push_back({ef + "down", {width, c.expert_ff}});
            }
            m.push_back({p + "feed_forward.experts.gate_up.weight", joined(std::move(gate_up), K::Matrix, w_std)});
            m.push_back({p + "feed_forward.experts.down.weight", joined(std::move(down), K::Matrix, inv_sqrt(c.expert_ff))});
        }
    }
    return m;
}

// A block without a feed-forward may still carry the gain of the norm behind it, and a layer that gives its values to the others (or has
// none to blend with) the weight of a blend it does not make.
std::vector<std::string> RevudraConfig::ignored_tensors() const {
    std::vector<std::string> out;
    const int source = value_source();
    for (size_t i = 0; i < layers.size(); ++i) {
        const Layer& c = layers[i];
        if (c.ff == 0 && c.experts == 0) out.push_back(std::format("l{}\\.norm2", i));
        if (c.mixer == Mixer::Attention && !(source >= 0 && c.v_mix && static_cast<int>(i) != source)) out.push_back(std::format("l{}\\.mix\\.vmix", i));
    }
    return out;
}

void register_revudra() {
    register_architecture({"revudra", {"Revudra", "RevudraForCausalLM"}, [](const Json& raw) -> std::unique_ptr<ArchitectureConfig> {
                               return RevudraConfig::parse(raw);
                           }});
}

}  // namespace liyab
