#include "vosurax.h"

#include <cmath>

#include "config_keys.h"

namespace liyab {

std::unique_ptr<VosuraxConfig> VosuraxConfig::parse(const Json& raw) {
    auto c = std::make_unique<VosuraxConfig>();
    c->raw = raw;
    c->vocab = int_in(raw, "vocab", "", 1);
    c->width = int_in(raw, "width", "", 1);
    c->norm_eps = number_in(object_in(raw, "norm", ""), "eps", "norm.");
    if (c->norm_eps < 0) throw invalid_model("invalid norm.eps {} in config.json", c->norm_eps);
    if (optional_in(raw, "max_positions") != nullptr) c->max_positions = int_in(raw, "max_positions", "", 1);
    const Json* layers = raw.find("layers");
    if (layers == nullptr || !layers->is_array() || layers->size() == 0) throw invalid_model("missing or invalid layers in config.json (need a list of layers)");
    for (size_t i = 0; i < layers->size(); ++i) {
        const Json& lj = (*layers)[i];
        const std::string where = std::format("layers[{}].", i);
        if (!lj.is_object()) throw invalid_model("invalid {} in config.json (need an object)", where);
        const std::string type = lj.get_string("type", "");
        const Json& m = object_in(lj, "mixer", where);
        const std::string mw = where + "mixer.";
        Layer l;
        auto memory = [&](const Json& j, const std::string& w) {
            l.heads = int_in(j, "heads", w, 1, 65535);
            l.dim = int_in(j, "dim", w, 1);
            l.vdim = int_in(j, "vdim", w, 1);
        };
        if (type == "retention") {
            memory(m, mw);
            const Json* decay = m.find("decay");
            if (decay == nullptr || !decay->is_array() || decay->size() != static_cast<size_t>(l.heads))
                throw invalid_model("missing or invalid {}decay in config.json (need one number a head)", mw);
            for (const auto& d : decay->items()) {
                if (!d.is_number() || !std::isfinite(d.as_number())) throw invalid_model("invalid {}decay in config.json", mw);
                l.decay.push_back(d.as_number());
            }
            if (const Json* rot = optional_in(m, "rot")) {
                l.rot_base = number_in(*rot, "base", mw + "rot.");
                l.rot_dims = int_in(*rot, "dims", mw + "rot.", 0, l.dim);
                if (l.rot_dims % 2 != 0 || l.rot_base <= 0) throw invalid_model("invalid {}rot in config.json: {} values to rotate, base {}", mw, l.rot_dims, l.rot_base);
            }
        } else if (type == "parallel") {
            l.parallel = true;
            const Json& left = object_in(m, "left", mw);
            const Json& right = object_in(m, "right", mw);
            const std::string lw = mw + "left.", rw = mw + "right.";
            l.a_heads = int_in(left, "heads", lw, 1, 65535);
            l.a_kv_heads = left.contains("kv_heads") ? int_in(left, "kv_heads", lw, 1, l.a_heads) : l.a_heads;
            if (l.a_heads % l.a_kv_heads != 0) throw invalid_model("invalid {}kv_heads in config.json: {} heads do not split over {}", lw, l.a_heads, l.a_kv_heads);
            l.a_dim = int_in(left, "dim", lw, 1);
            l.a_vdim = left.contains("vdim") ? int_in(left, "vdim", lw, 1) : l.a_dim;
            l.a_scale = number_in(left, "scale", lw);
            if (const Json* mask = optional_in(left, "mask")) l.a_chunk = int_in(*mask, "size", lw + "mask.", 1);
            memory(right, rw);
            l.gate_cap = number_in(right, "gate_cap", rw);
            if (!(l.gate_cap > 0)) throw invalid_model("invalid {}gate_cap in config.json (need a positive number)", rw);
        } else {
            throw unsupported("{}type '{}' is not supported; supported: retention, parallel", where, type);
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
                if (const Json* shared = optional_in(*mlp, "shared")) l.shared_ff = int_in(*shared, "ff", fw + "shared.", 1);
            } else {
                throw unsupported("{}kind '{}' is not supported; supported: dense, moe", fw, kind);
            }
        }
        c->layers.push_back(std::move(l));
    }
    if (const Json* loop = optional_in(raw, "loop")) {
        const int64_t L = static_cast<int64_t>(c->layers.size());
        c->loop_start = int_in(*loop, "start", "loop.", 0, L);
        c->loop_stop = int_in(*loop, "stop", "loop.", c->loop_start, L);
        c->loop_times = int_in(*loop, "times", "loop.", 1, 1024);
    }
    return c;
}

ModelSpec VosuraxConfig::model_spec() const {
    ModelSpec m;
    m.architecture = "vosurax";
    m.embedding = {vocab, width, 1.0};
    m.position = {"none", Json::object().set("max_positions", max_positions)};
    const PartSpec norm{"rms_norm", Json::object().set("size", width).set("groups", 1).set("eps", norm_eps).set("gain_offset", 1.0)};
    for (const Layer& c : layers) {
        LayerSpec l;
        l.arrangement = "pre_norm";
        l.slots.push_back({"mixer_norm", Role::Norm, norm});
        auto memory = [&](bool gated) {
            Json o = Json::object().set("hidden", width).set("n_head", c.heads).set("dim", c.dim).set("vdim", c.vdim).set("eps", norm_eps).set("head_norm", true);
            const double inv_root = 1.0 / std::sqrt(static_cast<double>(c.dim));
            if (gated) {
                o.set("recurrence", "gated").set("gate_cap", c.gate_cap).set("q_scale", inv_root).set("k_scale", 1.0).set("norm_gain", true).set("gate", "sigmoid");
            } else {
                o.set("recurrence", "fixed_decay").set("decay", Json::array_of(c.decay)).set("rot_dims", c.rot_dims).set("rot_base", c.rot_base)
                    .set("q_scale", 1.0).set("k_scale", inv_root).set("norm_gain", false).set("gate", "silu");
            }
            return PartSpec{"matrix_memory", o};
        };
        if (c.parallel) {
            const PartSpec left{"gated_attention", Json::object().set("hidden", width).set("n_head", c.a_heads).set("n_kv_head", c.a_kv_heads).set("dim", c.a_dim)
                                                       .set("vdim", c.a_vdim).set("scale", c.a_scale).set("chunk", c.a_chunk).set("qk_norm", true).set("bias", true)
                                                       .set("gate", "sigmoid").set("eps", norm_eps)};
            Json branches = Json::array();
            branches.push(Json::object().set("name", "left").set("part", left.to_json()));
            branches.push(Json::object().set("name", "right").set("part", memory(true).to_json()));
            l.slots.push_back({"mixer", Role::Mixer, {"branch_sum", Json::object().set("size", width).set("scale", 0.5).set("eps", norm_eps).set("branches", branches)}});
        } else {
            l.slots.push_back({"mixer", Role::Mixer, memory(false)});
        }
        if (c.ff > 0 || c.experts > 0) {
            l.slots.push_back({"ff_norm", Role::Norm, norm});
            if (c.ff > 0)
                l.slots.push_back({"feed_forward", Role::FeedForward,
                                   {"dense", Json::object().set("hidden", width).set("inner", c.ff).set("activation", "gelu_tanh").set("bias", false)}});
            else
                l.slots.push_back({"feed_forward", Role::FeedForward,
                                   {"routed", Json::object().set("hidden", width).set("experts", c.experts).set("top", c.top).set("inner", c.expert_ff)
                                                  .set("activation", "silu").set("score", "sigmoid").set("renormalise", false).set("weight_on", "input")
                                                  .set("shared_inner", c.shared_ff)}});
        }
        m.layers.push_back(std::move(l));
    }
    // The order of runs: the blocks before the stretch, the stretch `times` times, the rest.  Every run keeps a cache unit of its
    // own; the first run of every pass adds that pass's row of the offsets.
    const int L = static_cast<int>(layers.size());
    auto run = [&](int layer, int offset_row) { m.run_order.push_back({layer, static_cast<int>(m.run_order.size()), offset_row}); };
    if (loop_times > 0) {
        for (int i = 0; i < loop_start; ++i) run(i, -1);
        for (int t = 0; t < loop_times; ++t)
            for (int i = static_cast<int>(loop_start); i < loop_stop; ++i) run(i, i == loop_start ? t : -1);
        for (int i = static_cast<int>(loop_stop); i < L; ++i) run(i, -1);
        if (loop_stop > loop_start) m.pass_offsets = loop_times;
    } else {
        for (int i = 0; i < L; ++i) run(i, -1);
    }
    m.final_norm = norm;
    m.head = {vocab, width, false, false, 1.0, 0.0};
    m.max_positions = max_positions;
    return m;
}

CheckpointMap VosuraxConfig::checkpoint_map() const {
    using K = ParamKind;
    CheckpointMap m;
    const double w_std = 1.0 / std::sqrt(static_cast<double>(width));
    m.push_back({"embedding.weight", CheckpointTensor::one("embed", {vocab, width}, K::Table, "none", 0.0, 1.0)});
    m.push_back({"head.weight", CheckpointTensor::one("head", {vocab, width}, K::Matrix, "none", 0.0, w_std)});
    m.push_back({"final_norm.weight", CheckpointTensor::one("final.norm", {width}, K::Vector, "none", 0.0, 0.1)});
    if (loop_times > 0 && loop_stop > loop_start) m.push_back({"pass_offsets.weight", CheckpointTensor::one("loop.step", {loop_times, width}, K::Vector, "none", 0.0, 0.1)});
    for (size_t i = 0; i < layers.size(); ++i) {
        const Layer& c = layers[i];
        const std::string p = std::format("layers.{}.", i), f = std::format("l{}.", i);
        m.push_back({p + "mixer_norm.weight", CheckpointTensor::one(f + "norm1", {width}, K::Vector, "none", 0.0, 0.1)});
        auto memory = [&](const std::string& to, const std::string& from, bool gated) {
            const int64_t HD = c.heads * c.dim, HE = c.heads * c.vdim;
            std::vector<CheckpointSource> proj{{from + "q", {HD, width}}, {from + "k", {HD, width}}, {from + "v", {HE, width}}, {from + "g", {HE, width}}};
            if (gated) {
                proj.push_back({from + "i", {c.heads, width}});
                proj.push_back({from + "f", {c.heads, width}});
                m.push_back({to + "gate_bias", joined({{from + "i.b", {c.heads}}, {from + "f.b", {c.heads}}}, K::Vector, 1.0)});
                m.push_back({to + "norm.weight", CheckpointTensor::one(from + "norm", {HE}, K::Vector, "none", 1.0, 0.1)});
            }
            m.push_back({to + "proj.weight", joined(std::move(proj), K::Matrix, w_std)});
            m.push_back({to + "out.weight", CheckpointTensor::one(from + "o", {width, HE}, K::Matrix, "none", 0.0, 1.0 / std::sqrt(static_cast<double>(HE)))});
        };
        if (c.parallel) {
            const int64_t QD = c.a_heads * c.a_dim, KD = c.a_kv_heads * c.a_dim, VD = c.a_kv_heads * c.a_vdim, GD = c.a_heads * c.a_vdim;
            const std::string to = p + "mixer.left.", from = f + "mix.left.";
            m.push_back({to + "proj.weight", joined({{from + "q", {QD, width}}, {from + "k", {KD, width}}, {from + "v", {VD, width}}, {from + "g", {GD, width}}}, K::Matrix, w_std)});
            m.push_back({to + "qkv_bias", joined({{from + "q.b", {QD}}, {from + "k.b", {KD}}, {from + "v.b", {VD}}}, K::Vector, 0.1)});
            m.push_back({to + "q_norm.weight", CheckpointTensor::one(from + "q.norm", {c.a_dim}, K::Vector, "none", 1.0, 0.1)});
            m.push_back({to + "k_norm.weight", CheckpointTensor::one(from + "k.norm", {c.a_dim}, K::Vector, "none", 1.0, 0.1)});
            m.push_back({to + "out.weight", CheckpointTensor::one(from + "o", {width, GD}, K::Matrix, "none", 0.0, 1.0 / std::sqrt(static_cast<double>(GD)))});
            m.push_back({p + "mixer.left_out.weight", CheckpointTensor::one(f + "mix.left.out", {width}, K::Vector, "none", 1.0, 0.1)});
            memory(p + "mixer.right.", f + "mix.right.", true);
            m.push_back({p + "mixer.right_out.weight", CheckpointTensor::one(f + "mix.right.out", {width}, K::Vector, "none", 1.0, 0.1)});
        } else {
            memory(p + "mixer.", f + "mix.", false);
        }
        if (c.ff > 0 || c.experts > 0) m.push_back({p + "ff_norm.weight", CheckpointTensor::one(f + "norm2", {width}, K::Vector, "none", 0.0, 0.1)});
        if (c.ff > 0) {
            m.push_back({p + "feed_forward.up.weight", CheckpointTensor::one(f + "mlp.up", {c.ff, width}, K::Matrix, "none", 0.0, w_std)});
            m.push_back({p + "feed_forward.down.weight", CheckpointTensor::one(f + "mlp.down", {width, c.ff}, K::Matrix, "none", 0.0, 1.0 / std::sqrt(static_cast<double>(c.ff)))});
        } else if (c.experts > 0) {
            const double d_std = 1.0 / std::sqrt(static_cast<double>(c.expert_ff));
            m.push_back({p + "feed_forward.router.weight", CheckpointTensor::one(f + "mlp.router", {c.experts, width}, K::Matrix, "none", 0.0, w_std)});
            std::vector<CheckpointSource> gate_up, down;
            for (int64_t e = 0; e < c.experts; ++e) {
                const std::string ef = std::format("{}mlp.e{}.", f, e);
                gate_up.push_back({ef + "gate", {c.expert_ff, width}});
                gate_up.push_back({ef + "up", {c.expert_ff, width}});
                down.push_back({ef + "down", {width, c.expert_ff}});
            }
            m.push_back({p + "feed_forward.experts.gate_up.weight", joined(std::move(gate_up), K::Matrix, w_std)});
            m.push_back({p + "feed_forward.experts.down.weight", joined(std::move(down), K::Matrix, d_std)});
            if (c.shared_ff > 0) {
                m.push_back({p + "feed_forward.shared.gate_up.weight",
                             joined({{f + "mlp.shared.gate", {c.shared_ff, width}}, {f + "mlp.shared.up", {c.shared_ff, width}}}, K::Matrix, w_std)});
                m.push_back({p + "feed_forward.shared.down.weight",
                             CheckpointTensor::one(f + "mlp.shared.down", {width, c.shared_ff}, K::Matrix, "none", 0.0, 1.0 / std::sqrt(static_cast<double>(c.shared_ff)))});
            }
        }
    }
    return m;
}

// A block without a feed-forward may still carry the gain of the norm before it; a stretch that is empty its offsets.
std::vector<std::string> VosuraxConfig::ignored_tensors() const {
    std::vector<std::string> out;
    for (size_t i = 0; i < layers.size(); ++i)
        if (layers[i].ff == 0 && layers[i].experts == 0) out.push_back(std::format("l{}\\.norm2", i));
    if (!(loop_times > 0 && loop_stop > loop_start)) out.push_back("loop\\.step");
    return out;
}

void register_vosurax() {
    register_architecture({"vosurax", {"Vosurax", "VosuraxForCausalLM"}, [](const Json& raw) -> std::unique_ptr<ArchitectureConfig> {
                               return VosuraxConfig::parse(raw);
                           }});
}

}  // namespace liyab
