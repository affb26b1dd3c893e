// Parts of blocks whose mixers have gates, memories or several branches, and of feed-forwards with gates and routing:
// attention with normalised queries and keys, a chunked or sliding mask and an output gate; a matrix memory per head
// (fixed decay, or exponential gates with a running maximum); a mixer that sums several others, each over its own root
// mean square; the gated feed-forward; and the feed-forward of routed experts with an optional shared one.  Every
// size and constant is an option of the part's spec; none knows the model it is in.
#pragma once

#include <cmath>

#include "builtin_parts.h"

namespace liyab::builtin {

// A short list of floats that lives on the device from the first step on (which is never a recorded one).
class DeviceFloats {
public:
    std::vector<float> host;
    const float* get(cudaStream_t s) {
        if (dev_.data() == nullptr) {
            dev_ = DeviceBuffer(std::max<size_t>(host.size(), 1) * sizeof(float), true);
            if (!host.empty()) {
                LIYAB_CUDA(cudaMemcpyAsync(dev_.data(), host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice, s));
                LIYAB_CUDA(cudaStreamSynchronize(s));
            }
        }
        return static_cast<const float*>(dev_.data());
    }

private:
    DeviceBuffer dev_;
};

// A bias for some of a fused projection's columns: [zeros .. | part | .. zeros] on the device, put together at the first step.
class PartialBias {
public:
    void set(const float* part, int64_t at, int64_t count, int64_t total) { part_ = part; at_ = at; count_ = count; total_ = total; }
    const float* get(cudaStream_t s) {
        if (part_ == nullptr) return nullptr;
        if (joined_.data() == nullptr) {
            joined_ = DeviceBuffer(static_cast<size_t>(total_) * sizeof(float), true);
            LIYAB_CUDA(cudaMemcpyAsync(static_cast<float*>(joined_.data()) + at_, part_, static_cast<size_t>(count_) * sizeof(float), cudaMemcpyDeviceToDevice, s));
            LIYAB_CUDA(cudaStreamSynchronize(s));
        }
        return static_cast<const float*>(joined_.data());
    }

private:
    const float* part_ = nullptr;
    int64_t at_ = 0, count_ = 0, total_ = 0;
    DeviceBuffer joined_;
};

inline std::vector<float> rotation_frequencies(int dims, double base) {
    std::vector<float> f;
    for (int i = 0; i < dims / 2; ++i) f.push_back(static_cast<float>(std::pow(base, -2.0 * i / dims)));
    return f;
}

// ---- attention with normalised queries and keys, a mask and an output gate --------------------------------
// One projection makes [q (n_head x dim) | k (n_kv_head x dim) | v (n_kv_head x vdim) | g (n_head x vdim)] in 32-bit, with a
// bias on q, k and v where the part has one.  With `qk_norm` every query and key head is divided by its root mean square
// and multiplied by a gain of `dim` values shared by the heads.  score = (q . k) * scale over the keys that the mask
// lets through: `window` w (the w latest) or `chunk` c (the earlier keys of the query's own chunk of c positions, chunks
// counted from position 0 of the sequence), softmax, values; the heads are multiplied by gate(g) (`gate`: sigmoid, silu
// or none) before the output projection.  No rotation: positions act through the mask and, where the part has them, through
// two more options.  `q_temp_every` e > 0 with `q_temp_coef` c: the queries of position p are multiplied by
// 1 + c ln(floor((p + 1) / e) + 1) after their norm.  `distance_bias`: every head has two learned numbers (the parameter
// `distance`: r1 for all heads, then r2) and the score of the key d positions back loses r1 ln(1 + r2 d).  With `qk_gain` false
// the norm of queries and keys has no gain.  dim and vdim may differ: the cache and the attention kernels work on heads of
// `padded` values, the rest zeros, so the existing kernels serve.
// Further options.  `qk_norm_over` "projection": the norm runs over all of q (and all of k) at once instead of head by head, with gains of
// n_head x dim and n_kv_head x dim values.  `rot_dims` r > 0: after the norm the first r values of every query and key head are rotated, value i
// with value i + r/2, by the angle position * rot_base^(-2i/r).  `sink`: a learned number a head (the parameter `sink`) whose exponential
// joins the divisor of the head's softmax; it has no key and no value and is not scaled.  `value_blend`: "source" leaves the step's values
// (as projected) where later layers of the model find them; "blend" replaces its own by (1 - b) v + b v_source with the learned number `blend`
// before they are cached.  The source is the model's first layer that says so; all such layers have n_kv_head x vdim values alike.

class GatedAttention final : public Mixer {
public:
    GatedAttention(const PartSpec& s, const Params& p, const Runtime& rt) {
        hidden = need_int(s, "hidden");
        H = static_cast<int>(need_int(s, "n_head"));
        G = static_cast<int>(s.options.get_int("n_kv_head", H));
        D = static_cast<int>(need_int(s, "dim"));
        E = static_cast<int>(s.options.get_int("vdim", D));
        if (G <= 0 || H % G != 0) throw invalid_model("gated_attention: n_head {} is not a multiple of n_kv_head {}", H, G);
        shape.n_head = H;
        shape.n_kv_head = G;
        shape.head_dim = padded_head(std::max(D, E), rt.dtype);
        shape.scale = static_cast<float>(s.options.get_number("scale", 1.0 / std::sqrt(static_cast<double>(D))));
        shape.window = static_cast<int>(s.options.get_int("window", 0));
        shape.chunk = static_cast<int>(s.options.get_int("chunk", 0));
        if (shape.window < 0 || shape.chunk < 0 || (shape.window > 0 && shape.chunk > 0))
            throw invalid_model("gated_attention: a window ({}) or a chunk ({}), not both, and neither negative", shape.window, shape.chunk);
        qk_norm = s.options.get_bool("qk_norm", false);
        eps = static_cast<float>(s.options.get_number("eps", 1e-6));
        temp_coef = static_cast<float>(s.options.get_number("q_temp_coef", 0.0));
        temp_every = static_cast<int>(s.options.get_int("q_temp_every", 0));
        if (temp_every < 0) throw invalid_model("gated_attention: q_temp_every {} is negative", temp_every);
        const std::string gate_name = s.options.get_string("gate", "none");
        gate = gate_name == "none" ? -1 : kernels::gate_from_name(gate_name);
        proj = Linear(p, "proj.", "gated_attention.proj");
        out = Linear(p, "out.", "gated_attention.out");
        if (const Tensor* b = p.find("qkv_bias")) bias.set(static_cast<const float*>(b->data), 0, qkv_cols(), proj.weight.dim(0));
        if (qk_norm && s.options.get_bool("qk_gain", true)) {
            q_gain = f32_or_null(&p.at("q_norm.weight"));
            k_gain = f32_or_null(&p.at("k_norm.weight"));
        }
        if (s.options.get_bool("distance_bias", false)) shape.distance = f32_or_null(&p.at("distance"));
        const std::string over = s.options.get_string("qk_norm_over", "head");
        if (over != "head" && over != "projection") throw unsupported("gated_attention: qk_norm_over '{}' is not supported; supported: head, projection", over);
        norm_projection = qk_norm && over == "projection";
        rot_dims = static_cast<int>(s.options.get_int("rot_dims", 0));
        if (rot_dims < 0 || rot_dims > D || rot_dims % 2 != 0) throw invalid_model("gated_attention: {} of {} values cannot be rotated in pairs", rot_dims, D);
        freq.host = rotation_frequencies(rot_dims, s.options.get_number("rot_base", 10000.0));
        if (s.options.get_bool("sink", false)) shape.sink = f32_or_null(&p.at("sink"));
        const std::string vb = s.options.get_string("value_blend", "none");
        if (vb != "none" && vb != "source" && vb != "blend") throw unsupported("gated_attention: value_blend '{}' is not supported; supported: none, source, blend", vb);
        blend_source = vb == "source";
        if (vb == "blend") blend = f32_or_null(&p.at("blend"));
        rotary_store = norm_projection || rot_dims > 0 || vb != "none";
        if (rotary_store && temp_every > 0) throw unsupported("gated_attention: a temperature on the queries goes with neither rotation, norm over the projection nor blended values");
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t hidden = need_int(s, "hidden"), H = need_int(s, "n_head"), G = s.options.get_int("n_kv_head", H), D = need_int(s, "dim");
        const int64_t E = s.options.get_int("vdim", D);
        const bool gated = s.options.get_string("gate", "none") != "none";
        std::vector<ParamDecl> out;
        Linear::declare(out, "proj.", H * D + G * D + G * E + (gated ? H * E : 0), hidden, false);
        if (s.options.get_bool("bias", false)) out.push_back({"qkv_bias", {H * D + G * D + G * E}, ParamKind::Vector});
        if (s.options.get_bool("qk_norm", false) && s.options.get_bool("qk_gain", true)) {
            const bool whole = s.options.get_string("qk_norm_over", "head") == "projection";
            out.push_back({"q_norm.weight", {whole ? H * D : D}, ParamKind::Vector});
            out.push_back({"k_norm.weight", {whole ? G * D : D}, ParamKind::Vector});
        }
        if (s.options.get_bool("sink", false)) out.push_back({"sink", {H}, ParamKind::Vector});
        if (s.options.get_string("value_blend", "none") == "blend") out.push_back({"blend", {1}, ParamKind::Vector});
        if (s.options.get_bool("distance_bias", false)) out.push_back({"distance", {2 * H}, ParamKind::Vector});
        Linear::declare(out, "out.", hidden, H * E, false);
        return out;
    }
    // The head size the cache and the kernels work on: in bfloat16 the next size every tensor-core kernel takes, else a multiple of four.
    static int padded_head(int n, DType dt) {
        if (n > 256) throw unsupported("gated_attention: heads of {} values are more than the attention kernels take (256)", n);
        if (dt == DType::BF16) {
            int p = 16;
            while (p < n) p *= 2;
            return p;
        }
        return (n + 3) / 4 * 4;
    }
    bool capturable() const override { return true; }
    std::optional<KvNeed> kv_need() const override { return KvNeed{G, shape.head_dim, shape.chunk > 0 ? shape.chunk : shape.window}; }

    void forward(StepContext& ctx, const Rows& h, const Rows& x, CacheUnit unit) override { run(ctx, &h, nullptr, nullptr, x, &x, unit); }
    void forward_into(StepContext& ctx, const Rows& h, const Rows& y, CacheUnit unit) override { run(ctx, &h, nullptr, nullptr, y, nullptr, unit); }
    // A step of up to 16 tokens in bfloat16: the projection normalises the rows itself.
    bool normalises(const StepContext& ctx, const Rows& x_in) const override { return kernels::gemm_rows_normed_supports(ctx.runtime, x_in, proj.weight, ctx.n_tokens); }
    bool forward_from(StepContext& ctx, const Rows& x_in, const NormRecipe& norm, const Rows& x, CacheUnit unit) override {
        if (!normalises(ctx, x_in)) return false;
        run(ctx, nullptr, &x_in, &norm, x, &x, unit);
        return true;
    }
    void forward_from_into(StepContext& ctx, const Rows& x_in, const NormRecipe& norm, const Rows& y, CacheUnit unit) override {
        run(ctx, nullptr, &x_in, &norm, y, nullptr, unit);
    }

    kernels::AttentionShape shape;
    int64_t hidden = 0;
    int H = 0, G = 0, D = 0, E = 0, gate = -1;
    bool qk_norm = false, norm_projection = false, blend_source = false, rotary_store = false;
    int rot_dims = 0;
    const float* blend = nullptr;
    float eps = 1e-6f, temp_coef = 0.0f;
    int temp_every = 0;
    Linear proj, out;
    const float* q_gain = nullptr;
    const float* k_gain = nullptr;

private:
    int64_t qkv_cols() const { return static_cast<int64_t>(H) * D + static_cast<int64_t>(G) * (D + E); }
    // Either the normalised rows h, or the stream's rows x_in with the recipe of the norm before the mixer.
    void run(StepContext& ctx, const Rows* h, const Rows* x_in, const NormRecipe* norm, const Rows& y, const Rows* residual, CacheUnit unit) {
        const int T = ctx.n_tokens, P = shape.head_dim;
        const DType dt = ctx.runtime.dtype;
        Workspace& ws = *ctx.workspace;
        cudaStream_t s = ctx.stream();
        const Rows pr = ws.get("gated_attention.proj", T, proj.weight.dim(0), DType::F32);
        if (h != nullptr) kernels::linear(ctx.runtime, &ws, *h, proj.weight, bias.get(s), pr, T, kernels::kNone, nullptr);
        else kernels::gemm_rows_normed(s, *x_in, norm->gain, norm->offset, norm->eps, proj.weight, bias.get(s), pr, T, kernels::kNone, nullptr, nullptr, norm->rms,
                                       norm->gain_offset);
        const GroupView* view = nullptr;
        void* cache = ctx.kv(unit.read, &view);
        kernels::AttentionShape a = shape;
        a.page_size = view->group->page_size;
        const Rows q = ws.get("gated_attention.q", T, static_cast<int64_t>(H) * P, dt);
        const kernels::QkvColumns cols{0, H * D, H * D + G * D, H, G, D, E, P, a.page_size};
        if (rotary_store) {
            // The values that layers blend with travel from the source layer to the others in a buffer of the step.
            Rows shared;
            if (blend_source || blend != nullptr) shared = ws.get("gated_attention.value_source", T, static_cast<int64_t>(G) * E, DType::F32);
            kernels::qkv_rotary_store(s, pr, cols, q_gain, k_gain, q, unit.write ? cache : nullptr, view->slot_mapping, T, !qk_norm ? 0 : norm_projection ? 2 : 1, eps,
                                      ctx.positions, rot_dims > 0 ? freq.get(s) : nullptr, rot_dims, blend != nullptr ? &shared : nullptr,
                                      blend_source ? &shared : nullptr, blend);
        } else {
            kernels::qk_norm_store(s, pr, cols, q_gain, k_gain, q, unit.write ? cache : nullptr, view->slot_mapping, T, qk_norm, eps, ctx.positions, temp_coef,
                                   temp_every);
        }
        ctx.tap("attention.q", q);
        const Rows att = ws.get("gated_attention.att", T, static_cast<int64_t>(H) * P, dt);
        const int reach = shape.chunk > 0 ? shape.chunk : shape.window;
        attend(ctx, q, cache, *view, att, a, reach > 0 ? std::min(reach, ctx.max_positions) : ctx.max_positions);
        // Heads without a gate whose values fill the padded size are what the output projection reads, as they are.
        const bool as_they_are = gate < 0 && P == E;
        const Rows heads = as_they_are ? att : ws.get("gated_attention.heads", T, static_cast<int64_t>(H) * E, dt);
        if (!as_they_are) {
            const Rows g = gate >= 0 ? pr.columns(qkv_cols(), static_cast<int64_t>(H) * E) : Rows{};
            kernels::head_gate(s, att, P, g, nullptr, heads, T, H, E, false, std::max(gate, 0), eps);
        }
        ctx.tap("attention", heads);
        kernels::linear(ctx.runtime, &ws, heads, out.weight, nullptr, y, T, kernels::kNone, residual);
    }
    PartialBias bias;
    DeviceFloats freq;
};

// ---- a matrix memory per head ----------------------------------------------------------------------------------
// S_t = keep_t S_{t-1} + take_t k_t v_t^T, o_t = S_t^T q_t, per head, carried from token to token in the request's state slot
// (32-bit).  `recurrence` "fixed_decay": keep = decay[head], take = 1 (retention).  `recurrence` "gated": two more numbers a head come
// from the projection (with a bias), i = cap tanh(zi / cap) and f = logsigmoid(cap tanh(zf / cap)); with a running maximum m
// that starts at 0, m_t = max(f + m_{t-1}, i), keep = exp(f + m_{t-1} - m_t), take = exp(i - m_t); n_t follows the same
// recurrence with k alone and o_t is divided by max(|n_t . q_t|, exp(-m_t)) + 1e-6.  Queries and keys may be rotated (the first
// rot_dims values of a head, value j with value j + rot_dims/2, angle position * rot_base^(-2j/rot_dims)) and scaled (q_scale,
// k_scale, after the rotation).  Every head's o is divided by its root mean square (`head_norm`), times a gain over all heads'
// values where the part has one (`norm_gain`), times gate(g), then the output projection.
// One projection makes [q | k | v | g | zi | zf] in 32-bit.
// `qkv_activation` (silu, sigmoid, gelu_tanh, relu; default none) acts on q, k and v as they leave the projection (inside the memory's kernels, on the rows as they arrive; before them, as a pass of its own, in steps with long portions).  `norm_over` "all": instead of
// every head over its own root mean square, all heads' values together over one (with the gain `norm.weight` where `norm_gain` is set).

class MatrixMemory final : public Mixer {
public:
    MatrixMemory(const PartSpec& s, const Params& p) {
        hidden = need_int(s, "hidden");
        m.n_head = static_cast<int>(need_int(s, "n_head"));
        m.dim = static_cast<int>(need_int(s, "dim"));
        m.vdim = static_cast<int>(need_int(s, "vdim"));
        m.value_tile = kernels::memory_value_tile(m.dim, m.vdim);
        const std::string kind = s.options.get_string("recurrence", "fixed_decay");
        if (kind != "fixed_decay" && kind != "gated") throw unsupported("matrix_memory: recurrence '{}' is not supported; supported: fixed_decay, gated", kind);
        gated = kind == "gated";
        if (gated) {
            m.cap = static_cast<float>(s.options.get_number("gate_cap", 0.0));
            if (!(m.cap > 0.0f)) throw invalid_model("matrix_memory: gate_cap must be positive");
        } else {
            const Json* d = s.options.find("decay");
            if (d == nullptr || !d->is_array() || d->size() != static_cast<size_t>(m.n_head)) throw invalid_model("matrix_memory: 'decay' must list one number a head");
            for (const auto& v : d->items()) decay.host.push_back(static_cast<float>(v.as_number()));
        }
        m.rot_dims = static_cast<int>(s.options.get_int("rot_dims", 0));
        if (m.rot_dims < 0 || m.rot_dims > m.dim || m.rot_dims % 2 != 0) throw invalid_model("matrix_memory: {} of {} values cannot be rotated in pairs", m.rot_dims, m.dim);
        freq.host = rotation_frequencies(m.rot_dims, s.options.get_number("rot_base", 10000.0));
        m.q_scale = static_cast<float>(s.options.get_number("q_scale", 1.0));
        m.k_scale = static_cast<float>(s.options.get_number("k_scale", 1.0));
        head_norm = s.options.get_bool("head_norm", true);
        const std::string over = s.options.get_string("norm_over", "head");
        if (over != "head" && over != "all") throw unsupported("matrix_memory: norm_over '{}' is not supported; supported: head, all", over);
        norm_all = over == "all";
        const std::string qkv_act = s.options.get_string("qkv_activation", "none");
        if (qkv_act != "none") {
            m.qkv_act = kernels::gate_from_name(qkv_act);
            if (m.qkv_act > kernels::kRelu) throw unsupported("matrix_memory: qkv_activation '{}' is not supported; supported: none, sigmoid, silu, gelu_tanh, relu", qkv_act);
        }
        eps = static_cast<float>(s.options.get_number("eps", 1e-6));
        gate = kernels::gate_from_name(s.options.get_string("gate", "silu"));
        proj = Linear(p, "proj.", "matrix_memory.proj");
        out = Linear(p, "out.", "matrix_memory.out");
        if (gated) bias.set(static_cast<const float*>(p.at("gate_bias").data), gate_at(), 2 * m.n_head, proj.weight.dim(0));
        if (s.options.get_bool("norm_gain", false)) norm_gain = f32_or_null(&p.at("norm.weight"));
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t hidden = need_int(s, "hidden"), H = need_int(s, "n_head"), D = need_int(s, "dim"), E = need_int(s, "vdim");
        const bool gated = s.options.get_string("recurrence", "fixed_decay") == "gated";
        std::vector<ParamDecl> out;
        Linear::declare(out, "proj.", 2 * H * D + 2 * H * E + (gated ? 2 * H : 0), hidden, false);
        if (gated) out.push_back({"gate_bias", {2 * H}, ParamKind::Vector});
        if (s.options.get_bool("norm_gain", false)) out.push_back({"norm.weight", {H * E}, ParamKind::Vector});
        Linear::declare(out, "out.", hidden, H * E, false);
        return out;
    }
    bool capturable() const override { return true; }
    std::optional<StateNeed> state_need() const override { return StateNeed{{m.slot_floats()}, DType::F32}; }
    void forward(StepContext& ctx, const Rows& h, const Rows& x, CacheUnit unit) override { run(ctx, &h, nullptr, nullptr, x, &x, unit); }
    void forward_into(StepContext& ctx, const Rows& h, const Rows& y, CacheUnit unit) override { run(ctx, &h, nullptr, nullptr, y, nullptr, unit); }
    bool normalises(const StepContext& ctx, const Rows& x_in) const override { return kernels::gemm_rows_normed_supports(ctx.runtime, x_in, proj.weight, ctx.n_tokens); }
    bool forward_from(StepContext& ctx, const Rows& x_in, const NormRecipe& norm, const Rows& x, CacheUnit unit) override {
        if (!normalises(ctx, x_in)) return false;
        run(ctx, nullptr, &x_in, &norm, x, &x, unit);
        return true;
    }
    void forward_from_into(StepContext& ctx, const Rows& x_in, const NormRecipe& norm, const Rows& y, CacheUnit unit) override {
        run(ctx, nullptr, &x_in, &norm, y, nullptr, unit);
    }

    // Portions of this many rows or more go through the kernel that works in pieces.
    static constexpr int kChunkedFrom = 16;
    // Steps whose longest portion has this many rows or more take the three-launch form (a block per piece).
    static constexpr int kPiecesFrom = 128;
    kernels::MemoryShape m;
    int64_t hidden = 0;
    bool gated = false, head_norm = true, norm_all = false;
    int gate = kernels::kSilu;
    float eps = 1e-6f;
    Linear proj, out;
    const float* norm_gain = nullptr;

private:
    int64_t gate_at() const { return 2 * static_cast<int64_t>(m.n_head) * (m.dim + m.vdim); }
    void run(StepContext& ctx, const Rows* h, const Rows* x_in, const NormRecipe* norm, const Rows& y, const Rows* residual, CacheUnit unit) {
        if (!unit.write) throw invalid_model("matrix_memory: a memory is carried by the run that owns it; the run order lets another read it");
        const int T = ctx.n_tokens, H = m.n_head, D = m.dim, E = m.vdim;
        Workspace& ws = *ctx.workspace;
        cudaStream_t s = ctx.stream();
        const Rows pr = ws.get("matrix_memory.proj", T, proj.weight.dim(0), DType::F32);
        if (h != nullptr) kernels::linear(ctx.runtime, &ws, *h, proj.weight, bias.get(s), pr, T, kernels::kNone, nullptr);
        else kernels::gemm_rows_normed(s, *x_in, norm->gain, norm->offset, norm->eps, proj.weight, bias.get(s), pr, T, kernels::kNone, nullptr, nullptr, norm->rms,
                                       norm->gain_offset);
        const int64_t HD = static_cast<int64_t>(H) * D, HE = static_cast<int64_t>(H) * E;
        const Rows q = pr.columns(0, HD), k = pr.columns(HD, HD), v = pr.columns(2 * HD, HE), g = pr.columns(2 * HD + HE, HE);
        const Rows zi = pr.columns(gate_at(), H), zf = pr.columns(gate_at() + H, H);
        const Rows o = ws.get("matrix_memory.o", T, HE, DType::F32);
        const float* decays = gated ? nullptr : decay.get(s);
        const float* freqs = m.rot_dims > 0 ? freq.get(s) : nullptr;
        float* state = static_cast<float*>(ctx.state(unit.read));
        if (ctx.max_q_len >= kPiecesFrom) {
            // Long portions: every piece of 32 rows a block of its own, so that a few requests fill the GPU.  Its launches read a row
            // several times (a value tile each, sums and outputs apart), so an activation on q, k and v is cheaper as one pass before them
            // than inside them (measured: 2 x 1,024 rows, six layers: 3.23 against 3.29 ms a prefill); shorter steps save the launch instead.
            kernels::MemoryShape plain = m;
            if (m.qkv_act >= 0) {
                kernels::activate_columns(s, pr.columns(0, 2 * HD + HE), T, m.qkv_act);
                plain.qkv_act = -1;
            }
            float* scratch = static_cast<float*>(ws.flat("matrix_memory.pieces", kernels::memory_pieces_floats(T, ctx.n_seq, m), DType::F32));
            kernels::matrix_memory_pieces(s, q, k, v, gated ? &zi : nullptr, gated ? &zf : nullptr, decays, freqs, ctx.positions, ctx.q_start, ctx.state_slots, state,
                                          o, T, ctx.n_seq, plain, scratch);
        } else {
            kernels::matrix_memory(s, q, k, v, gated ? &zi : nullptr, gated ? &zf : nullptr, decays, freqs, ctx.positions, ctx.q_start, ctx.state_slots, state, o,
                                   ctx.n_seq, m, ctx.max_q_len >= kChunkedFrom);
        }
        ctx.tap("memory", o);
        const Rows heads = ws.get("matrix_memory.heads", T, HE, ctx.runtime.dtype);
        if (norm_all) kernels::row_norm_gate(s, o, g, norm_gain, heads, T, gate, eps);
        else kernels::head_gate(s, o, E, g, norm_gain, heads, T, H, E, head_norm, gate, eps);
        kernels::linear(ctx.runtime, &ws, heads, out.weight, nullptr, y, T, kernels::kNone, residual);
    }
    DeviceFloats decay, freq;
    PartialBias bias;
};

// ---- several mixers side by side ----------------------------------------------------------------------------------
// x += scale * sum_b rms(mixer_b(h)) * gain_b: every branch reads the same input, its output is divided by its root mean square
// over the width and multiplied by its gain.  Options: `branches` [{"name", "part": {kind, options}}], `scale`, `eps`, `size`.
// At most one branch may keep keys and values and at most one a state: both live under the block's one cache unit.

class BranchSum final : public Mixer {
public:
    BranchSum(const PartSpec& s, const Params& p, const Runtime& rt) : size(need_int(s, "size")), scale(static_cast<float>(s.options.get_number("scale", 1.0))),
                                                                       eps(static_cast<float>(s.options.get_number("eps", 1e-6))) {
        for (const auto& [name, part] : branch_specs(s)) {
            names.push_back(name);
            branches.push_back(mixers().get(part.kind).build(part, p.sub(name + "."), rt));
            gains.push_back(f32_or_null(&p.at(name + "_out.weight")));
        }
        int kv = 0, st = 0;
        for (const auto& b : branches) {
            kv += b->kv_need().has_value();
            st += b->state_need().has_value();
        }
        if (kv > 1 || st > 1) throw unsupported("branch_sum: at most one branch with keys and values and one with a state");
    }
    static std::vector<std::pair<std::string, PartSpec>> branch_specs(const PartSpec& s) {
        const Json* list = s.options.find("branches");
        if (list == nullptr || !list->is_array() || list->size() == 0 || list->size() > 4) throw invalid_model("branch_sum: 'branches' must list one to four mixers");
        std::vector<std::pair<std::string, PartSpec>> out;
        for (const auto& b : list->items()) out.push_back({b.at("name").as_string(), PartSpec::from_json(b.at("part"), "branch_sum.branches")});
        return out;
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        std::vector<ParamDecl> out;
        for (const auto& [name, part] : branch_specs(s)) {
            for (const auto& d : mixers().get(part.kind).parameters(part)) out.push_back({name + "." + d.name, d.shape, d.kind});
            out.push_back({name + "_out.weight", {need_int(s, "size")}, ParamKind::Vector});
        }
        return out;
    }
    bool capturable() const override {
        for (const auto& b : branches)
            if (!b->capturable()) return false;
        return true;
    }
    std::optional<KvNeed> kv_need() const override {
        for (const auto& b : branches)
            if (const auto n = b->kv_need()) return n;
        return std::nullopt;
    }
    std::optional<StateNeed> state_need() const override {
        for (const auto& b : branches)
            if (const auto n = b->state_need()) return n;
        return std::nullopt;
    }
    void forward(StepContext& ctx, const Rows& h, const Rows& x, CacheUnit unit) override { run(ctx, &h, nullptr, nullptr, x, unit); }
    // Where every branch can normalise the rows itself for this step, the norm before the mixer is not launched.
    bool normalises(const StepContext& ctx, const Rows& x_in) const override {
        for (const auto& b : branches)
            if (!b->normalises(ctx, x_in)) return false;
        return true;
    }
    bool forward_from(StepContext& ctx, const Rows& x_in, const NormRecipe& norm, const Rows& x, CacheUnit unit) override {
        if (!normalises(ctx, x_in)) return false;
        run(ctx, nullptr, &x_in, &norm, x, unit);
        return true;
    }
    int64_t size;
    float scale, eps;
    std::vector<std::string> names;
    std::vector<std::shared_ptr<Mixer>> branches;
    std::vector<const float*> gains;

private:
    void run(StepContext& ctx, const Rows* h, const Rows* x_in, const NormRecipe* norm, const Rows& x, CacheUnit unit) {
        std::vector<Rows> ys;
        for (size_t i = 0; i < branches.size(); ++i) {
            ys.push_back(ctx.workspace->get(std::format("branch_sum.{}", i), ctx.n_tokens, size, DType::F32));
            if (h != nullptr) branches[i]->forward_into(ctx, *h, ys.back(), unit);
            else branches[i]->forward_from_into(ctx, *x_in, *norm, ys.back(), unit);
            ctx.tap("branch." + names[i], ys.back());
        }
        kernels::rms_sum_add(ctx.stream(), x, ys, gains, ctx.n_tokens, scale, eps);
    }
};

// ---- the gated feed-forward: down(gate(W_gate h) * (W_up h)) ------------------------------------------------------
// One product makes [gate | up] in 32-bit, the gate's activation and the product of the halves are one pass, the second
// product adds into the stream.  `activation`: silu, sigmoid, gelu_tanh, relu, or capped with its two numbers `gate_alpha` and
// `gate_limit`: g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(alpha g') (u' + 1).

class GatedFeedForward final : public FeedForward {
public:
    GatedFeedForward(const PartSpec& s, const Params& p)
        : inner(need_int(s, "inner")), gate(kernels::gate_from_name(s.options.get_string("activation", "silu"))),
          alpha(static_cast<float>(s.options.get_number("gate_alpha", 1.0))), limit(static_cast<float>(s.options.get_number("gate_limit", 0.0))) {
        gate_up = Linear(p, "gate_up.", "gated.gate_up");
        down = Linear(p, "down.", "gated.down");
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t hidden = need_int(s, "hidden"), inner = need_int(s, "inner");
        std::vector<ParamDecl> out;
        Linear::declare(out, "gate_up.", 2 * inner, hidden, false);
        Linear::declare(out, "down.", hidden, inner, false);
        return out;
    }
    bool capturable() const override { return true; }
    void forward(StepContext& ctx, const Rows& h, const Rows& x) override {
        const int T = ctx.n_tokens;
        const Rows gu = ctx.workspace->get("gated.gate_up", T, 2 * inner, DType::F32);
        gate_up.forward(ctx, h, gu, T);
        finish(ctx, gu, x);
    }
    // As the dense feed-forward's: the [gate | up] product of a few tokens normalises the rows inside its kernel.
    bool forward_from(StepContext& ctx, const Rows& x_in, const NormRecipe& norm, const Rows& x) override {
        const int T = ctx.n_tokens;
        if (gate_up.bias != nullptr || !kernels::gemm_rows_normed_supports(ctx.runtime, x_in, gate_up.weight, T)) return false;
        const Rows gu = ctx.workspace->get("gated.gate_up", T, 2 * inner, DType::F32);
        kernels::gemm_rows_normed(ctx.stream(), x_in, norm.gain, norm.offset, norm.eps, gate_up.weight, nullptr, gu, T, kernels::kNone, nullptr, nullptr,
                                  norm.rms, norm.gain_offset);
        finish(ctx, gu, x);
        return true;
    }
    void forward_into(StepContext& ctx, const Rows& h, const Rows& y) override {
        const int T = ctx.n_tokens;
        const Rows gu = ctx.workspace->get("gated.gate_up", T, 2 * inner, DType::F32);
        gate_up.forward(ctx, h, gu, T);
        finish(ctx, gu, y, false);
    }
    int64_t inner;
    int gate;
    float alpha, limit;
    Linear gate_up, down;

private:
    void finish(StepContext& ctx, const Rows& gu, const Rows& x, bool add = true) {
        const int T = ctx.n_tokens;
        const Rows mid = ctx.workspace->get("gated.inner", T, inner, ctx.runtime.dtype);
        kernels::gated_act(ctx.stream(), gu, mid, T, gate, alpha, limit);
        down.forward(ctx, mid, x, T, kernels::kNone, add ? &x : nullptr);
    }
};

// ---- routed experts --------------------------------------------------------------------------------------------------
// z = router h in 32-bit; score = sigmoid(z) (`score` "sigmoid") or the softmax over the experts ("softmax"); every row goes to
// its `top` experts with the largest scores, weights = their scores (divided by their sum with `renormalise`; a softmax that is
// renormalised is the softmax over the chosen experts' z alone).  With `router_bias` a learned number an expert is added to z
// before the choice.  `weight_on` "input": the weight multiplies the expert's input, x += sum_e expert_e(w_e h); "output": its
// result, x += sum_e w_e expert_e(h).  expert = down(gate(W_gate a) * (W_up a)) without biases, `activation` as the gated
// feed-forward's (the capped form with `gate_alpha`, `gate_limit`).  With
// `shared_inner` > 0 a gated feed-forward of that size runs for every row and is added.  The experts' matrices are stacked:
// gate_up [experts x 2 inner, hidden] (per expert its gate rows, then its up rows) and down [experts x hidden, inner].
// `route` "table": no router; the parameter `table` (int32 [vocab, top], a row's entries all different) names the experts of every token id,
// each with the weight 1 / top.

class RoutedExperts final : public FeedForward {
public:
    RoutedExperts(const PartSpec& s, const Params& p)
        : hidden(need_int(s, "hidden")), inner(need_int(s, "inner")), experts(static_cast<int>(need_int(s, "experts"))), top(static_cast<int>(need_int(s, "top"))),
          gate(kernels::gate_from_name(s.options.get_string("activation", "silu"))), renormalise(s.options.get_bool("renormalise", false)),
          alpha(static_cast<float>(s.options.get_number("gate_alpha", 1.0))), limit(static_cast<float>(s.options.get_number("gate_limit", 0.0))) {
        if (top > experts) throw invalid_model("routed: top {} of {} experts", top, experts);
        const std::string score = s.options.get_string("score", "sigmoid");
        if (score != "sigmoid" && score != "softmax") throw unsupported("routed: score '{}' is not supported; supported: sigmoid, softmax", score);
        softmax = score == "softmax";
        const std::string weight_on = s.options.get_string("weight_on", "input");
        if (weight_on != "input" && weight_on != "output") throw unsupported("routed: weight_on '{}' is not supported; supported: input, output", weight_on);
        weight_on_output = weight_on == "output";
        const std::string route = s.options.get_string("route", "scores");
        if (route != "scores" && route != "table") throw unsupported("routed: route '{}' is not supported; supported: scores, table", route);
        by_table = route == "table";
        if (by_table) table = p.at("table");
        else router = p.at("router.weight");
        if (!by_table && s.options.get_bool("router_bias", false)) router_bias = f32_or_null(&p.at("router.bias"));
        gate_up = p.at("experts.gate_up.weight");
        down = p.at("experts.down.weight");
        if (s.options.get_int("shared_inner", 0) > 0) shared = std::make_unique<GatedFeedForward>(shared_spec(s), p.sub("shared."));
    }
    static PartSpec shared_spec(const PartSpec& s) {
        return {"gated", Json::object().set("hidden", need_int(s, "hidden")).set("inner", s.options.get_int("shared_inner", 0))
                             .set("activation", s.options.get_string("shared_activation", s.options.get_string("activation", "silu")))};
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t hidden = need_int(s, "hidden"), inner = need_int(s, "inner"), E = need_int(s, "experts");
        std::vector<ParamDecl> out;
        if (s.options.get_string("route", "scores") == "table") {
            out.push_back({"table", {need_int(s, "vocab"), need_int(s, "top")}, ParamKind::Index});
        } else {
            out.push_back({"router.weight", {E, hidden}, ParamKind::Matrix});
            if (s.options.get_bool("router_bias", false)) out.push_back({"router.bias", {E}, ParamKind::Vector});
        }
        for (ParamDecl d : std::vector<ParamDecl>{{"experts.gate_up.weight", {E * 2 * inner, hidden}, ParamKind::Matrix},
                                   {"experts.down.weight", {E * hidden, inner}, ParamKind::Matrix}})
            out.push_back(std::move(d));
        if (s.options.get_int("shared_inner", 0) > 0)
            for (const auto& d : GatedFeedForward::parameters(shared_spec(s))) out.push_back({"shared." + d.name, d.shape, d.kind});
        return out;
    }
    bool capturable() const override { return true; }
    void forward(StepContext& ctx, const Rows& h, const Rows& x) override { run(ctx, h, x, false); }
    // The rows' sums are written instead of added, so nothing has to be cleared first (a shared expert then adds to them).
    void forward_into(StepContext& ctx, const Rows& h, const Rows& y) override { run(ctx, h, y, true); }
    void run(StepContext& ctx, const Rows& h, const Rows& x, bool overwrite) {
        const int T = ctx.n_tokens, pairs = T * top;
        Workspace& ws = *ctx.workspace;
        cudaStream_t s = ctx.stream();
        // Per-row buffers hold `top` entries a row, so that they grow with the step's tokens as every other buffer does.
        int32_t* ids = static_cast<int32_t*>(ws.get("routed.ids", T, top, DType::I32).data);
        float* weights = ws.get("routed.weights", T, top, DType::F32).f32();
        int32_t* place = static_cast<int32_t*>(ws.get("routed.place", T, top, DType::I32).data);
        int32_t* pair_at = static_cast<int32_t*>(ws.get("routed.pair_at", T, top, DType::I32).data);
        int32_t* offsets = static_cast<int32_t*>(ws.flat("routed.offsets", experts + 1, DType::I32));
        if (by_table && pairs <= kLookupInPlan) {       // the look-up rides in the plan's launch (one block: worth it for steps of few rows)
            kernels::expert_plan_table(s, ctx.tokens, table, ids, weights, T, top, experts, offsets, place, pair_at);
        } else if (by_table) {
            kernels::router_table(s, ctx.tokens, table, ids, weights, T, top, experts);
            kernels::expert_plan(s, ids, pairs, experts, offsets, place, pair_at);
        } else {
            kernels::router_topk(s, h, router, ids, weights, T, top, softmax, renormalise, router_bias);
            kernels::expert_plan(s, ids, pairs, experts, offsets, place, pair_at);
        }
        Rows mid = ws.get("routed.inner", T, static_cast<int64_t>(top) * inner, ctx.runtime.dtype);
        mid = Rows{mid.data, mid.dtype, static_cast<int64_t>(pairs), inner, inner};
        Rows y = ws.get("routed.out", T, static_cast<int64_t>(top) * hidden, DType::F32);
        y = Rows{y.data, y.dtype, static_cast<int64_t>(pairs), hidden, hidden};
        kernels::expert_product(s, true, h, gate_up, experts, offsets, pair_at, weight_on_output ? nullptr : weights, mid, pairs, static_cast<int>(inner),
                                static_cast<int>(hidden), top, gate, alpha, limit);
        kernels::expert_product(s, false, mid, down, experts, offsets, pair_at, weights, y, pairs, static_cast<int>(hidden), static_cast<int>(inner), top, gate);
        kernels::expert_combine(s, x, y, place, T, top, weight_on_output ? weights : nullptr, overwrite);
        ctx.tap("routed", x);
        if (shared) shared->forward(ctx, h, x);
    }
    // Up to this many (row, choice) pairs the table's look-up is part of the plan's launch (measured: 2.7 + 2.6 us as two launches against 3.9 us
    // for 16 pairs; 16.6 + 3.5 us against 25.3 us for 4,096).
    static constexpr int kLookupInPlan = 1024;
    int64_t hidden, inner;
    int experts, top, gate;
    bool renormalise, softmax = false, weight_on_output = false, by_table = false;
    float alpha, limit;
    const float* router_bias = nullptr;
    Tensor router, table, gate_up, down;
    std::unique_ptr<GatedFeedForward> shared;
};

}  // namespace liyab::builtin
