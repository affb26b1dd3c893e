// Parts of blocks whose mixer and feed-forward read one normalised input side by side: the RMS norm in groups, the
// token shift before the mixer, attention over a cache of latent rows, the gated per-token side input, and the
// arrangement that puts them around the residual stream.  Every size and constant is an option of the part's spec;
// none knows the model it is in, and each can be used without the others.
#pragma once

#include <cmath>

#include "builtin_parts.h"

namespace liyab::builtin {

// ---- RMS norm in groups ------------------------------------------------------------------------------
// The row is cut into `groups` equal consecutive parts; every part is divided by sqrt(mean(part^2) + eps), and the
// whole row is multiplied by the gain.  groups = 1 is the plain RMS norm.  Statistics in 32-bit.  With the option
// `gain_offset` that number is added to every gain (1 for gains that are stored around zero).

class GroupedRmsNorm final : public Norm {
public:
    GroupedRmsNorm(const PartSpec& s, const Params& p)
        : size(need_int(s, "size")), groups(static_cast<int>(s.options.get_int("groups", 1))), eps(static_cast<float>(s.options.get_number("eps", 1e-6))),
          gain_offset(static_cast<float>(s.options.get_number("gain_offset", 0.0))) {
        if (groups < 1 || size % groups != 0) throw invalid_model("rms_norm: {} values do not split into {} equal groups", size, groups);
        weight = f32_or_null(&p.at("weight"));
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) { return {{"weight", {need_int(s, "size")}, ParamKind::Vector}}; }
    bool capturable() const override { return true; }
    void forward(StepContext& ctx, const Rows& x, const Rows& out, int n_rows, const int32_t* rows) override {
        kernels::rms_groups(ctx.stream(), x, rows, weight, out, n_rows, groups, eps, gain_offset);
    }
    // One group: the part after the norm may normalise the rows itself (a projection of a few tokens does).
    std::optional<NormRecipe> recipe() const override {
        if (groups != 1) return std::nullopt;
        return NormRecipe{weight, nullptr, eps, true, gain_offset};
    }
    int64_t size;
    int groups;
    float eps;
    float gain_offset;
    const float* weight = nullptr;
};

// ---- token shift ---------------------------------------------------------------------------------------
// m_t = h_t + (h_{t-1} - h_t) * w, element by element, with h_{t-1} the row before in the sequence as it came from
// the norm (zeros before a sequence's first row).  The state of a request is the last row it brought, in the compute
// type, so a row blends with the same numbers whether its neighbour came in this step or in an earlier one.

class LerpShift final : public Shift {
public:
    LerpShift(const PartSpec& s, const Params& p, const Runtime& rt) : size(need_int(s, "size")), dtype(rt.dtype) { weight = f32_or_null(&p.at("weight")); }
    static std::vector<ParamDecl> parameters(const PartSpec& s) { return {{"weight", {need_int(s, "size")}, ParamKind::Vector}}; }
    bool capturable() const override { return true; }
    StateNeed state_need() const override { return StateNeed{{size}, dtype}; }
    void forward(StepContext& ctx, const Rows& h, const Rows& m, void* state) override {
        kernels::token_shift(ctx.stream(), h, weight, m, state, layout(ctx));
    }
    bool forward_normed(StepContext& ctx, const Rows& x, Norm& norm, const Rows& h, const Rows& m, void* state) override {
        const auto* rms = dynamic_cast<const GroupedRmsNorm*>(&norm);
        if (rms == nullptr || rms->size != size || rms->gain_offset != 0.0f) return false;
        kernels::rms_shift(ctx.stream(), x, rms->weight, weight, h, m, state, layout(ctx), rms->groups, rms->eps);
        return true;
    }
    int64_t size;
    DType dtype;
    const float* weight = nullptr;

private:
    static kernels::ShiftLayout layout(const StepContext& ctx) {
        return {ctx.tok_seq, ctx.q_start, ctx.state_slots, ctx.n_tokens, ctx.n_seq, ctx.decode_only};
    }
};

// ---- attention over latent rows ---------------------------------------------------------------------
// Per position the cache keeps one row [c | r]: the latent c (kv_rank values, RMS-normed) from which every head's
// unrotated key (uk) and value (uv) are linear maps, and one rotated key part r (rot_dim values) shared by all heads.
// A head's query is [dim unrotated | rot_dim rotated].  The score of head h is
//     (q_h . (uk_h c_j) + q'_h . r_j) * scale = ((uk_h^T q_h) . c_j + q'_h . r_j) * scale,
// so the queries are widened once per step (uk_h^T q_h, kv_rank values a head) and attention runs on the cache rows
// as they are; the attended latents sum_j p_j c_j then pass through uv_h.  The rotation acts on the first `rot_dims`
// of the rot_dim values (value i pairs with i + rot_dims/2; angle = position * base^(-2i/rot_dims)).  `window` w > 0:
// position i sees j with 0 <= i - j < w.  With `own_latent` false the part has no down projection and reads the rows
// that another run of the model wrote (the run order names it); its window, heads and maps are its own.
// Further options.  `q_rank` r > 0: the queries come through a latent of their own, q = q_up (rms_norm(q_down h) * q_norm.weight); the down
// map is part of the one projection.  `rot_layout` "interleaved": the rotation pairs value 2i with 2i + 1 instead of i with i + rot_dims/2.
// `sink`: a learned number a head (the parameter `sink`) whose exponential joins the divisor of the head's softmax; no key, no value, not
// scaled.  `head_gate`: the projection also makes one number a head, and the head's result is multiplied by its sigmoid.
// The projection's rows: [queries or their latent | latent row (with own_latent) | gates (with head_gate)].

class LatentAttention final : public Mixer {
public:
    LatentAttention(const PartSpec& s, const Params& p) {
        hidden = need_int(s, "hidden");
        a.n_head = static_cast<int>(need_int(s, "n_head"));
        a.dim = static_cast<int>(need_int(s, "dim", 0));
        a.rot = static_cast<int>(need_int(s, "rot_dim", 0));
        a.rot_dims = static_cast<int>(s.options.get_int("rot_dims", a.rot));
        a.vdim = static_cast<int>(need_int(s, "vdim"));
        a.rank = static_cast<int>(need_int(s, "kv_rank"));
        a.window = static_cast<int>(s.options.get_int("window", 0));
        a.scale = static_cast<float>(s.options.get_number("scale", 1.0 / std::sqrt(static_cast<double>(a.dim + a.rot))));
        eps = static_cast<float>(s.options.get_number("eps", 1e-6));
        own_latent = s.options.get_bool("own_latent", true);
        q_rank = s.options.get_int("q_rank", 0);
        if (q_rank < 0) throw invalid_model("latent_attention: q_rank {} is negative", q_rank);
        const std::string layout = s.options.get_string("rot_layout", "half");
        if (layout != "half" && layout != "interleaved") throw unsupported("latent_attention: rot_layout '{}' is not supported; supported: half, interleaved", layout);
        a.interleaved = layout == "interleaved";
        head_gate = s.options.get_bool("head_gate", false);
        if (a.rot_dims < 0 || a.rot_dims > a.rot || a.rot_dims % 2 != 0)
            throw invalid_model("latent_attention: {} of {} rotated values cannot be rotated in pairs", a.rot_dims, a.rot);
        if (a.window < 0) throw invalid_model("latent_attention: window {} is negative", a.window);
        if (a.dim + a.rot <= 0) throw invalid_model("latent_attention: queries have no values");
        const double base = s.options.get_number("rot_base", 10000.0);
        for (int i = 0; i < a.rot_dims / 2; ++i) freq_host.push_back(static_cast<float>(std::pow(base, -2.0 * i / a.rot_dims)));
        q_cols = static_cast<int64_t>(a.n_head) * (a.dim + a.rot);
        proj = Linear(p, "proj.", "latent_attention.proj");
        out = Linear(p, "out.", "latent_attention.out");
        uk = p.at("uk.weight");
        uv = p.at("uv.weight");
        if (own_latent) latent_gain = f32_or_null(&p.at("latent_norm.weight"));
        if (q_rank > 0) {
            q_gain = f32_or_null(&p.at("q_norm.weight"));
            q_up = Linear(p, "q_up.", "latent_attention.q_up");
        }
        if (s.options.get_bool("sink", false)) a.sink = f32_or_null(&p.at("sink"));
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t hidden = need_int(s, "hidden"), H = need_int(s, "n_head"), dim = need_int(s, "dim", 0), rot = need_int(s, "rot_dim", 0);
        const int64_t vdim = need_int(s, "vdim"), rank = need_int(s, "kv_rank");
        const bool own = s.options.get_bool("own_latent", true), gated = s.options.get_bool("head_gate", false);
        const int64_t q_rank = s.options.get_int("q_rank", 0);
        std::vector<ParamDecl> out;
        // One projection makes the queries (or their latent) and, where the part has a latent of its own, the row [latent | rotated key] behind
        // them, then the heads' gates.
        Linear::declare(out, "proj.", (q_rank > 0 ? q_rank : H * (dim + rot)) + (own ? rank + rot : 0) + (gated ? H : 0), hidden, false);
        if (q_rank > 0) {
            out.push_back({"q_norm.weight", {q_rank}, ParamKind::Vector});
            Linear::declare(out, "q_up.", H * (dim + rot), q_rank, false);
        }
        if (s.options.get_bool("sink", false)) out.push_back({"sink", {H}, ParamKind::Vector});
        if (own) out.push_back({"latent_norm.weight", {rank}, ParamKind::Vector});
        out.push_back({"uk.weight", {H * dim, rank}, ParamKind::Matrix});
        out.push_back({"uv.weight", {H * vdim, rank}, ParamKind::Matrix});
        Linear::declare(out, "out.", hidden, H * vdim, false);
        return out;
    }
    bool capturable() const override { return true; }
    std::optional<KvNeed> kv_need() const override { return KvNeed{1, a.rank + a.rot, a.window, 1}; }

    void forward(StepContext& ctx, const Rows& h, const Rows& x, CacheUnit unit) override { run(ctx, h, x, &x, unit); }
    void forward_into(StepContext& ctx, const Rows& h, const Rows& y, CacheUnit unit) override { run(ctx, h, y, nullptr, unit); }

    void run(StepContext& ctx, const Rows& h, const Rows& y, const Rows* residual, CacheUnit unit) {
        if (unit.write != own_latent)
            throw invalid_model("latent_attention: a part with a latent of its own writes its cache unit, one without reads another run's; the run order says otherwise");
        const int T = ctx.n_tokens;
        const DType dt = ctx.runtime.dtype;
        Workspace& ws = *ctx.workspace;
        cudaStream_t s = ctx.stream();
        const float* freq = frequencies(s);
        const GroupView* view = nullptr;
        void* cache = ctx.kv(unit.read, &view);
        kernels::LatentShape shape = a;
        shape.page_size = view->group->page_size;
        const int D = a.rank + a.rot;
        // Queries (and this step's cache rows) in 32-bit: the norm of the latent and both rotations read them.
        const int64_t first_cols = q_rank > 0 ? q_rank : q_cols;
        const Rows qd = ws.get(own_latent ? "latent.qd" : "latent.q", T, proj.weight.dim(0), DType::F32);
        proj.forward(ctx, h, qd, T);
        const Rows row = own_latent ? qd.columns(first_cols, D) : Rows{};
        const Rows gates = head_gate ? qd.columns(first_cols + (own_latent ? D : 0), a.n_head) : Rows{};
        const Rows* gate = head_gate ? &gates : nullptr;
        Rows q = qd.columns(0, q_cols);
        if (q_rank > 0) {
            // The queries' own latent: normed in 32-bit, then up to the heads.
            q = ws.get("latent.q_up", T, q_cols, DType::F32);
            const Rows down = qd.columns(0, q_rank);
            if (q_up.bias == nullptr && kernels::gemm_rows_normed_supports(ctx.runtime, down, q_up.weight, T)) {
                // A step of up to 16 tokens in bfloat16: the product normalises its rows itself, as the projections behind a norm do.
                kernels::gemm_rows_normed(s, down, q_gain, nullptr, eps, q_up.weight, nullptr, q, T, kernels::kNone, nullptr, nullptr, true, 0.0f);
            } else {
                const Rows cq = ws.get("latent.cq", T, q_rank, dt);
                kernels::rms_groups(s, down, nullptr, q_gain, cq, T, 1, eps);
                q_up.forward(ctx, cq, q, T);
            }
        }
        // bfloat16 and a shape the tensor-core kernel takes: wide queries in bfloat16 for it; else 32-bit throughout.
        const bool tensor = dt == DType::BF16 && kernels::latent_mma_supports(shape);
        // Steps of few tokens are bound by their launches: one launch before the attention, one after it.
        const bool few = tensor && T <= kFewTokens && kernels::latent_few_supports(shape);
        const Rows wide = ws.get(tensor ? "latent.wide16" : "latent.wide", T, static_cast<int64_t>(a.n_head) * D, tensor ? DType::BF16 : DType::F32);
        if (few) {
            kernels::latent_prepare(s, q, uk, latent_gain, freq, ctx.positions, view->slot_mapping, own_latent ? cache : nullptr, wide, T, shape, eps,
                                    own_latent ? &row : nullptr);
        } else {
            if (own_latent) kernels::latent_store(s, row, latent_gain, freq, ctx.positions, view->slot_mapping, cache, dt, T, shape, eps);
            kernels::rope_heads(s, q, freq, ctx.positions, wide, T, shape);
            if (a.dim > 0)
                kernels::head_matmul(s, q, a.dim + a.rot, uk, static_cast<int64_t>(a.dim) * a.rank, a.rank, 1, wide, D, T, a.rank, a.dim, a.n_head);
            else
                LIYAB_CUDA(cudaMemset2DAsync(wide.data, static_cast<size_t>(wide.stride) * dtype_size(wide.dtype), 0, static_cast<size_t>(wide.cols) * dtype_size(wide.dtype),
                                             static_cast<size_t>(T), s));
        }
        ctx.tap("latent.wide", wide);
        // Steps with runs of tokens hand the attended latents on as bfloat16 where the 64-row kernel takes the shape.
        const bool rows16 = tensor && !few && ctx.max_q_len > 1 && kernels::latent_rows_supports(shape);
        const Rows attended = rows16 ? ws.get("latent.attended16", T, static_cast<int64_t>(a.n_head) * a.rank, DType::BF16)
                                     : ws.get("latent.attended", T, static_cast<int64_t>(a.n_head) * a.rank, DType::F32);
        const Rows values = ws.get("latent.values", T, static_cast<int64_t>(a.n_head) * a.vdim, dt);
        // A head's gate is one factor on everything the head puts out, so it acts where the softmax is divided (the values' map is linear).
        if (rows16) {
            kernels::latent_attention_rows16(s, wide, cache, ctx.q_start, ctx.n_past, view->block_table, view->table_width, attended, T, ctx.n_seq,
                                             ctx.max_q_len, shape, gate);
        } else if (tensor) {
            // A decode step's keys are cut over several blocks so that a few requests still fill the GPU.
            const int span = a.window > 0 ? std::min(a.window, ctx.max_positions) : ctx.max_positions;
            const int splits = ctx.decode_only ? kernels::latent_splits(ctx.n_seq, a.n_head, span) : 1;
            float *part_o = nullptr, *part_ml = nullptr;
            if (splits > 1) {
                part_o = static_cast<float*>(ws.flat("latent.part", static_cast<int64_t>(splits) * T * a.n_head * a.rank, DType::F32));
                part_ml = static_cast<float*>(ws.flat("latent.part_ml", static_cast<int64_t>(splits) * T * a.n_head * 2, DType::F32));
            }
            // Few tokens: the launch after the attention merges the parts and applies the gate; the sink acts where the parts meet, or in
            // the attention itself when the keys are not split.
            kernels::latent_attention_mma(s, wide, cache, ctx.q_start, ctx.n_past, view->block_table, view->table_width, attended, part_o, part_ml, T,
                                          ctx.n_seq, ctx.max_q_len, shape, splits, !few, few ? nullptr : gate);
            if (few) kernels::latent_finish(s, attended, part_o, part_ml, uv, values, T, shape, splits, gate);
        } else {
            kernels::latent_attention(s, dt, wide, cache, ctx.tok_seq, ctx.positions, view->block_table, view->table_width, attended, T, shape, gate);
        }
        if (!few) kernels::head_matmul(s, attended, a.rank, uv, static_cast<int64_t>(a.vdim) * a.rank, 1, a.rank, values, a.vdim, T, a.vdim, a.rank, a.n_head);
        ctx.tap("attention", values);
        out.forward(ctx, values, y, T, kernels::kNone, residual);
    }

    static constexpr int kFewTokens = 64;
    kernels::LatentShape a;
    int64_t hidden = 0, q_cols = 0, q_rank = 0;
    float eps = 1e-6f;
    bool own_latent = true, head_gate = false;
    Linear proj, out, q_up;
    const float* q_gain = nullptr;
    Tensor uk, uv;
    const float* latent_gain = nullptr;
    std::vector<float> freq_host;

private:
    // The rotation's frequencies on the device, made at the first step (which is never a recorded one).
    const float* frequencies(cudaStream_t s) {
        if (freq_dev.data() == nullptr) {
            freq_dev = DeviceBuffer(std::max<size_t>(freq_host.size(), 1) * sizeof(float), true);
            if (!freq_host.empty()) {
                LIYAB_CUDA(cudaMemcpyAsync(freq_dev.data(), freq_host.data(), freq_host.size() * sizeof(float), cudaMemcpyHostToDevice, s));
                LIYAB_CUDA(cudaStreamSynchronize(s));
            }
        }
        return static_cast<const float*>(freq_dev.data());
    }
    DeviceBuffer freq_dev;
};

// ---- gated per-token side input ------------------------------------------------------------------------
// From a side table with `dim` values per token id: g = gelu_tanh(gate x) * table[token]; y = proj g;
// x += y / sqrt(mean(y^2) + eps) * gain.  The two maps are `dim` wide, far narrower than the stream.

class GatedTokenSide final : public TokenInput {
public:
    GatedTokenSide(const PartSpec& s, const Params& p) : eps(static_cast<float>(s.options.get_number("eps", 1e-6))) {
        table = p.at("table");
        gate = p.at("gate.weight");
        proj = p.at("proj.weight");
        gain = f32_or_null(&p.at("norm.weight"));
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t hidden = need_int(s, "hidden"), dim = need_int(s, "dim"), vocab = need_int(s, "vocab");
        return {{"table", {vocab, dim}, ParamKind::Table},
                {"gate.weight", {dim, hidden}, ParamKind::Matrix},
                {"proj.weight", {hidden, dim}, ParamKind::Matrix},
                {"norm.weight", {hidden}, ParamKind::Vector}};
    }
    bool capturable() const override { return true; }
    void forward(StepContext& ctx, const Rows& x) override {
        kernels::token_side(ctx.runtime, ctx.workspace, x, ctx.tokens, table, gate, proj, gain, ctx.n_tokens, eps);
    }
    float eps;
    Tensor table, gate, proj;
    const float* gain = nullptr;
};

// ---- the parallel arrangement ------------------------------------------------------------------------------
// h = norm(x); x += mixer(shift(h)) + feed_forward(h); then the token input acts on x.  Slots: `norm` and `mixer`
// always; `shift`, `feed_forward` and `token_input` where the layer has them.  The feed-forward reads h unshifted.

class ParallelBlock final : public Arrangement {
public:
    ParallelBlock(const LayerSpec& spec, const LayerParts& parts) : norm(parts.get<Norm>("norm")), mixer(parts.get<Mixer>("mixer")), keep_(parts) {
        size_t known = 2;
        if (spec.find("shift") != nullptr) { shift = &parts.get<Shift>("shift"); ++known; }
        if (spec.find("feed_forward") != nullptr) { feed_forward = &parts.get<FeedForward>("feed_forward"); ++known; }
        if (spec.find("token_input") != nullptr) { token_input = &parts.get<TokenInput>("token_input"); ++known; }
        if (spec.slots.size() != known) throw invalid_model("arrangement 'parallel' takes the slots norm, shift, mixer, feed_forward and token_input only");
    }
    bool capturable() const override {
        return norm.capturable() && mixer.capturable() && (shift == nullptr || shift->capturable()) &&
               (feed_forward == nullptr || feed_forward->capturable()) && (token_input == nullptr || token_input->capturable());
    }
    std::vector<Mixer*> mixers() const override { return {&mixer}; }
    std::vector<StateNeed> extra_states() const override { return shift != nullptr ? std::vector<StateNeed>{shift->state_need()} : std::vector<StateNeed>{}; }
    void forward(StepContext& ctx, const Rows& x, CacheUnit unit) override {
        const int T = ctx.n_tokens;
        const Rows h = ctx.workspace->get("block.normed", T, x.cols, ctx.runtime.dtype);
        Rows m = h;
        ctx.phase(Phase::Norm);
        if (shift != nullptr) {
            m = ctx.workspace->get("block.shifted", T, x.cols, ctx.runtime.dtype);
            void* state = ctx.state(unit.extra_state(0));
            if (!shift->forward_normed(ctx, x, norm, h, m, state)) {
                norm.forward(ctx, x, h, T, nullptr);
                shift->forward(ctx, h, m, state);
            }
        } else {
            norm.forward(ctx, x, h, T, nullptr);
        }
        ctx.tap("norm", h);
        ctx.tap("shift", m);
        ctx.phase(Phase::Mixer);
        mixer.forward(ctx, m, x, unit);
        ctx.tap("mixer", x);
        if (feed_forward != nullptr) {
            ctx.phase(Phase::FeedForward);
            feed_forward->forward(ctx, h, x);
            ctx.tap("feed_forward", x);
        }
        if (token_input != nullptr) {
            token_input->forward(ctx, x);
            ctx.tap("token_input", x);
        }
    }
    Norm& norm;
    Mixer& mixer;
    Shift* shift = nullptr;
    FeedForward* feed_forward = nullptr;
    TokenInput* token_input = nullptr;

private:
    LayerParts keep_;
};

}  // namespace liyab::builtin
