// Parts for designs whose mixers carry a state space per head, and the position encoding that goes with them here:
// a sinusoid added where the tokens are embedded (with an optional RMS norm of the embedded rows), and the mixer
// `state_space` (a selective state space in the dual form: per head a matrix N x vdim that decays by a factor made from
// the input and takes the outer product of an input-made key and the step-scaled values).  Every size and constant is an
// option of the part's spec; none knows the model it is in.
#pragma once

#include <cmath>

#include "gated_parts.h"

namespace liyab::builtin {

// ---- a sinusoid of the position, added to the embedded row -----------------------------------------------------
// x[t] = table[token] * scale + e(p), e[2i] = sin(p w_i), e[2i + 1] = cos(p w_i), w_i = base^(-2i / size).  With `norm` the row is
// then divided by its root mean square (`eps` inside the root) and multiplied by the gain `norm.weight`.  The frequencies are made
// in double precision on the host and travel as two floats each, so that the angle of a far position is as exact as a near one's.

class SinusoidPosition final : public PositionEncoding {
public:
    SinusoidPosition(const PartSpec& s, const Params& p)
        : size(need_int(s, "size")), max_(s.options.get_int("max_positions", int64_t{1} << 30)), eps(static_cast<float>(s.options.get_number("eps", 1e-6))) {
        const double base = s.options.get_number("base", 10000.0);
        if (!(base > 0)) throw invalid_model("sinusoid: base {} is not positive", base);
        for (int64_t i = 0; 2 * i < size; ++i) {
            const double w = std::pow(base, -2.0 * static_cast<double>(i) / static_cast<double>(size));
            const float hi = static_cast<float>(w);
            freq.host.push_back(hi);
            freq.host.push_back(static_cast<float>(w - static_cast<double>(hi)));
        }
        if (s.options.get_bool("norm", false)) gain = f32_or_null(&p.at("norm.weight"));
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        if (!s.options.get_bool("norm", false)) return {};
        return {{"norm.weight", {need_int(s, "size")}, ParamKind::Vector}};
    }
    bool capturable() const override { return true; }
    int64_t max_positions() const override { return max_; }
    void embed(StepContext& ctx, const Tensor& table, float scale, const Rows& x) override {
        kernels::embed_sinusoid(ctx.stream(), ctx.tokens, ctx.positions, table, freq.get(ctx.stream()), gain, x, ctx.n_tokens, scale, eps);
    }
    int64_t size, max_;
    float eps;
    const float* gain = nullptr;

private:
    DeviceFloats freq;
};

// ---- a state space per head whose step depends on the input ------------------------------------------------------
// One projection makes [z (inner) | x (inner) | B (groups x n_state) | C (groups x n_state) | dt (n_head)] in 32-bit, inner = n_head x vdim.
// x, B and C pass a causal convolution per channel over `taps` inputs (weights [channels, taps], the last column the current token's,
// zeros before a sequence's start, an optional bias) and SiLU.  dt = softplus(dt + dt_bias).  Per head h, with its group's B and C
// (head h reads group h / (n_head / groups)):
//     S_t = exp(-exp(a_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T        (S is n_state x vdim, 32-bit, zero at a sequence's start)
//     y_t = S_t^T C_t + skip_h x_t.
// All heads' y times silu(z), cut into `norm_groups` equal parts each over its own root mean square, times the gain `norm.weight`,
// then the output projection.  The recurrence is the matrix memory's with a decay a token and head: keys B, values dt x, queries C,
// heads of a group sharing keys and queries.  A request's state slot holds the memory ([head][value tile][N x tile | N | 1]) and,
// behind it, the convolution's last taps - 1 inputs ([taps - 1][channels]).

class StateSpaceMixer final : public Mixer {
public:
    StateSpaceMixer(const PartSpec& s, const Params& p) {
        hidden = need_int(s, "hidden");
        ss.n_head = static_cast<int>(need_int(s, "n_head"));
        ss.vdim = static_cast<int>(need_int(s, "vdim"));
        ss.n_state = static_cast<int>(need_int(s, "n_state"));
        ss.groups = static_cast<int>(s.options.get_int("groups", 1));
        ss.taps = static_cast<int>(s.options.get_int("taps", 1));
        norm_groups = static_cast<int>(s.options.get_int("norm_groups", 1));
        eps = static_cast<float>(s.options.get_number("eps", 1e-6));
        if (ss.groups < 1 || ss.n_head % ss.groups != 0) throw invalid_model("state_space: {} heads do not split over {} groups", ss.n_head, ss.groups);
        if (ss.taps < 1 || ss.taps > 64) throw invalid_model("state_space: a convolution over {} inputs is outside [1, 64]", ss.taps);
        if (norm_groups < 1 || ss.inner() % norm_groups != 0) throw invalid_model("state_space: {} values do not split into {} equal groups", ss.inner(), norm_groups);
        m.n_head = ss.n_head;
        m.dim = ss.n_state;
        m.vdim = ss.vdim;
        m.value_tile = kernels::memory_value_tile(m.dim, m.vdim);
        m.qk_share = ss.n_head / ss.groups;
        m.slot_stride = m.slot_floats() + ss.conv_floats();
        proj = Linear(p, "proj.", "state_space.proj");
        out = Linear(p, "out.", "state_space.out");
        taps = f32_or_null(&p.at("conv.weight"));
        tap_bias = f32_or_null(p.find("conv.bias"));
        dt_bias = f32_or_null(p.find("dt_bias"));
        a_log = f32_or_null(&p.at("a_log"));
        skip = f32_or_null(p.find("skip"));
        norm_gain = f32_or_null(p.find("norm.weight"));
    }
    static std::vector<ParamDecl> parameters(const PartSpec& s) {
        const int64_t hidden = need_int(s, "hidden"), H = need_int(s, "n_head"), E = need_int(s, "vdim"), N = need_int(s, "n_state");
        const int64_t G = s.options.get_int("groups", 1), K = s.options.get_int("taps", 1), inner = H * E, channels = inner + 2 * G * N;
        std::vector<ParamDecl> out;
        Linear::declare(out, "proj.", inner + channels + H, hidden, false);
        out.push_back({"conv.weight", {channels, K}, ParamKind::Vector});
        if (s.options.get_bool("conv_bias", true)) out.push_back({"conv.bias", {channels}, ParamKind::Vector});
        if (s.options.get_bool("dt_bias", true)) out.push_back({"dt_bias", {H}, ParamKind::Vector});
        out.push_back({"a_log", {H}, ParamKind::Vector});
        if (s.options.get_bool("skip", true)) out.push_back({"skip", {H}, ParamKind::Vector});
        if (s.options.get_bool("norm_gain", true)) out.push_back({"norm.weight", {inner}, ParamKind::Vector});
        Linear::declare(out, "out.", hidden, inner, false);
        return out;
    }
    bool capturable() const override { return true; }
    std::optional<StateNeed> state_need() const override { return StateNeed{{m.stride()}, DType::F32}; }
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

    kernels::StateSpaceShape ss;
    kernels::MemoryShape m;
    int64_t hidden = 0;
    int norm_groups = 1;
    float eps = 1e-6f;
    Linear proj, out;
    const float* taps = nullptr;
    const float* tap_bias = nullptr;
    const float* dt_bias = nullptr;
    const float* a_log = nullptr;
    const float* skip = nullptr;
    const float* norm_gain = nullptr;

private:
    void run(StepContext& ctx, const Rows* h, const Rows* x_in, const NormRecipe* norm, const Rows& y, const Rows* residual, CacheUnit unit) {
        if (!unit.write) throw invalid_model("state_space: a state is carried by the run that owns it; the run order lets another read it");
        const int T = ctx.n_tokens;
        Workspace& ws = *ctx.workspace;
        cudaStream_t s = ctx.stream();
        const Rows pr = ws.get("state_space.proj", T, proj.weight.dim(0), DType::F32);
        if (h != nullptr) kernels::linear(ctx.runtime, &ws, *h, proj.weight, nullptr, pr, T, kernels::kNone, nullptr);
        else kernels::gemm_rows_normed(s, *x_in, norm->gain, norm->offset, norm->eps, proj.weight, nullptr, pr, T, kernels::kNone, nullptr, nullptr, norm->rms,
                                       norm->gain_offset);
        const int64_t inner = ss.inner(), GN = static_cast<int64_t>(ss.groups) * ss.n_state;
        float* state = static_cast<float*>(ctx.state(unit.read));
        const Rows rows = ws.get("state_space.rows", T, ss.prepared_cols(), DType::F32);
        kernels::ssm_prepare(s, pr, taps, tap_bias, dt_bias, a_log, state + m.slot_floats(), m.stride(), ctx.tok_seq, ctx.q_start, ctx.state_slots, rows, T,
                             ctx.n_seq, ss, ctx.decode_only);
        const Rows xs = rows.columns(0, inner), keys = rows.columns(inner, GN), queries = rows.columns(inner + GN, GN);
        const Rows values = rows.columns(inner + 2 * GN, inner), log_keep = rows.columns(2 * inner + 2 * GN, ss.n_head);
        const Rows o = ws.get("state_space.o", T, inner, DType::F32);
        if (ctx.max_q_len >= MatrixMemory::kPiecesFrom) {
            float* scratch = static_cast<float*>(ws.flat("state_space.pieces", kernels::memory_pieces_floats(T, ctx.n_seq, m), DType::F32));
            kernels::matrix_memory_pieces(s, queries, keys, values, nullptr, &log_keep, nullptr, nullptr, ctx.positions, ctx.q_start, ctx.state_slots, state, o, T,
                                          ctx.n_seq, m, scratch);
        } else {
            kernels::matrix_memory(s, queries, keys, values, nullptr, &log_keep, nullptr, nullptr, ctx.positions, ctx.q_start, ctx.state_slots, state, o, ctx.n_seq, m,
                                   ctx.max_q_len >= MatrixMemory::kChunkedFrom);
        }
        ctx.tap("memory", o);
        const Rows heads = ws.get("state_space.heads", T, inner, ctx.runtime.dtype);
        const Rows z = pr.columns(0, inner);
        kernels::gated_group_norm(s, o, skip != nullptr ? &xs : nullptr, skip, ss.vdim, &z, norm_gain, heads, T, norm_groups, eps);
        ctx.tap("state_space", heads);
        kernels::linear(ctx.runtime, &ws, heads, out.weight, nullptr, y, T, kernels::kNone, residual);
    }
};

}  // namespace liyab::builtin
