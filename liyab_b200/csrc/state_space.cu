// The pieces around a state space per head whose step depends on the input (the recurrence itself is the matrix memory's,
// with a decay a token and head: matrix_memory.cu):
//
//   lb_ssm_prepare        from the float rows of the input projection [z | x B C | dt]: a short causal convolution per channel over
//                         x, B and C with SiLU (the taps before a portion's first row come from the request's state, zeros before a
//                         sequence's start), dt = softplus(dt + dt_bias), and the rows the recurrence reads:
//                         [x (inner) | B (G N) | C (G N) | dt x (inner) | -exp(A_log) dt (H)].
//   lb_ssm_conv_state     the last taps - 1 inputs of every request's channels become its state (a launch of its own for steps with
//                         portions, where a portion's first rows read the state while later rows would replace it; a step of single
//                         tokens does it in lb_ssm_prepare).
//   lb_gated_group_norm   y = (o + D[head] x) * silu(z), cut into equal groups each over its own root mean square, times a gain.
//
// lb_ssm_prepare has a form with a channel a thread for any sizes and one with four channels a thread for rows on 16-byte borders.
// Everything is 32-bit: the convolution's inputs stay the float sums of the projection, so a row's result does not depend on
// where its sequence was cut.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float ss_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float ss_silu(float z) { return z * ss_sigmoid(z); }

struct PrepareArgs {
    const float* proj;         // [T, ld]
    int64_t ld;
    int xbc_off, dt_off;       // columns of the convolution's channels and of dt
    const float* taps;         // [channels][K]
    const float* tap_bias;     // [channels] or null
    const float* dt_bias;      // [H] or null
    const float* a_log;        // [H]
    float* state;              // + slot * slot_stride: [K - 1][channels], oldest first
    int64_t slot_stride;
    const int32_t* tok_seq;    // [T]
    const int32_t* q_start;    // [S + 1]
    const int32_t* slots;      // [S]
    float* out;                // [T, ldo]
    int64_t ldo;
    int H, E, GN2, K;          // heads, values a head, 2 x groups x state size, taps
    int update_state;          // a step of single tokens: the row's inputs enter the state here
};

__global__ void __launch_bounds__(256) ssm_prepare_kernel(PrepareArgs a) {
    extern __shared__ float dt_s[];      // [H]
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, seq = a.tok_seq[t];
    const int first = a.q_start[seq], i = t - first;
    const int inner = a.H * a.E, channels = inner + a.GN2, K = a.K;
    const float* row = a.proj + (size_t)t * a.ld;
    float* out = a.out + (size_t)t * a.ldo;
    float* st = a.state + (size_t)a.slots[seq] * a.slot_stride;
    // A row's channels are spread over the blocks (row, 0 .. gridDim.y - 1): every block makes the heads' steps for itself, the
    // first one writes them.
    for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
        const float dt = lb_softplus(row[a.dt_off + h] + (a.dt_bias != nullptr ? a.dt_bias[h] : 0.0f));
        dt_s[h] = dt;
        if (blockIdx.y == 0) out[2 * inner + a.GN2 + h] = -expf(a.a_log[h]) * dt;
    }
    __syncthreads();
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        const float* w = a.taps + (size_t)c * K;
        float acc = a.tap_bias != nullptr ? a.tap_bias[c] : 0.0f;
        for (int j = 0; j < K; ++j) {
            const int idx = i - (K - 1) + j;       // the input's place in the portion; negative: in the state
            const float u = idx >= 0 ? a.proj[(size_t)(first + idx) * a.ld + a.xbc_off + c] : st[(size_t)(K - 1 + idx) * channels + c];
            acc = fmaf(w[j], u, acc);
        }
        const float y = ss_silu(acc);
        out[c] = y;
        if (c < inner) out[inner + a.GN2 + c] = dt_s[c / a.E] * y;
        if (a.update_state) {
            for (int r = 0; r + 1 < K - 1; ++r) st[(size_t)r * channels + c] = st[(size_t)(r + 1) * channels + c];
            if (K > 1) st[(size_t)(K - 2) * channels + c] = row[a.xbc_off + c];
        }
    }
}

// The same four channels a thread, where every row, the state and the output start on 16 bytes and a head's values are a multiple
// of four (so four channels share a step): 16-byte loads and stores, a quarter of the instructions.  KT = 4: the taps of a channel are
// one 16-byte load and the loop over them is unrolled; KT = 0: any number of taps.
template <int KT>
__global__ void __launch_bounds__(256) ssm_prepare_vec4_kernel(PrepareArgs a) {
    extern __shared__ float dt_s[];      // [H]
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, seq = a.tok_seq[t];
    const int first = a.q_start[seq], i = t - first;
    const int inner = a.H * a.E, channels = inner + a.GN2, K = KT > 0 ? KT : a.K;
    const float* row = a.proj + (size_t)t * a.ld;
    float* out = a.out + (size_t)t * a.ldo;
    float* st = a.state + (size_t)a.slots[seq] * a.slot_stride;
    for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
        const float dt = lb_softplus(row[a.dt_off + h] + (a.dt_bias != nullptr ? a.dt_bias[h] : 0.0f));
        dt_s[h] = dt;
        if (blockIdx.y == 0) out[2 * inner + a.GN2 + h] = -expf(a.a_log[h]) * dt;
    }
    __syncthreads();
    for (int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x); c < channels; c += 4 * gridDim.y * blockDim.x) {
        float4 acc = a.tap_bias != nullptr ? *reinterpret_cast<const float4*>(a.tap_bias + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float* w = a.taps + (size_t)c * K;
        auto input = [&](int j) {
            const int idx = i - (K - 1) + j;       // the input's place in the portion; negative: in the state
            return idx >= 0 ? *reinterpret_cast<const float4*>(a.proj + (size_t)(first + idx) * a.ld + a.xbc_off + c)
                            : *reinterpret_cast<const float4*>(st + (size_t)(K - 1 + idx) * channels + c);
        };
        if constexpr (KT == 4) {
            const float4 w0 = *reinterpret_cast<const float4*>(w), w1 = *reinterpret_cast<const float4*>(w + 4);
            const float4 w2 = *reinterpret_cast<const float4*>(w + 8), w3 = *reinterpret_cast<const float4*>(w + 12);
            const float4 u0 = input(0), u1 = input(1), u2 = input(2), u3 = input(3);
            acc.x = fmaf(w0.w, u3.x, fmaf(w0.z, u2.x, fmaf(w0.y, u1.x, fmaf(w0.x, u0.x, acc.x))));
            acc.y = fmaf(w1.w, u3.y, fmaf(w1.z, u2.y, fmaf(w1.y, u1.y, fmaf(w1.x, u0.y, acc.y))));
            acc.z = fmaf(w2.w, u3.z, fmaf(w2.z, u2.z, fmaf(w2.y, u1.z, fmaf(w2.x, u0.z, acc.z))));
            acc.w = fmaf(w3.w, u3.w, fmaf(w3.z, u2.w, fmaf(w3.y, u1.w, fmaf(w3.x, u0.w, acc.w))));
        } else {
            for (int j = 0; j < K; ++j) {
                const float4 u = input(j);
                acc.x = fmaf(w[j], u.x, acc.x);
                acc.y = fmaf(w[K + j], u.y, acc.y);
                acc.z = fmaf(w[2 * K + j], u.z, acc.z);
                acc.w = fmaf(w[3 * K + j], u.w, acc.w);
            }
        }
        const float4 y = make_float4(ss_silu(acc.x), ss_silu(acc.y), ss_silu(acc.z), ss_silu(acc.w));
        *reinterpret_cast<float4*>(out + c) = y;
        if (c < inner) {
            const float dt = dt_s[c / a.E];
            *reinterpret_cast<float4*>(out + inner + a.GN2 + c) = make_float4(dt * y.x, dt * y.y, dt * y.z, dt * y.w);
        }
        if (a.update_state) {
            for (int r = 0; r + 1 < K - 1; ++r)
                *reinterpret_cast<float4*>(st + (size_t)r * channels + c) = *reinterpret_cast<const float4*>(st + (size_t)(r + 1) * channels + c);
            if (K > 1) *reinterpret_cast<float4*>(st + (size_t)(K - 2) * channels + c) = *reinterpret_cast<const float4*>(row + a.xbc_off + c);
        }
    }
}

__global__ void __launch_bounds__(256) ssm_conv_state_kernel(const float* __restrict__ proj, int64_t ld, int xbc_off, float* __restrict__ state,
                                                             int64_t slot_stride, const int32_t* __restrict__ q_start, const int32_t* __restrict__ slots,
                                                             int channels, int K) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int seq = blockIdx.x;
    const int first = q_start[seq], len = q_start[seq + 1] - first;
    if (len <= 0) return;
    float* st = state + (size_t)slots[seq] * slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        // Entry r takes input len - (K - 1) + r of the portion, or, where that lies before the portion, an entry further on in the
        // old state: ascending r never reads what it has written.
        for (int r = 0; r < K - 1; ++r) {
            const int idx = len - (K - 1) + r;
            st[(size_t)r * channels + c] = idx >= 0 ? proj[(size_t)(first + idx) * ld + xbc_off + c] : st[(size_t)(K - 1 + idx) * channels + c];
        }
    }
}

// A block per (row, group).
template <typename T>
__global__ void __launch_bounds__(256) gated_group_norm_kernel(const float* __restrict__ o, int64_t ldo, const float* __restrict__ skip, int64_t lds,
                                                               const float* __restrict__ skip_gain, int head, const float* __restrict__ z, int64_t ldz,
                                                               const float* __restrict__ weight, T* __restrict__ out, int64_t ld_out, int part, float eps) {
    __shared__ float scratch[33];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int r = blockIdx.x, c0 = blockIdx.y * part;
    constexpr int kKeep = 4;
    const bool kept = part <= kKeep * (int)blockDim.x;
    auto value = [&](int c) {
        float v = o[(size_t)r * ldo + c];
        if (skip != nullptr) v = fmaf(skip_gain[c / head], skip[(size_t)r * lds + c], v);
        if (z != nullptr) v *= ss_silu(z[(size_t)r * ldz + c]);
        return v;
    };
    float held[kKeep];
    float ss = 0.0f;
    if (kept) {
#pragma unroll
        for (int e = 0; e < kKeep; ++e) {
            const int c = threadIdx.x + e * blockDim.x;
            held[e] = c < part ? value(c0 + c) : 0.0f;
            ss = fmaf(held[e], held[e], ss);
        }
    } else {
        for (int c = threadIdx.x; c < part; c += blockDim.x) {
            const float v = value(c0 + c);
            ss = fmaf(v, v, ss);
        }
    }
    const float inv = 1.0f / sqrtf(lb_block_sum(ss, scratch) / (float)part + eps);
    if (kept) {
#pragma unroll
        for (int e = 0; e < kKeep; ++e) {
            const int c = threadIdx.x + e * blockDim.x;
            if (c < part) out[(size_t)r * ld_out + c0 + c] = lb_from_float<T>(held[e] * inv * (weight != nullptr ? weight[c0 + c] : 1.0f));
        }
        return;
    }
    for (int c = threadIdx.x; c < part; c += blockDim.x)
        out[(size_t)r * ld_out + c0 + c] = lb_from_float<T>(value(c0 + c) * inv * (weight != nullptr ? weight[c0 + c] : 1.0f));
}

}  // namespace

extern "C" int lb_ssm_prepare(const float* proj, int64_t ld, int xbc_off, int dt_off, const float* taps, const float* tap_bias, const float* dt_bias,
                              const float* a_log, float* state, int64_t slot_stride, const int32_t* tok_seq, const int32_t* q_start, const int32_t* slots,
                              float* out, int64_t ldo, int n_tokens, int n_seq, int n_head, int vdim, int group_values, int n_taps, int decode_only,
                              void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && n_seq >= 0 && n_head > 0 && vdim > 0 && group_values >= 0 && n_taps >= 1 && n_taps <= 64,
                 "state space: bad sizes heads=%d vdim=%d taps=%d", n_head, vdim, n_taps);
    const int channels = n_head * vdim + group_values;
    LB_CHECK_ARG(slot_stride >= (int64_t)(n_taps - 1) * channels && ldo >= 2 * (int64_t)n_head * vdim + group_values + n_head,
                 "state space: the state slots or the output rows are too small");
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    PrepareArgs a{proj, ld, xbc_off, dt_off, taps, tap_bias, dt_bias, a_log, state, slot_stride, tok_seq, q_start, slots, out, ldo,
                  n_head, vdim, group_values, n_taps, decode_only ? 1 : 0};
    const int by = (channels + 255) / 256;
    auto on16 = [](const void* p) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool vec4 = vdim % 4 == 0 && group_values % 4 == 0 && ld % 4 == 0 && xbc_off % 4 == 0 && ldo % 4 == 0 && slot_stride % 4 == 0 && on16(proj) &&
                      on16(out) && on16(state) && on16(tap_bias) && (n_taps != 4 || on16(taps));
    if (vec4) {
        const int bq = (channels / 4 + 255) / 256;
        const dim3 grid(n_tokens, bq < 64 ? bq : 64);
        if (n_taps == 4) LB_CHECK_CUDA(lb_launch_overlapped(ssm_prepare_vec4_kernel<4>, grid, dim3(256), (size_t)n_head * sizeof(float), s, a));
        else LB_CHECK_CUDA(lb_launch_overlapped(ssm_prepare_vec4_kernel<0>, grid, dim3(256), (size_t)n_head * sizeof(float), s, a));
    } else {
        LB_CHECK_CUDA(lb_launch_overlapped(ssm_prepare_kernel, dim3(n_tokens, by < 64 ? by : 64), dim3(256), (size_t)n_head * sizeof(float), s, a));
    }
    if (!decode_only && n_taps > 1) {
        LB_CHECK_CUDA(lb_launch_overlapped(ssm_conv_state_kernel, dim3(n_seq, by), dim3(256), 0, s, proj, ld, xbc_off, state, slot_stride, q_start, slots,
                                           channels, n_taps));
    }
    return LB_OK;
}

extern "C" int lb_gated_group_norm(int out_dtype, const float* o, int64_t ldo, const float* skip, int64_t lds, const float* skip_gain, int head,
                                   const float* z, int64_t ldz, const float* weight, void* out, int64_t ld_out, int n_rows, int width, int groups,
                                   float eps, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && width > 0 && groups > 0 && width % groups == 0 && (skip == nullptr || (skip_gain != nullptr && head > 0)),
                 "gated group norm: %d values do not split into %d equal groups", width, groups);
    if (n_rows == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const int part = width / groups, threads = part > 512 ? 256 : 128;
    const dim3 grid(n_rows, groups);
    if (out_dtype == LB_F32)
        LB_CHECK_CUDA(lb_launch_overlapped(gated_group_norm_kernel<float>, grid, dim3(threads), 0, s, o, ldo, skip, lds, skip_gain, head, z, ldz, weight,
                                           (float*)out, ld_out, part, eps));
    else if (out_dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(gated_group_norm_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, o, ldo, skip, lds, skip_gain, head, z, ldz,
                                           weight, (__nv_bfloat16*)out, ld_out, part, eps));
    else return lb_fail(LB_ERR_INVALID_ARGUMENT, "gated group norm: unknown dtype %d", out_dtype);
    return LB_OK;
}
