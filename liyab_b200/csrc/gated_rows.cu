// Row-wise pieces around mixers with gates and with several branches: a vector added to every row of the stream, the
// sum of several branches' outputs each over its own root mean square, queries and keys normalised per head on their
// way to the attention kernels and the cache, the gate on a mixer's heads (with or without a norm per head), and the
// product of the two halves of a gated feed-forward.  Statistics, gates and activations are 32-bit whatever the
// element type of the rows.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float lb_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float lb_gate(float z, int act) { return act == 1 ? z * lb_sigmoid(z) : lb_sigmoid(z); }

// ---------------------------------------------------------------- x[r, :] += v
__global__ void add_row_kernel(float* __restrict__ x, int64_t ldx, const float* __restrict__ v, int n_rows, int width) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const long total = (long)n_rows * width;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long r = i / width;
        const int c = (int)(i - r * width);
        x[(size_t)r * ldx + c] += v[c];
    }
}

// ---------------------------------------------------------------- x[r, :] += scale * sum_i rms(y_i[r, :]) * w_i
// A block per row; the branches' sums of squares one after the other, then the columns with the branches added in order.
struct Branches {
    const float* y[4];
    const float* w[4];
    int64_t ld[4];
    int n;
};

__global__ void rms_sum_add_kernel(float* __restrict__ x, int64_t ldx, Branches b, int width, float scale, float eps, __nv_bfloat16* __restrict__ x16,
                                   int64_t ld16) {
    __shared__ float scratch[33];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int r = blockIdx.x;
    // Rows of up to four values a thread are read once, all branches' values asked for together, and kept in registers.
    constexpr int kKeep = 4;
    const bool kept = width <= kKeep * (int)blockDim.x;
    float held[4][kKeep];
    if (kept) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int e = 0; e < kKeep; ++e) {
                const int c = threadIdx.x + e * blockDim.x;
                held[i][e] = (i < b.n && c < width) ? b.y[i][(size_t)r * b.ld[i] + c] : 0.0f;
            }
    }
    float inv[4];
    for (int i = 0; i < b.n; ++i) {
        const float* y = b.y[i] + (size_t)r * b.ld[i];
        float ss = 0.0f;
        if (kept) {
#pragma unroll
            for (int e = 0; e < kKeep; ++e) ss = fmaf(held[i][e], held[i][e], ss);
        } else {
            for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(y[c], y[c], ss);
        }
        inv[i] = 1.0f / sqrtf(lb_block_sum(ss, scratch) / (float)width + eps);
    }
    if (kept) {
#pragma unroll
        for (int e = 0; e < kKeep; ++e) {
            const int c = threadIdx.x + e * blockDim.x;
            if (c >= width) break;
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (i >= b.n) break;
                float v = held[i][e] * inv[i];
                if (b.w[i] != nullptr) v *= b.w[i][c];
                acc += v;
            }
            const float sum = x[(size_t)r * ldx + c] + scale * acc;
            x[(size_t)r * ldx + c] = sum;
            if (x16 != nullptr) x16[(size_t)r * ld16 + c] = __float2bfloat16_rn(sum);
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.0f;
        for (int i = 0; i < b.n; ++i) {
            float v = b.y[i][(size_t)r * b.ld[i] + c] * inv[i];
            if (b.w[i] != nullptr) v *= b.w[i][c];
            acc += v;
        }
        const float sum = x[(size_t)r * ldx + c] + scale * acc;
        x[(size_t)r * ldx + c] = sum;
        if (x16 != nullptr) x16[(size_t)r * ld16 + c] = __float2bfloat16_rn(sum);
    }
}

// One branch, rows of up to 128 * NV values that split into 16-byte pieces: a warp per row.  The row of y, the row of x and the gains are
// all asked for at once (16 bytes a lane and piece), the sum of squares meets by shuffles, and the sums go back without a block-wide barrier;
// a step of a few rows is then two round trips to memory, and a step of thousands streams at the copy rate.
template <int NV>
__global__ void __launch_bounds__(128) rms_add_warp_kernel(float* __restrict__ x, int64_t ldx, const float* __restrict__ y, int64_t ldy,
                                                           const float* __restrict__ w, int n_rows, int width, float scale, float eps,
                                                           __nv_bfloat16* __restrict__ x16, int64_t ld16) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int lane = threadIdx.x & 31, r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const int pieces = width >> 2;
    const float4* yr = reinterpret_cast<const float4*>(y + (size_t)r * ldy);
    float4* xr = reinterpret_cast<float4*>(x + (size_t)r * ldx);
    const float4* wr = reinterpret_cast<const float4*>(w);
    float4 yv[NV], xv[NV], wv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int p = lane + 32 * i;
        const bool in = p < pieces;
        yv[i] = in ? yr[p] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        xv[i] = in ? xr[p] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        wv[i] = in && w != nullptr ? wr[p] : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) ss = fmaf(yv[i].x, yv[i].x, fmaf(yv[i].y, yv[i].y, fmaf(yv[i].z, yv[i].z, fmaf(yv[i].w, yv[i].w, ss))));
    const float f = scale / sqrtf(lb_warp_sum(ss) / (float)width + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int p = lane + 32 * i;
        if (p >= pieces) break;
        float4 o;
        o.x = fmaf(yv[i].x * f, wv[i].x, xv[i].x);
        o.y = fmaf(yv[i].y * f, wv[i].y, xv[i].y);
        o.z = fmaf(yv[i].z * f, wv[i].z, xv[i].z);
        o.w = fmaf(yv[i].w * f, wv[i].w, xv[i].w);
        xr[p] = o;
        if (x16 != nullptr) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(x16 + (size_t)r * ld16 + 4 * p) = pk;
        }
    }
}

// ---------------------------------------------------------------- queries and keys normalised per head; keys and values to the cache
// A block per token.  From the float row [.. q (H x D) .. k (G x D) .. v (G x E) ..]: every query head over its root mean
// square times qw into the query rows [H x P] (P >= D, E; the rest zeros), every key head the same with kw into the K plane
// and every value head as it is into the V plane of the cache [page][K|V][G][slot][P].  With `norm` 0 the heads pass as
// they are.  A warp per head, the head's values in the lanes.
template <typename T>
__global__ void qk_norm_store_kernel(const float* __restrict__ proj, int64_t ld, int q_off, int k_off, int v_off, const float* __restrict__ qw,
                                     const float* __restrict__ kw, T* __restrict__ q_out, int64_t ldq, T* __restrict__ cache,
                                     const int32_t* __restrict__ slot_mapping, int H, int G, int D, int E, int P, int page_size, int norm, float eps,
                                     const int32_t* __restrict__ positions, float temp_coef, int temp_every) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const float* row = proj + (size_t)t * ld;
    // The queries' temperature: 1 + coef ln(floor((pos + 1) / every) + 1), one factor a token.
    const float temperature = temp_every > 0 ? fmaf(temp_coef, logf((float)((positions[t] + 1) / temp_every + 1)), 1.0f) : 1.0f;
    const int slot = cache != nullptr ? slot_mapping[t] : -1;
    const size_t plane = (size_t)G * page_size * P;
    for (int job = warp; job < H + 2 * G; job += n_warps) {
        const float* src;
        const float* gain = nullptr;
        T* dst;
        int n;
        bool normed = norm != 0;
        if (job < H) {
            src = row + q_off + (size_t)job * D;
            gain = qw;
            dst = q_out + (size_t)t * ldq + (size_t)job * P;
            n = D;
        } else {
            if (slot < 0) continue;
            const int page = slot / page_size, off = slot - page * page_size;
            const bool is_v = job >= H + G;
            const int g = job - H - (is_v ? G : 0);
            src = row + (is_v ? v_off + (size_t)g * E : k_off + (size_t)g * D);
            gain = kw;
            dst = cache + (size_t)page * 2 * plane + (is_v ? plane : 0) + ((size_t)g * page_size + off) * P;
            n = is_v ? E : D;
            if (is_v) normed = false;
        }
        float inv = 1.0f;
        if (normed) {
            float ss = 0.0f;
            for (int d = lane; d < n; d += 32) ss = fmaf(src[d], src[d], ss);
            inv = 1.0f / sqrtf(lb_warp_sum(ss) / (float)n + eps);
        }
        const float factor = job < H ? temperature : 1.0f;
        for (int d = lane; d < P; d += 32) {
            float v = 0.0f;
            if (d < n) {
                v = src[d] * inv;
                if (normed && gain != nullptr) v *= gain[d];
                v *= factor;
            }
            dst[d] = lb_from_float<T>(v);
        }
    }
}

// ---------------------------------------------------------------- the gate on a mixer's heads
// out[t, h * E + c] = f(o[t, h * o_head + c]) * gain[h * E + c] * act(g[t, h * E + c]); f divides a head's E values by their
// root mean square when `norm` is set.  A warp per (token, head); act 0 = sigmoid, 1 = silu; g null: no gate.
template <typename TI, typename TO>
__global__ void head_gate_kernel(const TI* __restrict__ o, int64_t ldo, int o_head, const float* __restrict__ g, int64_t ldg,
                                 const float* __restrict__ gain, TO* __restrict__ out, int64_t ld_out, int n_tokens, int H, int E, int norm,
                                 int act, float eps) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int lane = threadIdx.x & 31;
    const long pair = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (pair >= (long)n_tokens * H) return;
    const int t = (int)(pair / H), h = (int)(pair - (long)t * H);
    const TI* src = o + (size_t)t * ldo + (size_t)h * o_head;
    float inv = 1.0f;
    if (norm) {
        float ss = 0.0f;
        for (int c = lane; c < E; c += 32) {
            const float v = lb_to_float(src[c]);
            ss = fmaf(v, v, ss);
        }
        inv = 1.0f / sqrtf(lb_warp_sum(ss) / (float)E + eps);
    }
    for (int c = lane; c < E; c += 32) {
        float v = lb_to_float(src[c]) * inv;
        if (gain != nullptr) v *= gain[(size_t)h * E + c];
        if (g != nullptr) v *= lb_gate(g[(size_t)t * ldg + (size_t)h * E + c], act);
        out[(size_t)t * ld_out + (size_t)h * E + c] = lb_from_float<TO>(v);
    }
}

// ---------------------------------------------------------------- mid[r, c] = act(gu[r, c]) * gu[r, F + c]
template <typename TO>
__global__ void gated_act_kernel(const float* __restrict__ gu, int64_t ld, TO* __restrict__ mid, int64_t ldm, int n_rows, int F, int act, float alpha,
                                 float limit) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const long total = (long)n_rows * F;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long r = i / F;
        const int c = (int)(i - r * F);
        const float a = gu[(size_t)r * ld + c], u = gu[(size_t)r * ld + F + c];
        mid[(size_t)r * ldm + c] = lb_from_float<TO>(lb_gated_pair(a, u, act, alpha, limit));
    }
}

int grid_for(long total, int threads) { return (int)min((total + threads - 1) / threads, (long)148 * 16); }

}  // namespace

extern "C" int lb_add_row(float* x, int64_t ldx, const float* v, int n_rows, int width, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && width > 0, "add_row: bad sizes");
    if (n_rows == 0) return LB_OK;
    LB_CHECK_CUDA(lb_launch_overlapped(add_row_kernel, dim3(grid_for((long)n_rows * width, 256)), dim3(256), 0, static_cast<cudaStream_t>(stream), x, ldx, v,
                                       n_rows, width));
    return LB_OK;
}

extern "C" int lb_rms_sum_add(float* x, int64_t ldx, int n_branches, const float* const* y, const int64_t* ldy, const float* const* weight, int n_rows,
                              int width, float scale, float eps, void* stream) {
    return lb_rms_sum_add_rounded(x, ldx, n_branches, y, ldy, weight, n_rows, width, scale, eps, nullptr, 0, stream);
}

extern "C" int lb_rms_sum_add_rounded(float* x, int64_t ldx, int n_branches, const float* const* y, const int64_t* ldy, const float* const* weight,
                                      int n_rows, int width, float scale, float eps, void* x16, int64_t ld16, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && width > 0 && n_branches >= 1 && n_branches <= 4, "rms_sum_add: %d branches (1 to 4)", n_branches);
    if (n_rows == 0) return LB_OK;
    // One branch whose rows split into 16-byte pieces: a warp a row.
    if (n_branches == 1 && width % 4 == 0 && width <= 2048 && ldx % 4 == 0 && ldy[0] % 4 == 0 && ld16 % 4 == 0 &&
        ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y[0]) | reinterpret_cast<uintptr_t>(weight != nullptr ? weight[0] : nullptr)) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(x16) & 7) == 0) {
        const float* w = weight != nullptr ? weight[0] : nullptr;
        const dim3 grid((unsigned)((n_rows + 3) / 4)), block(128);
        auto s = static_cast<cudaStream_t>(stream);
        auto x16p = static_cast<__nv_bfloat16*>(x16);
#define LB_WARP_ROWS(NV) LB_CHECK_CUDA(lb_launch_overlapped(rms_add_warp_kernel<NV>, grid, block, 0, s, x, ldx, y[0], ldy[0], w, n_rows, width, scale, eps, x16p, ld16))
        if (width <= 256) LB_WARP_ROWS(2);
        else if (width <= 512) LB_WARP_ROWS(4);
        else if (width <= 1024) LB_WARP_ROWS(8);
        else LB_WARP_ROWS(16);
#undef LB_WARP_ROWS
        return LB_OK;
    }
    Branches b{};
    b.n = n_branches;
    for (int i = 0; i < n_branches; ++i) {
        b.y[i] = y[i];
        b.ld[i] = ldy[i];
        b.w[i] = weight != nullptr ? weight[i] : nullptr;
    }
    const int threads = width > 512 ? 256 : 128;
    LB_CHECK_CUDA(lb_launch_overlapped(rms_sum_add_kernel, dim3(n_rows), dim3(threads), 0, static_cast<cudaStream_t>(stream), x, ldx, b, width, scale, eps,
                                       static_cast<__nv_bfloat16*>(x16), ld16));
    return LB_OK;
}

extern "C" int lb_qk_norm_store(int dtype, const float* proj, int64_t ld, int q_off, int k_off, int v_off, const float* q_weight, const float* k_weight,
                                void* q_out, int64_t ldq, void* cache, const int32_t* slot_mapping, int n_tokens, int n_head, int n_kv_head, int dim,
                                int vdim, int padded, int page_size, int norm, float eps, void* stream) {
    return lb_qk_norm_store_tempered(dtype, proj, ld, q_off, k_off, v_off, q_weight, k_weight, q_out, ldq, cache, slot_mapping, n_tokens, n_head, n_kv_head,
                                     dim, vdim, padded, page_size, norm, eps, nullptr, 0.0f, 0, stream);
}

extern "C" int lb_qk_norm_store_tempered(int dtype, const float* proj, int64_t ld, int q_off, int k_off, int v_off, const float* q_weight,
                                         const float* k_weight, void* q_out, int64_t ldq, void* cache, const int32_t* slot_mapping, int n_tokens, int n_head,
                                         int n_kv_head, int dim, int vdim, int padded, int page_size, int norm, float eps, const int32_t* positions,
                                         float temp_coef, int temp_every, void* stream) {
    LB_CHECK_ARG(temp_every >= 0 && (temp_every == 0 || positions != nullptr), "qk_norm_store: a temperature needs the tokens' positions");
    LB_CHECK_ARG(n_tokens >= 0 && n_head > 0 && n_kv_head > 0 && dim > 0 && vdim > 0 && padded >= dim && padded >= vdim && page_size > 0,
                 "qk_norm_store: bad sizes heads=%d/%d dim=%d vdim=%d padded=%d", n_head, n_kv_head, dim, vdim, padded);
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const int jobs = n_head + 2 * n_kv_head, threads = 32 * min(8, jobs);
    if (dtype == LB_F32)
        LB_CHECK_CUDA(lb_launch_overlapped(qk_norm_store_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, proj, ld, q_off, k_off, v_off, q_weight, k_weight,
                                           (float*)q_out, ldq, (float*)cache, slot_mapping, n_head, n_kv_head, dim, vdim, padded, page_size, norm, eps,
                                           positions, temp_coef, temp_every));
    else if (dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(qk_norm_store_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, proj, ld, q_off, k_off, v_off, q_weight,
                                           k_weight, (__nv_bfloat16*)q_out, ldq, (__nv_bfloat16*)cache, slot_mapping, n_head, n_kv_head, dim, vdim, padded,
                                           page_size, norm, eps, positions, temp_coef, temp_every));
    else return lb_fail(LB_ERR_INVALID_ARGUMENT, "qk_norm_store: unknown dtype %d", dtype);
    return LB_OK;
}

extern "C" int lb_head_gate(int in_dtype, int out_dtype, const void* o, int64_t ldo, int o_head, const float* g, int64_t ldg, const float* gain, void* out,
                            int64_t ld_out, int n_tokens, int n_head, int vdim, int norm, int act, float eps, void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && n_head > 0 && vdim > 0 && o_head >= vdim && (act == 0 || act == 1), "head_gate: bad sizes heads=%d vdim=%d act=%d", n_head,
                 vdim, act);
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const long pairs = (long)n_tokens * n_head;
    const dim3 grid((unsigned)((pairs + 3) / 4)), block(128);
    using B = __nv_bfloat16;
    if (in_dtype == LB_F32 && out_dtype == LB_F32)
        LB_CHECK_CUDA(lb_launch_overlapped(head_gate_kernel<float, float>, grid, block, 0, s, (const float*)o, ldo, o_head, g, ldg, gain, (float*)out, ld_out,
                                           n_tokens, n_head, vdim, norm, act, eps));
    else if (in_dtype == LB_F32 && out_dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(head_gate_kernel<float, B>, grid, block, 0, s, (const float*)o, ldo, o_head, g, ldg, gain, (B*)out, ld_out, n_tokens,
                                           n_head, vdim, norm, act, eps));
    else if (in_dtype == LB_BF16 && out_dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(head_gate_kernel<B, B>, grid, block, 0, s, (const B*)o, ldo, o_head, g, ldg, gain, (B*)out, ld_out, n_tokens, n_head,
                                           vdim, norm, act, eps));
    else return lb_fail(LB_ERR_INVALID_ARGUMENT, "head_gate: types %d -> %d are not built", in_dtype, out_dtype);
    return LB_OK;
}

extern "C" int lb_gated_act(int out_dtype, const float* gu, int64_t ld, void* mid, int64_t ldm, int n_rows, int inner, int act, void* stream) {
    return lb_gated_act_kind(out_dtype, gu, ld, mid, ldm, n_rows, inner, act, 0.0f, 0.0f, stream);
}

extern "C" int lb_gated_act_kind(int out_dtype, const float* gu, int64_t ld, void* mid, int64_t ldm, int n_rows, int inner, int act, float alpha, float limit,
                                 void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && inner > 0 && act >= 0 && act <= LB_GATE_CAPPED, "gated_act: bad sizes");
    if (n_rows == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const dim3 grid(grid_for((long)n_rows * inner, 256)), block(256);
    if (out_dtype == LB_F32)
        LB_CHECK_CUDA(lb_launch_overlapped(gated_act_kernel<float>, grid, block, 0, s, gu, ld, (float*)mid, ldm, n_rows, inner, act, alpha, limit));
    else if (out_dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(gated_act_kernel<__nv_bfloat16>, grid, block, 0, s, gu, ld, (__nv_bfloat16*)mid, ldm, n_rows, inner, act, alpha, limit));
    else return lb_fail(LB_ERR_INVALID_ARGUMENT, "gated_act: unknown dtype %d", out_dtype);
    return LB_OK;
}
