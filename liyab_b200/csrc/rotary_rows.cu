// Row-wise pieces around attention whose queries and keys are normed over the whole projection and rotated, whose values
// blend with an earlier layer's, and around mixers whose heads are normed together: queries, keys and values on their way
// to the attention kernels and the cache; the norm over all heads with a gate; an activation over some columns of a
// projection; and the experts of a row looked up by its token id.  Statistics, angles, gates and activations are 32-bit
// whatever the element type of the rows.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float rr_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------- queries, keys and values: norm, rotation, blend, store
// A block per token.  From the float row [.. q (H x D) .. k (G x D) .. v (G x E) ..]:
//   norm_mode 0: queries and keys as they are; 1: every head over its own root mean square, gains [D] shared by the heads;
//   2: all of q (and all of k) over one root mean square, gains [H x D] and [G x D];
//   then the first rot_dims values of every query and key head are rotated, value i with value i + rot_dims / 2, by the
//   angle position * freq[i];
//   values: with v_first_in, v = (1 - lambda) v + lambda v_first_in[t]; with v_first_out, the row's own values are left there.
// Queries go to q_out [H x P] (P >= D, E; the rest zeros), keys and values into the cache [page][K|V][G][slot][P].
template <typename T>
__global__ void qkv_rotary_store_kernel(const float* __restrict__ proj, int64_t ld, int q_off, int k_off, int v_off, const float* __restrict__ qw,
                                        const float* __restrict__ kw, T* __restrict__ q_out, int64_t ldq, T* __restrict__ cache,
                                        const int32_t* __restrict__ slot_mapping, int H, int G, int D, int E, int P, int page_size, int norm_mode, float eps,
                                        const int32_t* __restrict__ positions, const float* __restrict__ freq, int rot_dims,
                                        const float* __restrict__ v_first_in, float* __restrict__ v_first_out, int64_t ldv, const float* __restrict__ lambda) {
    __shared__ float red[2][32];
    extern __shared__ float turn[];            // [rot_dims]: cosine then sine of every pair's angle, made once for all heads of the token
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const float* row = proj + (size_t)t * ld;
    // What the rest waits for is asked for together: the position, the slot, the blend's weight and the rows' values for the two sums.
    const int pos = positions != nullptr ? positions[t] : 0;
    const int slot = cache != nullptr ? slot_mapping[t] : -1;
    const float lam = v_first_in != nullptr ? lambda[0] : 0.0f;
    const int half = rot_dims / 2;
    float sq = 0.0f, sk = 0.0f;
    if (norm_mode == 2) {
        for (int i = threadIdx.x; i < H * D; i += blockDim.x) sq = fmaf(row[q_off + i], row[q_off + i], sq);
        for (int i = threadIdx.x; i < G * D; i += blockDim.x) sk = fmaf(row[k_off + i], row[k_off + i], sk);
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * freq[i], &turn[half + i], &turn[i]);
    // Both sums of squares meet behind one barrier (which also makes the angles visible); every thread adds the warps' shares
    // in the same order.
    sq = lb_warp_sum(sq);
    sk = lb_warp_sum(sk);
    if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
    __syncthreads();
    float inv_q = 1.0f, inv_k = 1.0f;
    if (norm_mode == 2) {
        float tq = 0.0f, tk = 0.0f;
        for (int w = 0; w < n_warps; ++w) { tq += red[0][w]; tk += red[1][w]; }
        inv_q = 1.0f / sqrtf(tq / (float)(H * D) + eps);
        inv_k = 1.0f / sqrtf(tk / (float)(G * D) + eps);
    }
    const size_t plane = (size_t)G * page_size * P;
    for (int job = warp; job < H + 2 * G; job += n_warps) {
        if (job >= H + G) {                     // a value head
            const int g = job - H - G;
            const float* src = row + v_off + (size_t)g * E;
            T* dst = nullptr;
            if (slot >= 0) {
                const int page = slot / page_size, off = slot - page * page_size;
                dst = cache + (size_t)page * 2 * plane + plane + ((size_t)g * page_size + off) * P;
            }
            for (int d = lane; d < P; d += 32) {
                float v = 0.0f;
                if (d < E) {
                    v = src[d];
                    if (v_first_out != nullptr) v_first_out[(size_t)t * ldv + (size_t)g * E + d] = v;
                    if (v_first_in != nullptr) v = (1.0f - lam) * v + lam * v_first_in[(size_t)t * ldv + (size_t)g * E + d];
                }
                if (dst != nullptr) dst[d] = lb_from_float<T>(v);
            }
            continue;
        }
        const bool is_q = job < H;
        const int head = is_q ? job : job - H;
        if (!is_q && slot < 0) continue;
        const float* src = row + (is_q ? q_off : k_off) + (size_t)head * D;
        const float* gain = is_q ? qw : kw;
        if (gain != nullptr && norm_mode == 2) gain += (size_t)head * D;
        T* dst;
        if (is_q) {
            dst = q_out + (size_t)t * ldq + (size_t)head * P;
        } else {
            const int page = slot / page_size, off = slot - page * page_size;
            dst = cache + (size_t)page * 2 * plane + ((size_t)head * page_size + off) * P;
        }
        float inv = is_q ? inv_q : inv_k;
        if (norm_mode == 1) {
            float ss = 0.0f;
            for (int d = lane; d < D; d += 32) ss = fmaf(src[d], src[d], ss);
            inv = 1.0f / sqrtf(lb_warp_sum(ss) / (float)D + eps);
        }
        auto normed = [&](int d) {
            float v = src[d] * inv;
            if (norm_mode != 0 && gain != nullptr) v *= gain[d];
            return v;
        };
        for (int d = lane; d < P; d += 32) {
            float v = 0.0f;
            if (d < D) {
                if (d < rot_dims) {
                    const int i = d < half ? d : d - half;
                    const float cs = turn[i], sn = turn[half + i];
                    const float lo = normed(i), hi = normed(i + half);
                    v = d < half ? lo * cs - hi * sn : hi * cs + lo * sn;
                } else {
                    v = normed(d);
                }
            }
            dst[d] = lb_from_float<T>(v);
        }
    }
}

// ---------------------------------------------------------------- out = rms(o over the whole row) * gain * gate(g)
// A block per row; rows of up to four values a thread stay in registers between the sum of squares and the write.
template <typename TO>
__global__ void row_norm_gate_kernel(const float* __restrict__ o, int64_t ldo, const float* __restrict__ g, int64_t ldg, const float* __restrict__ gain,
                                     TO* __restrict__ out, int64_t ld_out, int width, int act, float eps) {
    __shared__ float scratch[33];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int r = blockIdx.x;
    const float* src = o + (size_t)r * ldo;
    constexpr int kKeep = 4;
    const bool kept = width <= kKeep * (int)blockDim.x;
    float held[kKeep];
    float ss = 0.0f;
    if (kept) {
#pragma unroll
        for (int e = 0; e < kKeep; ++e) {
            const int c = threadIdx.x + e * blockDim.x;
            held[e] = c < width ? src[c] : 0.0f;
            ss = fmaf(held[e], held[e], ss);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(src[c], src[c], ss);
    }
    const float inv = 1.0f / sqrtf(lb_block_sum(ss, scratch) / (float)width + eps);
    auto finish = [&](int c, float v) {
        v *= inv;
        if (gain != nullptr) v *= gain[c];
        if (g != nullptr) {
            const float z = g[(size_t)r * ldg + c];
            v *= act == LB_GATE_SILU ? z * rr_sigmoid(z) : rr_sigmoid(z);
        }
        out[(size_t)r * ld_out + c] = lb_from_float<TO>(v);
    };
    if (kept) {
#pragma unroll
        for (int e = 0; e < kKeep; ++e) {
            const int c = threadIdx.x + e * blockDim.x;
            if (c < width) finish(c, held[e]);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) finish(c, src[c]);
    }
}

// The same for rows of up to 128 * NV values that split into 16-byte pieces: a warp a row, the row, its gates and the gains asked for at
// once, the sum of squares by shuffles, no block-wide barrier.
template <typename TO, int NV>
__global__ void __launch_bounds__(128) row_norm_gate_warp_kernel(const float* __restrict__ o, int64_t ldo, const float* __restrict__ g, int64_t ldg,
                                                                 const float* __restrict__ gain, TO* __restrict__ out, int64_t ld_out, int n_rows, int width,
                                                                 int act, float eps) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int lane = threadIdx.x & 31, r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const int pieces = width >> 2;
    const float4* orow = reinterpret_cast<const float4*>(o + (size_t)r * ldo);
    const float4* grow = g != nullptr ? reinterpret_cast<const float4*>(g + (size_t)r * ldg) : nullptr;
    const float4* wrow = reinterpret_cast<const float4*>(gain);
    float4 ov[NV], gv[NV], wv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int p = lane + 32 * i;
        const bool in = p < pieces;
        ov[i] = in ? orow[p] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        gv[i] = in && grow != nullptr ? grow[p] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        wv[i] = in && gain != nullptr ? wrow[p] : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) ss = fmaf(ov[i].x, ov[i].x, fmaf(ov[i].y, ov[i].y, fmaf(ov[i].z, ov[i].z, fmaf(ov[i].w, ov[i].w, ss))));
    const float inv = 1.0f / sqrtf(lb_warp_sum(ss) / (float)width + eps);
    auto gate = [&](float z) { return grow == nullptr ? 1.0f : act == LB_GATE_SILU ? z * rr_sigmoid(z) : rr_sigmoid(z); };
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int p = lane + 32 * i;
        if (p >= pieces) break;
        const float a = ov[i].x * inv * wv[i].x * gate(gv[i].x), b = ov[i].y * inv * wv[i].y * gate(gv[i].y);
        const float c = ov[i].z * inv * wv[i].z * gate(gv[i].z), d = ov[i].w * inv * wv[i].w * gate(gv[i].w);
        TO* dst = out + (size_t)r * ld_out + 4 * p;
        if constexpr (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst) = pk;
        }
    }
}

template <typename TO>
int launch_row_norm_gate_warp(const float* o, int64_t ldo, const float* g, int64_t ldg, const float* gain, TO* out, int64_t ld_out, int n_rows, int width, int act,
                              float eps, cudaStream_t s) {
    const dim3 grid((unsigned)((n_rows + 3) / 4)), block(128);
#define LB_WARP_ROWS(NV) LB_CHECK_CUDA(lb_launch_overlapped(row_norm_gate_warp_kernel<TO, NV>, grid, block, 0, s, o, ldo, g, ldg, gain, out, ld_out, n_rows, width, act, eps))
    if (width <= 256) LB_WARP_ROWS(2);
    else if (width <= 512) LB_WARP_ROWS(4);
    else if (width <= 1024) LB_WARP_ROWS(8);
    else LB_WARP_ROWS(16);
#undef LB_WARP_ROWS
    return LB_OK;
}

// ---------------------------------------------------------------- x[r, c] = act(x[r, c]) for c < cols, in place
__device__ __forceinline__ float rr_activate(float z, int act) {
    return act == LB_GATE_SILU ? z * rr_sigmoid(z) : act == LB_GATE_GELU_TANH ? lb_gelu_tanh(z) : act == LB_GATE_RELU ? fmaxf(z, 0.0f) : rr_sigmoid(z);
}

// Blocks walk the rows, threads the columns (16 bytes a thread and trip where the rows allow: VEC).
template <bool VEC>
__global__ void activate_columns_kernel(float* __restrict__ x, int64_t ld, int n_rows, int cols, int act) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
        float* row = x + (size_t)r * ld;
        if (VEC) {
            float4* row4 = reinterpret_cast<float4*>(row);
            for (int c = threadIdx.x; c < cols / 4; c += blockDim.x) {
                float4 v = row4[c];
                v.x = rr_activate(v.x, act);
                v.y = rr_activate(v.y, act);
                v.z = rr_activate(v.z, act);
                v.w = rr_activate(v.w, act);
                row4[c] = v;
            }
        } else {
            for (int c = threadIdx.x; c < cols; c += blockDim.x) row[c] = rr_activate(row[c], act);
        }
    }
}

// ---------------------------------------------------------------- a row's experts from a table by token id, equal weights
__global__ void router_table_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ table, int32_t* __restrict__ ids,
                                    float* __restrict__ weights, int n_rows, int top, int n_experts, int vocab) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * top) return;
    const int r = i / top, j = i - r * top;
    const int tok = min(max(tokens[r], 0), vocab - 1);
    // An entry outside the experts would send the products out of their matrices: it is kept inside (a file with such a table is refused at load).
    ids[i] = min(max(table[(size_t)tok * top + j], 0), n_experts - 1);
    weights[i] = 1.0f / (float)top;
}


}  // namespace

extern "C" int lb_qkv_rotary_store(int dtype, const float* proj, int64_t ld, int q_off, int k_off, int v_off, const float* q_weight, const float* k_weight,
                                   void* q_out, int64_t ldq, void* cache, const int32_t* slot_mapping, int n_tokens, int n_head, int n_kv_head, int dim,
                                   int vdim, int padded, int page_size, int norm_mode, float eps, const int32_t* positions, const float* freq, int rot_dims,
                                   const float* v_first_in, float* v_first_out, int64_t ldv, const float* lambda, void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && n_head > 0 && n_kv_head > 0 && dim > 0 && vdim > 0 && padded >= dim && padded >= vdim && page_size > 0,
                 "qkv_rotary_store: bad sizes heads=%d/%d dim=%d vdim=%d padded=%d", n_head, n_kv_head, dim, vdim, padded);
    LB_CHECK_ARG(norm_mode >= 0 && norm_mode <= 2, "qkv_rotary_store: norm mode %d (0 none, 1 a head, 2 the whole projection)", norm_mode);
    LB_CHECK_ARG(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || (freq != nullptr && positions != nullptr)),
                 "qkv_rotary_store: %d of %d values cannot be rotated in pairs, or no frequencies and positions were given", rot_dims, dim);
    LB_CHECK_ARG(v_first_in == nullptr || lambda != nullptr, "qkv_rotary_store: a blend of values needs its weight");
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    // A warp a head where a block holds them all (a step of few tokens is then one pass); eight warps in turn for steps of many tokens.
    const int jobs = n_head + 2 * n_kv_head, threads = 32 * min(n_tokens <= 64 ? 16 : 8, jobs);
    const size_t smem = (size_t)max(rot_dims, 1) * sizeof(float);
    if (dtype == LB_F32)
        LB_CHECK_CUDA(lb_launch_overlapped(qkv_rotary_store_kernel<float>, dim3(n_tokens), dim3(threads), smem, s, proj, ld, q_off, k_off, v_off, q_weight, k_weight,
                                           (float*)q_out, ldq, (float*)cache, slot_mapping, n_head, n_kv_head, dim, vdim, padded, page_size, norm_mode, eps,
                                           positions, freq, rot_dims, v_first_in, v_first_out, ldv, lambda));
    else if (dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(qkv_rotary_store_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), smem, s, proj, ld, q_off, k_off, v_off, q_weight,
                                           k_weight, (__nv_bfloat16*)q_out, ldq, (__nv_bfloat16*)cache, slot_mapping, n_head, n_kv_head, dim, vdim, padded,
                                           page_size, norm_mode, eps, positions, freq, rot_dims, v_first_in, v_first_out, ldv, lambda));
    else return lb_fail(LB_ERR_INVALID_ARGUMENT, "qkv_rotary_store: unknown dtype %d", dtype);
    return LB_OK;
}

extern "C" int lb_row_norm_gate(int out_dtype, const float* o, int64_t ldo, const float* g, int64_t ldg, const float* gain, void* out, int64_t ld_out,
                                int n_rows, int width, int act, float eps, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && width > 0 && (act == LB_GATE_SIGMOID || act == LB_GATE_SILU), "row_norm_gate: bad sizes width=%d act=%d", width, act);
    if (n_rows == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const uintptr_t places = reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(gain) | reinterpret_cast<uintptr_t>(out);
    // Steps of many rows take a warp a row; a few rows are better spread over a block each (a lane's 24 gates one after the other took a
    // decode step's launch from 4.5 to 5.8 us, while 2,048 rows went from 9.0 to 7.0 us).
    if (n_rows > 64 && width % 4 == 0 && width <= 2048 && ldo % 4 == 0 && ldg % 4 == 0 && ld_out % 4 == 0 && (places & 15) == 0 && (out_dtype == LB_F32 || out_dtype == LB_BF16)) {
        if (out_dtype == LB_F32) return launch_row_norm_gate_warp<float>(o, ldo, g, ldg, gain, (float*)out, ld_out, n_rows, width, act, eps, s);
        return launch_row_norm_gate_warp<__nv_bfloat16>(o, ldo, g, ldg, gain, (__nv_bfloat16*)out, ld_out, n_rows, width, act, eps, s);
    }
    const int threads = width > 512 ? 256 : 128;
    if (out_dtype == LB_F32)
        LB_CHECK_CUDA(lb_launch_overlapped(row_norm_gate_kernel<float>, dim3(n_rows), dim3(threads), 0, s, o, ldo, g, ldg, gain, (float*)out, ld_out, width, act, eps));
    else if (out_dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(row_norm_gate_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, s, o, ldo, g, ldg, gain, (__nv_bfloat16*)out, ld_out,
                                           width, act, eps));
    else return lb_fail(LB_ERR_INVALID_ARGUMENT, "row_norm_gate: unknown dtype %d", out_dtype);
    return LB_OK;
}

extern "C" int lb_activate_columns(float* x, int64_t ld, int n_rows, int cols, int act, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && cols > 0 && act >= LB_GATE_SIGMOID && act <= LB_GATE_RELU, "activate_columns: bad sizes cols=%d act=%d", cols, act);
    if (n_rows == 0) return LB_OK;
    const bool vec = cols % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    const int threads = cols >= 1024 ? 256 : 128;
    const dim3 grid((unsigned)min(n_rows, 148 * 16));
    if (vec) LB_CHECK_CUDA(lb_launch_overlapped(activate_columns_kernel<true>, grid, dim3(threads), 0, static_cast<cudaStream_t>(stream), x, ld, n_rows, cols, act));
    else LB_CHECK_CUDA(lb_launch_overlapped(activate_columns_kernel<false>, grid, dim3(threads), 0, static_cast<cudaStream_t>(stream), x, ld, n_rows, cols, act));
    return LB_OK;
}

extern "C" int lb_router_table(const int32_t* tokens, const int32_t* table, int32_t* ids, float* weights, int n_rows, int top, int n_experts, int vocab,
                               void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && top > 0 && n_experts > 0 && vocab > 0, "router_table: bad sizes top=%d experts=%d vocab=%d", top, n_experts, vocab);
    if (n_rows == 0) return LB_OK;
    const int total = n_rows * top;
    LB_CHECK_CUDA(lb_launch_overlapped(router_table_kernel, dim3((total + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), tokens, table, ids, weights,
                                       n_rows, top, n_experts, vocab));
    return LB_OK;
}
