// Attention over a cache of latent rows.
//
// A position's cache row is [c | r]: a latent c of `rank` values, from which every head's keys and values are
// linear maps (k_h = U_h c, v_h = V_h c), and one rotated key part r of `rot` values shared by all heads.  The
// maps are moved to the query's side, so that attention runs on the cache rows as they are:
//     score_h(i, j) = ((U_h^T q_h) . c_j + q'_h . r_j) * scale,      out_h(i) = V_h (sum_j p_h(i, j) c_j)
// with q_h the unrotated and q'_h the rotated part of head h's query.  The pieces:
//   lb_latent_store    d = [rank | rot] per token -> RMS norm of the first part, rotation of the second, into the pages
//   lb_rope_heads      rotation of the queries' rotated parts into the wide queries [T, H, rank + rot]
//   lb_head_matmul     a product per head (U_h^T q_h into the wide queries; V_h on the attended latents)
//   lb_latent_attention  softmax attention of wide queries over the rows, causal, optionally windowed
// All arithmetic here is 32-bit (FMA units); the element type only says how rows and weights are stored.
// Summation orders depend on a token's position only, never on the batch or on how a sequence was cut.
#include "api.h"
#include "common.cuh"

#include <math_constants.h>

namespace {

// The pair (u, v) = (x[i], x[i + half]) at angle a = position * freq[i] becomes (u cos a - v sin a, v cos a + u sin a).
// Where pair i of a rotation over `rot_dims` values lies: (i, i + rot_dims / 2), or side by side (2i, 2i + 1) when `interleaved`.
__device__ __forceinline__ int pair_lo(int i, int interleaved) { return interleaved ? 2 * i : i; }
__device__ __forceinline__ int pair_hi(int i, int half, int interleaved) { return interleaved ? 2 * i + 1 : half + i; }
// What multiplies a (token, head)'s result besides the softmax: sigmoid of the head's gate, where there is one.
__device__ __forceinline__ float head_factor(const float* gate, int64_t ldg, int t, int h) {
    return gate != nullptr ? 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h])) : 1.0f;
}

__device__ __forceinline__ void rotate_pair(float u, float v, int position, float freq, float* ru, float* rv) {
    float sn, cs;
    sincosf((float)position * freq, &sn, &cs);
    *ru = u * cs - v * sn;
    *rv = v * cs + u * sn;
}

template <typename T>
__global__ void latent_store_kernel(const float* __restrict__ d, int64_t ldd, const float* __restrict__ gain, const float* __restrict__ freq,
                                    const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping, T* __restrict__ cache,
                                    int rank, int rot, int rot_dims, float eps, int interleaved) {
    __shared__ float scratch[33];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x;
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    const float* in = d + (size_t)t * ldd;
    T* out = cache + (size_t)slot * (rank + rot);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
    const float inv = 1.0f / sqrtf(lb_block_sum(ss, scratch) / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) out[i] = lb_from_float<T>(in[i] * inv * gain[i]);
    const int half = rot_dims / 2, p = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float u, v;
        const int a = rank + pair_lo(i, interleaved), b = rank + pair_hi(i, half, interleaved);
        rotate_pair(in[a], in[b], p, freq[i], &u, &v);
        out[a] = lb_from_float<T>(u);
        out[b] = lb_from_float<T>(v);
    }
    for (int i = rot_dims + threadIdx.x; i < rot; i += blockDim.x) out[rank + i] = lb_from_float<T>(in[rank + i]);
}

// q: [T, H * (dim + rot)], head by head [dim | rot]; wide: [T, H * (rank + rot)] float, head by head [rank | rot].
template <typename T, typename TW>
__global__ void rope_heads_kernel(const T* __restrict__ q, int64_t ldq, const float* __restrict__ freq, const int32_t* __restrict__ positions,
                                  TW* __restrict__ wide, int64_t ldw, int n_head, int dim, int rot, int rot_dims, int rank, int interleaved) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, p = positions[t], half = rot_dims / 2;
    const int keep = rot - rot_dims, per_head = half + keep;
    for (int idx = threadIdx.x; idx < n_head * per_head; idx += blockDim.x) {
        const int h = idx / per_head, i = idx - h * per_head;
        const T* in = q + (size_t)t * ldq + (size_t)h * (dim + rot) + dim;
        TW* out = wide + (size_t)t * ldw + (size_t)h * (rank + rot) + rank;
        if (i < half) {
            float u, v;
            const int a = pair_lo(i, interleaved), b = pair_hi(i, half, interleaved);
            rotate_pair(lb_to_float(in[a]), lb_to_float(in[b]), p, freq[i], &u, &v);
            out[a] = lb_from_float<TW>(u);
            out[b] = lb_from_float<TW>(v);
        } else {
            out[rot_dims + i - half] = lb_from_float<TW>(lb_to_float(in[rot_dims + i - half]));
        }
    }
}

// Steps of few tokens (bfloat16): everything between the projection and the attention in one launch.  Block (t, h) widens head h's
// query of token t: the rotated part as rope_heads_kernel does; the unrotated part through the keys' map uk_h [dim, rank], which
// the block first brings into shared memory in 16-byte pieces (all requests in flight at once), then a thread per latent value.
// Block (t, n_head), where the part has a latent of its own, stores the token's cache row as latent_store_kernel does.
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const float* __restrict__ qd, int64_t ldq, const __nv_bfloat16* __restrict__ uk, const float* __restrict__ gain,
                      const float* __restrict__ freq, const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping,
                      __nv_bfloat16* __restrict__ cache, __nv_bfloat16* __restrict__ wide, int64_t ldw, int n_head, int dim, int rot, int rot_dims,
                      int rank, float eps, int q_cols, const float* __restrict__ latent, int64_t ldl, int interleaved) {
    extern __shared__ __align__(16) unsigned char prep_sm[];
    __nv_bfloat16* map = reinterpret_cast<__nv_bfloat16*>(prep_sm);                     // [dim][rank]
    float* qsm = reinterpret_cast<float*>(prep_sm + (((size_t)dim * rank * 2 + 15) & ~(size_t)15));     // the head's query [dim + rot]
    __shared__ float scratch[33];
    const int t = blockIdx.x, h = blockIdx.y, half = rot_dims / 2;
    if (h < n_head) {                          // the map does not depend on the kernel before: asked for ahead of the wait
        const uint4* src = reinterpret_cast<const uint4*>(uk + (size_t)h * dim * rank);
        uint4* dst = reinterpret_cast<uint4*>(map);
        for (int i = threadIdx.x; i < dim * rank / 8; i += blockDim.x) dst[i] = src[i];
    }
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int p = positions[t];
    if (h == n_head) {
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        const float* in = latent != nullptr ? latent + (size_t)t * ldl : qd + (size_t)t * ldq + q_cols;
        __nv_bfloat16* out = cache + (size_t)slot * (rank + rot);
        float ss = 0.0f;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
        const float inv = 1.0f / sqrtf(lb_block_sum(ss, scratch) / (float)rank + eps);
        for (int i = threadIdx.x; i < rank; i += blockDim.x) out[i] = __float2bfloat16_rn(in[i] * inv * gain[i]);
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float u, v;
            const int a = rank + pair_lo(i, interleaved), b = rank + pair_hi(i, half, interleaved);
            rotate_pair(in[a], in[b], p, freq[i], &u, &v);
            out[a] = __float2bfloat16_rn(u);
            out[b] = __float2bfloat16_rn(v);
        }
        for (int i = rot_dims + threadIdx.x; i < rot; i += blockDim.x) out[rank + i] = __float2bfloat16_rn(in[rank + i]);
        return;
    }
    const float* q = qd + (size_t)t * ldq + (size_t)h * (dim + rot);
    for (int i = threadIdx.x; i < dim + rot; i += blockDim.x) qsm[i] = q[i];
    __syncthreads();
    __nv_bfloat16* out = wide + (size_t)t * ldw + (size_t)h * (rank + rot);
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float u, v;
        const int a = pair_lo(i, interleaved), b = pair_hi(i, half, interleaved);
        rotate_pair(qsm[dim + a], qsm[dim + b], p, freq[i], &u, &v);
        out[rank + a] = __float2bfloat16_rn(u);
        out[rank + b] = __float2bfloat16_rn(v);
    }
    for (int i = rot_dims + threadIdx.x; i < rot; i += blockDim.x) out[rank + i] = __float2bfloat16_rn(qsm[dim + i]);
    for (int n = threadIdx.x; n < rank; n += blockDim.x) {
        float acc = 0.0f;
        for (int d = 0; d < dim; ++d) acc = fmaf(qsm[d], __bfloat162float(map[(size_t)d * rank + n]), acc);
        out[n] = __float2bfloat16_rn(acc);
    }
}

// Steps of few tokens (bfloat16): everything between the attention and the output projection in one launch.  Block (t, h) merges the
// parts of a split attention (or takes the attended latent as it is), then maps it through the values' map uv_h [vdim, rank]: a warp
// per value, lanes along the latent in 16-byte pieces, four values' pieces in flight.
__global__ void __launch_bounds__(128)
latent_finish_kernel(const float* __restrict__ attended, int64_t lda, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                     const __nv_bfloat16* __restrict__ uv, __nv_bfloat16* __restrict__ values, int64_t ldv, int n_tokens, int n_head, int rank, int vdim,
                     int n_splits, const float* __restrict__ sink, const float* __restrict__ gate, int64_t ldg) {
    extern __shared__ float osm[];             // the attended latent [rank], then the parts' factors [n_splits]
    float* factor = osm + rank;
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (n_splits > 1) {
        // The parts' sums for this thread's first two latent values are asked for before the factors are made (up to 16 parts).
        constexpr int kParts = 16;
        float ahead[2][kParts];
        const bool fits = n_splits <= kParts;
        if (fits) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int d = threadIdx.x + k * blockDim.x;
#pragma unroll
                for (int s = 0; s < kParts; ++s)
                    ahead[k][s] = (d < rank && s < n_splits) ? part_o[(((size_t)s * n_tokens + t) * n_head + h) * rank + d] : 0.0f;
            }
        }
        if (warp == 0) {                       // factor_s = 2^(m_s - m) / sum_s 2^(m_s - m) l_s, parts in their order
            float ms = -CUDART_INF_F, ls = 0.0f;
            if (lane < n_splits) {
                const float2 ml = *reinterpret_cast<const float2*>(part_ml + (((size_t)lane * n_tokens + t) * n_head + h) * 2);
                ms = ml.x;
                ls = ml.y;
            }
            // A head's sink joins the divisor as a part without values: maximum sink (in the parts' base-2 scale), sum 1.
            const float sk = sink != nullptr ? sink[h] * 1.4426950408889634f : -CUDART_INF_F;
            const float m = fmaxf(lb_warp_max(ms), sk);
            const float e = ms == -CUDART_INF_F ? 0.0f : exp2f(ms - m);
            float l = sink != nullptr ? exp2f(sk - m) : 0.0f;
            for (int s = 0; s < n_splits; ++s) l += __shfl_sync(0xffffffffu, e * ls, s);
            if (lane < n_splits) factor[lane] = e / l;
        }
        __syncthreads();
        int d_from = threadIdx.x;
        if (fits) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int d = threadIdx.x + k * blockDim.x;
                if (d < rank) {
                    float acc = 0.0f;
#pragma unroll
                    for (int s = 0; s < kParts; ++s)
                        if (s < n_splits) acc = fmaf(factor[s], ahead[k][s], acc);
                    osm[d] = acc;
                }
            }
            d_from = threadIdx.x + 2 * blockDim.x;
        }
        for (int d = d_from; d < rank; d += blockDim.x) {
            float acc = 0.0f;
#pragma unroll 4
            for (int s = 0; s < n_splits; ++s) acc = fmaf(factor[s], part_o[(((size_t)s * n_tokens + t) * n_head + h) * rank + d], acc);
            osm[d] = acc;
        }
    } else {
        for (int d = threadIdx.x; d < rank; d += blockDim.x) osm[d] = attended[(size_t)t * lda + (size_t)h * rank + d];
    }
    __syncthreads();
    const float times = head_factor(gate, ldg, t, h);
    const int pieces = rank / 8;
    // A warp's values in batches of eight; a batch's first pieces are all asked for before any is used.
    for (int v0 = warp; v0 < vdim; v0 += 32) {
        uint4 ahead[8];
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const int v = v0 + 4 * b;
            ahead[b] = make_uint4(0u, 0u, 0u, 0u);
            if (v < vdim && lane < pieces) ahead[b] = *reinterpret_cast<const uint4*>(uv + ((size_t)h * vdim + v) * rank + lane * 8);
        }
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const int v = v0 + 4 * b;
            if (v >= vdim) break;                                  // uniform across the warp
            const __nv_bfloat16* row = uv + ((size_t)h * vdim + v) * rank;
            float acc = 0.0f;
            for (int c = lane; c < pieces; c += 32) {
                const uint4 raw = c == lane ? ahead[b] : *reinterpret_cast<const uint4*>(row + c * 8);
                const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = __bfloat1622float2(w[k]);
                    acc = fmaf(f.x, osm[c * 8 + 2 * k], acc);
                    acc = fmaf(f.y, osm[c * 8 + 2 * k + 1], acc);
                }
            }
            acc = lb_warp_sum(acc);
            if (lane == 0) values[(size_t)t * ldv + (size_t)h * vdim + v] = __float2bfloat16_rn(acc * times);
        }
    }
}

// C[t, h * c_head + n] = sum_k A[t, h * a_head + k] * B[h * b_head + k * b_k + n * b_n] for n < N, k < K.
// Tiles of 32 rows x 64 columns, K in chunks of 32 added in ascending order: a row's sums do not depend on the batch.
template <typename TA, typename TB, typename TC>
__global__ void __launch_bounds__(256)
head_matmul_kernel(const TA* __restrict__ A, int64_t lda, int64_t a_head, const TB* __restrict__ B, int64_t b_head, int64_t b_k, int64_t b_n,
                   TC* __restrict__ C, int64_t ldc, int64_t c_head, int M, int N, int K) {
    __shared__ float As[32][33];
    __shared__ float Bs[32][65];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int h = blockIdx.z, m0 = blockIdx.y * 32, n0 = blockIdx.x * 64;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const TA* a = A + (size_t)h * a_head;
    const TB* b = B + (size_t)h * b_head;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += 32) {
        for (int idx = threadIdx.x; idx < 32 * 32; idx += 256) {
            const int r = idx >> 5, k = idx & 31;
            As[r][k] = (m0 + r < M && k0 + k < K) ? lb_to_float(a[(size_t)(m0 + r) * lda + k0 + k]) : 0.0f;
        }
        if (b_n == 1) {
            for (int idx = threadIdx.x; idx < 32 * 64; idx += 256) {
                const int k = idx >> 6, n = idx & 63;
                Bs[k][n] = (k0 + k < K && n0 + n < N) ? lb_to_float(b[(size_t)(k0 + k) * b_k + (n0 + n)]) : 0.0f;
            }
        } else {
            for (int idx = threadIdx.x; idx < 32 * 64; idx += 256) {
                const int n = idx >> 5, k = idx & 31;
                Bs[k][n] = (k0 + k < K && n0 + n < N) ? lb_to_float(b[(size_t)(k0 + k) * b_k + (size_t)(n0 + n) * b_n]) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {
            const float a0 = As[ty * 2][k], a1 = As[ty * 2 + 1][k];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float bv = Bs[k][tx + 16 * j];
                acc[0][j] = fmaf(a0, bv, acc[0][j]);
                acc[1][j] = fmaf(a1, bv, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = m0 + ty * 2 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n < N) C[(size_t)r * ldc + (size_t)h * c_head + n] = lb_from_float<TC>(acc[i][j]);
        }
    }
}

// One block per (token, group of four heads), one warp per head.  The token's visible rows, from the first visible
// position in steps of 32, are staged as floats in shared memory once for the four heads; lane j of a warp makes the
// score of row j, the warp keeps a running softmax over the steps, and every lane owns the latent's values
// lane, lane + 32, ... of the weighted sum.  RPL bounds rank by 32 * RPL.
constexpr int kHeadsPerBlock = 4;

template <typename T, int RPL>
__global__ void __launch_bounds__(128)
latent_attention_kernel(const float* __restrict__ wide, int64_t ldw, const T* __restrict__ cache, const int32_t* __restrict__ tok_seq,
                        const int32_t* __restrict__ positions, const int32_t* __restrict__ block_table, int table_stride, float* __restrict__ out,
                        int64_t ldo, int n_head, int rank, int rot, int page_size, float scale, int window, const float* __restrict__ sink,
                        const float* __restrict__ gate, int64_t ldg) {
    extern __shared__ float sm[];
    const int D = rank + rot, DS = D | 1;                 // odd row stride: lanes reading one column of 32 rows hit 32 banks
    float* qs = sm;                                        // [4][D]
    float* tile = qs + kHeadsPerBlock * D;                 // [32][DS]
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * kHeadsPerBlock + warp;
    const bool active = h < n_head;
    const int p = positions[t];
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int32_t* table = block_table + (size_t)tok_seq[t] * table_stride;
    for (int i = threadIdx.x; i < kHeadsPerBlock * D; i += blockDim.x) {
        const int hh = blockIdx.y * kHeadsPerBlock + i / D;
        qs[i] = hh < n_head ? wide[(size_t)t * ldw + (size_t)hh * D + (i % D)] : 0.0f;
    }
    float m = -CUDART_INF_F, l = 0.0f, o[RPL];
#pragma unroll
    for (int r = 0; r < RPL; ++r) o[r] = 0.0f;
    const float* qh = qs + warp * D;
    for (int j0 = lo; j0 <= p; j0 += 32) {
        __syncthreads();                                   // the tile of the step before has been used (and qs is written)
        for (int kk = warp; kk < 32; kk += 4) {
            const int j = j0 + kk;
            float* dst = tile + kk * DS;
            if (j <= p) {
                const T* src = cache + ((size_t)table[j / page_size] * page_size + (j % page_size)) * D;
                for (int d = lane; d < D; d += 32) dst[d] = lb_to_float(src[d]);
            } else {
                for (int d = lane; d < D; d += 32) dst[d] = 0.0f;
            }
        }
        __syncthreads();
        if (!active) continue;
        const float* row = tile + lane * DS;
        float dot = 0.0f;
        for (int d = 0; d < D; ++d) dot = fmaf(qh[d], row[d], dot);
        const float sc = j0 + lane <= p ? dot * scale : -CUDART_INF_F;
        const float m_new = fmaxf(m, lb_warp_max(sc));     // finite: the step's first row is visible
        const float corr = expf(m - m_new);               // 0 at the first step (m = -inf)
        const float pj = expf(sc - m_new);
        l = l * corr + lb_warp_sum(pj);
#pragma unroll
        for (int r = 0; r < RPL; ++r) o[r] *= corr;
        for (int kk = 0; kk < 32; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, pj, kk);
            const float* c = tile + kk * DS;
#pragma unroll
            for (int r = 0; r < RPL; ++r) {
                const int d = lane + 32 * r;
                if (d < rank) o[r] = fmaf(pk, c[d], o[r]);
            }
        }
        m = m_new;
    }
    if (!active) return;
    // A head's sink adds exp(sink) to the divisor (no key, no value); the head's gate multiplies the result.
    if (sink != nullptr) {
        const float top = fmaxf(m, sink[h]), f = expf(m - top);
        l = l * f + expf(sink[h] - top);
#pragma unroll
        for (int r = 0; r < RPL; ++r) o[r] *= f;
    }
    const float inv = head_factor(gate, ldg, t, h) / l;
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int d = lane + 32 * r;
        if (d < rank) out[(size_t)t * ldo + (size_t)h * rank + d] = o[r] * inv;
    }
}

template <typename T, int RPL>
int launch_latent_attention(const float* wide, int64_t ldw, const void* cache, const int32_t* tok_seq, const int32_t* positions,
                            const int32_t* block_table, int table_stride, float* out, int64_t ldo, int n_tokens, int n_head, int rank, int rot,
                            int page_size, float scale, int window, const float* sink, const float* gate, int64_t ldg, cudaStream_t s) {
    const int D = rank + rot;
    const size_t smem = ((size_t)kHeadsPerBlock * D + 32 * (size_t)(D | 1)) * sizeof(float);
    if (smem > 220 * 1024) return lb_fail(LB_ERR_UNSUPPORTED, "latent attention: cache rows of %d values do not fit a block", D);
    if (smem > 48 * 1024) LB_CHECK_CUDA(cudaFuncSetAttribute(latent_attention_kernel<T, RPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const dim3 grid(n_tokens, (n_head + kHeadsPerBlock - 1) / kHeadsPerBlock);
    LB_CHECK_CUDA(lb_launch_overlapped(latent_attention_kernel<T, RPL>, grid, dim3(128), smem, s, wide, ldw, (const T*)cache, tok_seq, positions,
                                       block_table, table_stride, out, ldo, n_head, rank, rot, page_size, scale, window, sink, gate, ldg));
    return LB_OK;
}

template <typename T>
int pick_latent_attention(const float* wide, int64_t ldw, const void* cache, const int32_t* tok_seq, const int32_t* positions,
                          const int32_t* block_table, int table_stride, float* out, int64_t ldo, int n_tokens, int n_head, int rank, int rot,
                          int page_size, float scale, int window, const float* sink, const float* gate, int64_t ldg, cudaStream_t s) {
#define LB_LATENT(RPL) launch_latent_attention<T, RPL>(wide, ldw, cache, tok_seq, positions, block_table, table_stride, out, ldo, n_tokens, n_head, \
                                                       rank, rot, page_size, scale, window, sink, gate, ldg, s)
    if (rank <= 128) return LB_LATENT(4);
    if (rank <= 256) return LB_LATENT(8);
    if (rank <= 512) return LB_LATENT(16);
    if (rank <= 1024) return LB_LATENT(32);
#undef LB_LATENT
    return lb_fail(LB_ERR_UNSUPPORTED, "latent attention: a latent of %d values is more than the kernel takes (1024)", rank);
}

template <typename TA, typename TB, typename TC>
int launch_head_matmul(const void* A, int64_t lda, int64_t a_head, const void* B, int64_t b_head, int64_t b_k, int64_t b_n, void* C, int64_t ldc,
                       int64_t c_head, int M, int N, int K, int n_head, cudaStream_t s) {
    const dim3 grid((N + 63) / 64, (M + 31) / 32, n_head);
    LB_CHECK_CUDA(lb_launch_overlapped(head_matmul_kernel<TA, TB, TC>, grid, dim3(256), 0, s, (const TA*)A, lda, a_head, (const TB*)B, b_head, b_k, b_n,
                                       (TC*)C, ldc, c_head, M, N, K));
    return LB_OK;
}

}  // namespace

extern "C" int lb_latent_store(int cache_dtype, const float* d, int64_t ldd, const float* gain, const float* freq, const int32_t* positions,
                               const int32_t* slot_mapping, void* cache, int n_tokens, int rank, int rot, int rot_dims, float eps, void* stream) {
    return lb_latent_store_ext(cache_dtype, d, ldd, gain, freq, positions, slot_mapping, cache, n_tokens, rank, rot, rot_dims, eps, nullptr, stream);
}

extern "C" int lb_latent_store_ext(int cache_dtype, const float* d, int64_t ldd, const float* gain, const float* freq, const int32_t* positions,
                                   const int32_t* slot_mapping, void* cache, int n_tokens, int rank, int rot, int rot_dims, float eps,
                                   const lb_latent_extras* extras, void* stream) {
    const int interleaved = extras != nullptr ? extras->interleaved : 0;
    LB_CHECK_ARG(n_tokens >= 0 && rank > 0 && rot >= 0 && rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0,
                 "latent store: bad sizes rank=%d rot=%d rotated=%d", rank, rot, rot_dims);
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const int threads = rank >= 512 ? 256 : 128;
    if (cache_dtype == LB_F32)
        LB_CHECK_CUDA(lb_launch_overlapped(latent_store_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, d, ldd, gain, freq, positions, slot_mapping,
                                           (float*)cache, rank, rot, rot_dims, eps, interleaved));
    else if (cache_dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(latent_store_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, d, ldd, gain, freq, positions,
                                           slot_mapping, (__nv_bfloat16*)cache, rank, rot, rot_dims, eps, interleaved));
    else return lb_fail(LB_ERR_INVALID_ARGUMENT, "latent store: unknown dtype %d", cache_dtype);
    return LB_OK;
}

// Whether the two launches for steps of few tokens take the shape: the keys' map of a head fits a block's shared memory and both maps
// split into 16-byte pieces; at most 32 parts.
extern "C" int lb_latent_few_supports(int dim, int rot, int rank, int vdim, int n_splits) {
    return dim > 0 && rank % 8 == 0 && ((size_t)dim * rank) % 8 == 0 && (size_t)dim * rank * 2 + (size_t)(dim + rot) * 4 + 16 <= 200 * 1024 && vdim > 0 &&
                   n_splits >= 1 && n_splits <= 32 ? 1 : 0;
}

extern "C" int lb_latent_prepare(const float* qd, int64_t ldq, const void* uk, const float* gain, const float* freq, const int32_t* positions,
                                 const int32_t* slot_mapping, void* cache, void* wide, int64_t ldw, int n_tokens, int n_head, int dim, int rot, int rot_dims,
                                 int rank, float eps, void* stream) {
    return lb_latent_prepare_ext(qd, ldq, uk, gain, freq, positions, slot_mapping, cache, wide, ldw, n_tokens, n_head, dim, rot, rot_dims, rank, eps, nullptr,
                                 stream);
}

extern "C" int lb_latent_prepare_ext(const float* qd, int64_t ldq, const void* uk, const float* gain, const float* freq, const int32_t* positions,
                                     const int32_t* slot_mapping, void* cache, void* wide, int64_t ldw, int n_tokens, int n_head, int dim, int rot,
                                     int rot_dims, int rank, float eps, const lb_latent_extras* extras, void* stream) {
    const lb_latent_extras x = extras != nullptr ? *extras : lb_latent_extras{};
    LB_CHECK_ARG(n_tokens >= 0 && n_head > 0 && n_head < 65535 && dim >= 0 && rot >= 0 && rot_dims <= rot && rot_dims % 2 == 0 && rank > 0,
                 "latent queries: bad sizes heads=%d dim=%d rot=%d rotated=%d", n_head, dim, rot, rot_dims);
    if (n_tokens == 0) return LB_OK;
    if (!lb_latent_few_supports(dim, rot, rank, 8, 2)) return lb_fail(LB_ERR_UNSUPPORTED, "latent queries: the keys' map of %d x %d values does not fit a block", dim, rank);
    const dim3 grid(n_tokens, n_head + (cache != nullptr ? 1 : 0));
    const size_t smem = (((size_t)dim * rank * 2 + 15) & ~(size_t)15) + (size_t)(dim + rot) * sizeof(float);
    if (smem > 48 * 1024) LB_CHECK_CUDA(cudaFuncSetAttribute(latent_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LB_CHECK_CUDA(lb_launch_overlapped(latent_prepare_kernel, grid, dim3(128), smem, static_cast<cudaStream_t>(stream), qd, ldq,
                                       (const __nv_bfloat16*)uk, gain, freq, positions, slot_mapping, (__nv_bfloat16*)cache, (__nv_bfloat16*)wide, ldw, n_head, dim,
                                       rot, rot_dims, rank, eps, n_head * (dim + rot), x.latent, x.ldl, x.interleaved));
    return LB_OK;
}

extern "C" int lb_latent_finish(const float* attended, int64_t lda, const float* part_o, const float* part_ml, const void* uv, void* values, int64_t ldv,
                                int n_tokens, int n_head, int rank, int vdim, int n_splits, void* stream) {
    return lb_latent_finish_ext(attended, lda, part_o, part_ml, uv, values, ldv, n_tokens, n_head, rank, vdim, n_splits, nullptr, stream);
}

extern "C" int lb_latent_finish_ext(const float* attended, int64_t lda, const float* part_o, const float* part_ml, const void* uv, void* values,
                                    int64_t ldv, int n_tokens, int n_head, int rank, int vdim, int n_splits, const lb_latent_extras* extras, void* stream) {
    const lb_latent_extras x = extras != nullptr ? *extras : lb_latent_extras{};
    LB_CHECK_ARG(n_tokens >= 0 && n_head > 0 && n_head <= 65535 && rank > 0 && rank % 8 == 0 && vdim > 0 && n_splits >= 1 && n_splits <= 32,
                 "latent values: bad sizes heads=%d rank=%d vdim=%d parts=%d", n_head, rank, vdim, n_splits);
    if (n_tokens == 0) return LB_OK;
    LB_CHECK_CUDA(lb_launch_overlapped(latent_finish_kernel, dim3(n_tokens, n_head), dim3(128), (size_t)(rank + 32) * sizeof(float), static_cast<cudaStream_t>(stream),
                                       attended, lda, part_o, part_ml, (const __nv_bfloat16*)uv, (__nv_bfloat16*)values, ldv, n_tokens, n_head, rank, vdim,
                                       n_splits, x.sink, x.gate, x.ldg));
    return LB_OK;
}

extern "C" int lb_rope_heads(int q_dtype, int wide_dtype, const void* q, int64_t ldq, const float* freq, const int32_t* positions, void* wide, int64_t ldw,
                             int n_tokens, int n_head, int dim, int rot, int rot_dims, int rank, void* stream) {
    return lb_rope_heads_ext(q_dtype, wide_dtype, q, ldq, freq, positions, wide, ldw, n_tokens, n_head, dim, rot, rot_dims, rank, 0, stream);
}

extern "C" int lb_rope_heads_ext(int q_dtype, int wide_dtype, const void* q, int64_t ldq, const float* freq, const int32_t* positions, void* wide,
                                 int64_t ldw, int n_tokens, int n_head, int dim, int rot, int rot_dims, int rank, int interleaved, void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && n_head > 0 && dim >= 0 && rot >= 0 && rot_dims <= rot && rot_dims % 2 == 0 && rank > 0,
                 "rotation of queries: bad sizes heads=%d dim=%d rot=%d rotated=%d", n_head, dim, rot, rot_dims);
    if (n_tokens == 0 || rot == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    if (q_dtype == LB_F32 && wide_dtype == LB_F32)
        LB_CHECK_CUDA(lb_launch_overlapped(rope_heads_kernel<float, float>, dim3(n_tokens), dim3(128), 0, s, (const float*)q, ldq, freq, positions,
                                           (float*)wide, ldw, n_head, dim, rot, rot_dims, rank, interleaved));
    else if (q_dtype == LB_F32 && wide_dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(rope_heads_kernel<float, __nv_bfloat16>, dim3(n_tokens), dim3(128), 0, s, (const float*)q, ldq, freq, positions,
                                           (__nv_bfloat16*)wide, ldw, n_head, dim, rot, rot_dims, rank, interleaved));
    else return lb_fail(LB_ERR_UNSUPPORTED, "rotation of queries: element types %d -> %d are not built", q_dtype, wide_dtype);
    return LB_OK;
}

extern "C" int lb_head_matmul(int a_dtype, int b_dtype, int c_dtype, const void* A, int64_t lda, int64_t a_head, const void* B, int64_t b_head,
                              int64_t b_k, int64_t b_n, void* C, int64_t ldc, int64_t c_head, int M, int N, int K, int n_head, void* stream) {
    LB_CHECK_ARG(M >= 0 && N > 0 && K > 0 && n_head > 0 && n_head <= 65535, "product per head: bad sizes M=%d N=%d K=%d heads=%d", M, N, K, n_head);
    if (M == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    using B16 = __nv_bfloat16;
#define LB_HEADS(TA, TB, TC) return launch_head_matmul<TA, TB, TC>(A, lda, a_head, B, b_head, b_k, b_n, C, ldc, c_head, M, N, K, n_head, s)
    if (a_dtype == LB_F32 && b_dtype == LB_F32 && c_dtype == LB_F32) LB_HEADS(float, float, float);
    if (a_dtype == LB_BF16 && b_dtype == LB_BF16 && c_dtype == LB_F32) LB_HEADS(B16, B16, float);
    if (a_dtype == LB_F32 && b_dtype == LB_BF16 && c_dtype == LB_BF16) LB_HEADS(float, B16, B16);
    if (a_dtype == LB_F32 && b_dtype == LB_BF16 && c_dtype == LB_F32) LB_HEADS(float, B16, float);
#undef LB_HEADS
    return lb_fail(LB_ERR_UNSUPPORTED, "product per head: element types %d x %d -> %d are not built", a_dtype, b_dtype, c_dtype);
}

extern "C" int lb_latent_attention(int cache_dtype, const float* wide, int64_t ldw, const void* cache, const int32_t* tok_seq,
                                   const int32_t* positions, const int32_t* block_table, int table_stride, float* out, int64_t ldo, int n_tokens,
                                   int n_head, int rank, int rot, int page_size, float scale, int window, void* stream) {
    return lb_latent_attention_ext(cache_dtype, wide, ldw, cache, tok_seq, positions, block_table, table_stride, out, ldo, n_tokens, n_head, rank, rot,
                                   page_size, scale, window, nullptr, stream);
}

extern "C" int lb_latent_attention_ext(int cache_dtype, const float* wide, int64_t ldw, const void* cache, const int32_t* tok_seq,
                                       const int32_t* positions, const int32_t* block_table, int table_stride, float* out, int64_t ldo, int n_tokens,
                                       int n_head, int rank, int rot, int page_size, float scale, int window, const lb_latent_extras* extras,
                                       void* stream) {
    const lb_latent_extras x = extras != nullptr ? *extras : lb_latent_extras{};
    LB_CHECK_ARG(n_tokens >= 0 && n_head > 0 && rank > 0 && rot >= 0 && page_size > 0 && window >= 0,
                 "latent attention: bad sizes heads=%d rank=%d rot=%d page=%d window=%d", n_head, rank, rot, page_size, window);
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    if (cache_dtype == LB_F32)
        return pick_latent_attention<float>(wide, ldw, cache, tok_seq, positions, block_table, table_stride, out, ldo, n_tokens, n_head, rank, rot,
                                            page_size, scale, window, x.sink, x.gate, x.ldg, s);
    if (cache_dtype == LB_BF16)
        return pick_latent_attention<__nv_bfloat16>(wide, ldw, cache, tok_seq, positions, block_table, table_stride, out, ldo, n_tokens, n_head, rank,
                                                    rot, page_size, scale, window, x.sink, x.gate, x.ldg, s);
    return lb_fail(LB_ERR_INVALID_ARGUMENT, "latent attention: unknown dtype %d", cache_dtype);
}
