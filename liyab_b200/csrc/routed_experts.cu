// A feed-forward of many small experts of which every row uses a few.
//
//   lb_router_topk     z = router . h in 32-bit, score = sigmoid(z) (or the softmax over the experts), the `top` largest
//                      per row (ties to the lower expert), their scores as weights (optionally divided by their sum).
//   lb_expert_plan     the (row, choice) pairs sorted by expert, stably: offsets per expert, the sorted place of every
//                      pair and the pair at every place.  One block; nothing returns to the host.
//   lb_expert_product  for every expert the product of its pairs' rows with its own matrix, in tiles of rows that never
//                      span two experts.  Either the first half of an expert, mid = act(gate . a) * (up . a) with
//                      a = weight * h[row] gathered through the plan, or the second, y = down . mid.  32-bit FMA sums with K
//                      in ascending order, so a row's result does not depend on which other rows share its tile.
//   lb_expert_combine  x[row] += the sum of its pairs' results, in the order of its choices.
#include "api.h"
#include "common.cuh"

#include <math_constants.h>

namespace {

__device__ __forceinline__ float lb_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------- router
template <typename T>
__global__ void router_topk_kernel(const T* __restrict__ h, int64_t ldh, const T* __restrict__ router, int32_t* __restrict__ ids,
                                   float* __restrict__ weights, int E, int width, int top, int softmax, int renormalise, const float* __restrict__ bias) {
    extern __shared__ float z[];       // [E]
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const T* row = h + (size_t)t * ldh;
    // A warp per expert; a lane's terms are asked for eight at a time, so that a short row is one or two round trips.  The order of
    // a lane's sum stays ascending, so z does not depend on the batch.
    for (int e = warp; e < E; e += n_warps) {
        const T* w = router + (size_t)e * width;
        float acc = 0.0f;
        for (int c0 = lane; c0 < width; c0 += 32 * 8) {
            float a[8], b[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int c = c0 + 32 * u;
                a[u] = c < width ? lb_to_float(row[c]) : 0.0f;
                b[u] = c < width ? lb_to_float(w[c]) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) acc = fmaf(a[u], b[u], acc);
        }
        acc = lb_warp_sum(acc);
        if (lane == 0) z[e] = bias != nullptr ? acc + bias[e] : acc;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    float zmax = -CUDART_INF_F, zsum = 0.0f;
    if (softmax) {
        for (int e = 0; e < E; ++e) zmax = fmaxf(zmax, z[e]);
        for (int e = 0; e < E; ++e) zsum += expf(z[e] - zmax);
    }
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
        int best = 0;
        for (int e = 1; e < E; ++e)
            if (z[e] > z[best]) best = e;
        const float s = softmax ? expf(z[best] - zmax) / zsum : lb_sigmoid(z[best]);
        ids[(size_t)t * top + k] = best;
        weights[(size_t)t * top + k] = s;
        total += s;
        z[best] = -CUDART_INF_F;
    }
    if (renormalise)
        for (int k = 0; k < top; ++k) weights[(size_t)t * top + k] /= total;
}

// ---------------------------------------------------------------- plan
// offsets [E + 1]; place[pair] = where the pair stands in the sorted order; pair_at[place] = the pair.
// With `tokens` and `table` (int32 [vocab, top]) the pairs' experts are first looked up by the rows' token ids, pair (r, j) -> table[tokens[r]][j],
// left in ids_global, and every pair's weight 1 / top in `weights`: the routing without a router, in the plan's own launch.
__global__ void __launch_bounds__(1024) expert_plan_kernel(int32_t* __restrict__ ids_global, int n_pairs, int E, int32_t* __restrict__ offsets,
                                                           int32_t* __restrict__ place, int32_t* __restrict__ pair_at, int staged,
                                                           const int32_t* __restrict__ tokens, const int32_t* __restrict__ table, int vocab, int top,
                                                           float* __restrict__ weights) {
    extern __shared__ int counts[];    // [E + 1], then the pairs' experts where they fit (`staged`)
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    if (tokens != nullptr) {
        for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
            const int r = p / top, tok = min(max(tokens[r], 0), vocab - 1);
            ids_global[p] = min(max(table[(size_t)tok * top + (p - r * top)], 0), E - 1);      // an entry outside the experts is kept inside
            weights[p] = 1.0f / (float)top;
        }
        __syncthreads();                // the block's own writes are what it reads below
    }
    // Every warp walks all pairs twice: from shared memory where they fit, so that a walk is not a chain of round trips.
    const int32_t* ids = ids_global;
    if (staged) {
        int* mine = counts + E + 1;
        for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) mine[p] = ids_global[p];
        ids = mine;
        __syncthreads();
    }
    for (int e = warp; e < E; e += n_warps) {
        int n = 0;
        for (int p0 = 0; p0 < n_pairs; p0 += 32) {
            const int p = p0 + lane;
            n += __popc(__ballot_sync(0xffffffffu, p < n_pairs && ids[p] == e));
        }
        if (lane == 0) counts[e] = n;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            const int n = counts[e];
            counts[e] = at;
            offsets[e] = at;
            at += n;
        }
        counts[E] = at;
        offsets[E] = at;
    }
    __syncthreads();
    for (int e = warp; e < E; e += n_warps) {
        int at = counts[e];
        for (int p0 = 0; p0 < n_pairs; p0 += 32) {
            const int p = p0 + lane;
            const bool mine = p < n_pairs && ids[p] == e;
            const unsigned mask = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int where = at + __popc(mask & ((1u << lane) - 1u));
                place[p] = where;
                pair_at[where] = p;
            }
            at += __popc(mask);
        }
    }
}

// ---------------------------------------------------------------- the experts' products
struct ProductArgs {
    const void* a;             // first half: the rows h [T, lda]; second half: mid [pairs, lda]
    int64_t lda;
    const void* w;             // [E][rows_per_expert][K]
    int64_t expert_stride;     // elements between two experts' matrices
    const int32_t* offsets;    // [E + 1]
    const int32_t* pair_at;    // [pairs]
    const float* weights;      // [pairs], or null where the weight multiplies the experts' results instead (lb_expert_combine_weighted)
    void* out;                 // first half: mid [pairs, ldo] of the element type; second: y [pairs, ldo] float
    int64_t ldo;
    int E, N, K, top, act;
    float alpha, limit;        // the capped gate's two numbers
};

constexpr int kBN = 64, kBK = 16;

// 256 threads as 16 x 16; a thread makes TM x 4 results.  GATED: two matrices a tile (rows [0, N) gate, [N, 2N) up).
template <typename T, int TM, bool GATED>
__global__ void __launch_bounds__(256) expert_product_kernel(ProductArgs p) {
    constexpr int BM = 16 * TM;
    __shared__ float As[kBK][BM + 1];
    __shared__ float Bs[GATED ? 2 : 1][kBK][kBN + 1];
    __shared__ int tile_info[2];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, found = -1, first = 0;
        for (int e = 0; e < p.E; ++e) {
            const int n = p.offsets[e + 1] - p.offsets[e], tiles = (n + BM - 1) / BM;
            if (tile < tiles) {
                found = e;
                first = p.offsets[e] + tile * BM;
                break;
            }
            tile -= tiles;
        }
        tile_info[0] = found;
        tile_info[1] = first;
    }
    __syncthreads();
    const int e = tile_info[0];
    if (e < 0) return;
    const int r0 = tile_info[1], r_end = p.offsets[e + 1];
    const int n0 = blockIdx.y * kBN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const T* W = static_cast<const T*>(p.w) + (size_t)e * p.expert_stride;
    const T* A = static_cast<const T*>(p.a);

    // What this thread stages: element (row ar, k ak) of the A tile, TM of them, and (feature bn, k bk) of the B tile, four.
    float acc[TM][4], acc2[GATED ? TM : 1][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.0f;
            if (GATED) acc2[i][j] = 0.0f;
        }
    const int ak = threadIdx.x & 15, ar0 = threadIdx.x >> 4;      // rows ar0 + 16 * i
    const T* a_src[TM];
    float a_scale[TM];
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = r0 + ar0 + 16 * i;
        a_src[i] = nullptr;
        a_scale[i] = 1.0f;
        if (r < r_end) {
            if (GATED) {
                const int pair = p.pair_at[r];
                a_src[i] = A + (size_t)(pair / p.top) * p.lda;
                if (p.weights != nullptr) a_scale[i] = p.weights[pair];
            } else {
                a_src[i] = A + (size_t)r * p.lda;
            }
        }
    }
    for (int k0 = 0; k0 < p.K; k0 += kBK) {
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int k = k0 + ak;
            As[ak][ar0 + 16 * i] = (a_src[i] != nullptr && k < p.K) ? lb_to_float(a_src[i][k]) * a_scale[i] : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int n = n0 + ar0 + 16 * i, k = k0 + ak;
            const bool ok = n < p.N && k < p.K;
            Bs[0][ak][ar0 + 16 * i] = ok ? lb_to_float(W[(size_t)n * p.K + k]) : 0.0f;
            if (GATED) Bs[1][ak][ar0 + 16 * i] = ok ? lb_to_float(W[(size_t)(p.N + n) * p.K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kBK; ++kk) {
            float av[TM], bv[4], bv2[4];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                bv[j] = Bs[0][kk][tx * 4 + j];
                if (GATED) bv2[j] = Bs[1][kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
                    if (GATED) acc2[i][j] = fmaf(av[i], bv2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = r0 + ty * TM + i;
        if (r >= r_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            if (GATED) {
                static_cast<T*>(p.out)[(size_t)r * p.ldo + n] = lb_from_float<T>(lb_gated_pair(acc[i][j], acc2[i][j], p.act, p.alpha, p.limit));
            } else {
                static_cast<float*>(p.out)[(size_t)r * p.ldo + n] = acc[i][j];
            }
        }
    }
}

// ---------------------------------------------------------------- the same products on the tensor cores (bfloat16)
// 64 rows x 64 features a block, K in steps of 32, four warps of 16 rows each (`mma.sync m16n8k16`, 32-bit sums).  Both operands'
// tiles come by cp.async through a ring of three stages, two steps ahead of the products; the first half multiplies its 32-bit sums
// by the pair's weight before the gate (the weight on the expert's input, moved past the two linear maps).  Needs K, the rows' stride and the
// experts' stride to be multiples of 8 elements and 16-byte aligned bases.
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kMM = 64, kMN = 64, kMK = 32, kMLD = kMK + 8, kMStages = 3;
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <bool GATED>
__global__ void __launch_bounds__(128) expert_product_mma_kernel(ProductArgs p) {
    using B16 = __nv_bfloat16;
    __shared__ __align__(16) B16 As[kMStages][kMM][kMLD];
    __shared__ __align__(16) B16 Bs[kMStages][GATED ? 2 : 1][kMN][kMLD];
    __shared__ int tile_info[2];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, found = -1, first = 0;
        for (int e = 0; e < p.E; ++e) {
            const int n = p.offsets[e + 1] - p.offsets[e], tiles = (n + kMM - 1) / kMM;
            if (tile < tiles) {
                found = e;
                first = p.offsets[e] + tile * kMM;
                break;
            }
            tile -= tiles;
        }
        tile_info[0] = found;
        tile_info[1] = first;
    }
    __syncthreads();
    const int e = tile_info[0];
    if (e < 0) return;
    const int r0 = tile_info[1], r_end = p.offsets[e + 1];
    const int n0 = blockIdx.y * kMN;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const B16* W = static_cast<const B16*>(p.w) + (size_t)e * p.expert_stride;
    const B16* A = static_cast<const B16*>(p.a);

    // This thread's two 16-byte pieces of every A tile and of every B tile: piece v -> (row v / 4, elements (v % 4) * 8 ..).  The first
    // half's rows are the pairs' rows of h as they are: the pair's weight multiplies the sums in the epilogue (W (w h) = w (W h)).
    const B16* a_src[2];
    const B16* b_src[2];
    int piece_row[2], piece_k[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int v = threadIdx.x + 128 * i;
        piece_row[i] = v >> 2;
        piece_k[i] = (v & 3) * 8;
        const int r = r0 + piece_row[i];
        a_src[i] = nullptr;
        if (r < r_end) a_src[i] = GATED ? A + (size_t)(p.pair_at[r] / p.top) * p.lda : A + (size_t)r * p.lda;
        const int n = n0 + piece_row[i];
        b_src[i] = n < p.N ? W + (size_t)n * p.K : nullptr;
    }
    auto fetch = [&](int k0, int stage) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int k = k0 + piece_k[i];
            const bool a_ok = a_src[i] != nullptr && k < p.K, b_ok = b_src[i] != nullptr && k < p.K;
            cp_async16(&As[stage][piece_row[i]][piece_k[i]], a_ok ? a_src[i] + k : W, a_ok);
            cp_async16(&Bs[stage][0][piece_row[i]][piece_k[i]], b_ok ? b_src[i] + k : W, b_ok);
            if (GATED) cp_async16(&Bs[stage][1][piece_row[i]][piece_k[i]], b_ok ? b_src[i] + (size_t)p.N * p.K + k : W, b_ok);
        }
    };

    float acc[8][4], acc2[GATED ? 8 : 1][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.0f;
            if (GATED) acc2[i][j] = 0.0f;
        }
    const int steps = (p.K + kMK - 1) / kMK;
    // kMStages - 1 steps ahead; one group per step, empty past the last.
#pragma unroll
    for (int i = 0; i < kMStages - 1; ++i) {
        if (i < steps) fetch(i * kMK, i);
        cp_async_commit();
    }
    for (int it = 0; it < steps; ++it) {
        const int stage = it % kMStages;
        cp_async_wait<kMStages - 2>();          // this step's group
        __syncthreads();                        // .. from every thread; and everyone is done with the stage that is filled next
        if (it + kMStages - 1 < steps) fetch((it + kMStages - 1) * kMK, (it + kMStages - 1) % kMStages);
        cp_async_commit();
        const int mat = lane >> 3, r = lane & 7;
#pragma unroll
        for (int kk = 0; kk < kMK / 16; ++kk) {
            uint32_t af[4];
            ldmatrix_x4(af, smem_addr(&As[stage][warp * 16 + (mat & 1) * 8 + r][kk * 16 + (mat >> 1) * 8]));
#pragma unroll
            for (int nt = 0; nt < 8; nt += 2) {
                uint32_t b[4];
                ldmatrix_x4(b, smem_addr(&Bs[stage][0][(nt + (mat >> 1)) * 8 + r][kk * 16 + (mat & 1) * 8]));
                mma_bf16(acc[nt], af, b[0], b[1]);
                mma_bf16(acc[nt + 1], af, b[2], b[3]);
                if (GATED) {
                    ldmatrix_x4(b, smem_addr(&Bs[stage][1][(nt + (mat >> 1)) * 8 + r][kk * 16 + (mat & 1) * 8]));
                    mma_bf16(acc2[nt], af, b[0], b[1]);
                    mma_bf16(acc2[nt + 1], af, b[2], b[3]);
                }
            }
        }
    }
    // The rows' weights (first half), then the gate.
    float w_lo = 1.0f, w_hi = 1.0f;
    if (GATED && p.weights != nullptr) {
        const int lo = r0 + warp * 16 + g, hi = lo + 8;
        if (lo < r_end) w_lo = p.weights[p.pair_at[lo]];
        if (hi < r_end) w_hi = p.weights[p.pair_at[hi]];
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e4 = 0; e4 < 4; ++e4) {
            const int row = r0 + warp * 16 + g + (e4 >= 2 ? 8 : 0), n = n0 + nt * 8 + 2 * t + (e4 & 1);
            if (row >= r_end || n >= p.N) continue;
            if (GATED) {
                const float w = e4 >= 2 ? w_hi : w_lo;
                static_cast<B16*>(p.out)[(size_t)row * p.ldo + n] = __float2bfloat16_rn(lb_gated_pair(w * acc[nt][e4], w * acc2[nt][e4], p.act, p.alpha, p.limit));
            } else {
                static_cast<float*>(p.out)[(size_t)row * p.ldo + n] = acc[nt][e4];
            }
        }
}

template <bool GATED>
int launch_product_mma(const ProductArgs& p, int n_pairs, cudaStream_t s) {
    const int tiles = (n_pairs + kMM - 1) / kMM + min(p.E, n_pairs);
    const dim3 grid((unsigned)tiles, (unsigned)((p.N + kMN - 1) / kMN)), block(128);
    LB_CHECK_CUDA(lb_launch_overlapped(expert_product_mma_kernel<GATED>, grid, block, 0, s, p));
    return LB_OK;
}

bool mma_takes(const ProductArgs& p) {
    return p.K % 8 == 0 && p.lda % 8 == 0 && p.expert_stride % 8 == 0 && ((uintptr_t)p.a & 15) == 0 && ((uintptr_t)p.w & 15) == 0;
}

// ---------------------------------------------------------------- the same products for a few pairs (bfloat16)
// A decode step brings a pair or two an expert: a 64-row tile would be one row of work behind a long loop over K.  Here a warp takes
// one pair and F of its expert's output features (both matrices' where GATED), K split over its lanes in 16-byte loads.  Nothing
// waits on anything it need not: the expert of a pair is found by one round of loads (every lane an offset, a ballot), the input row
// is read by the lanes themselves, and 1,024 values of K of every row a warp reads travel together (cp.async, 20 pieces of 16 bytes a
// lane in flight, whatever the compiler makes of the loop), so a launch is two round trips to memory and the stream of the experts'
// matrices, with every SM taking part.  Sums are 32-bit in a fixed order; alignment as the tensor-core form's.
template <bool GATED>
__global__ void __launch_bounds__(128) expert_product_rows_kernel(ProductArgs p) {
    using B16 = __nv_bfloat16;
    constexpr int F = GATED ? 2 : 4, kAhead = 4;
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n0 = (blockIdx.y * 4 + warp) * F;
    if (n0 >= p.N) return;
    // The expert whose rows hold r: as many experts after the first start at or before r.
    int e = 0;
    for (int base = 1; base < p.E; base += 32) {
        const bool at_or_before = base + lane < p.E && p.offsets[base + lane] <= r;
        e += __popc(__ballot_sync(0xffffffffu, at_or_before));
    }
    const int pair = p.pair_at[r];
    const uint4* a_row = reinterpret_cast<const uint4*>(static_cast<const B16*>(p.a) + (size_t)(GATED ? pair / p.top : r) * p.lda);
    const B16* W = static_cast<const B16*>(p.w) + (size_t)e * p.expert_stride;
    const int k8 = p.K / 8;
    const uint4* w[GATED ? 2 * F : F];
#pragma unroll
    for (int f = 0; f < F; ++f) {
        const int n = min(n0 + f, p.N - 1);                   // past the last feature: the last one again, not stored
        w[f] = reinterpret_cast<const uint4*>(W + (size_t)n * p.K);
        if (GATED) w[F + f] = reinterpret_cast<const uint4*>(W + (size_t)(p.N + n) * p.K);
    }
    constexpr int M = GATED ? 2 * F : F;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
    auto dot8 = [](const uint4& wv, const uint4& av, float sum) {
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 wf = __bfloat1622float2(wp[q]), af = __bfloat1622float2(ap[q]);
            sum = fmaf(wf.x, af.x, sum);
            sum = fmaf(wf.y, af.y, sum);
        }
        return sum;
    };
    // Every lane copies its own 16-byte pieces into places of its own and reads them back after its own wait: no barrier.
    __shared__ __align__(16) uint4 ahead[4][kAhead][M + 1][32];
    for (int i0 = lane; i0 < k8; i0 += 32 * kAhead) {
#pragma unroll
        for (int s = 0; s < kAhead; ++s) {
            const int i = i0 + 32 * s;
            const bool in = i < k8;                           // past the end: zeros
            cp_async16(&ahead[warp][s][M][lane], a_row + (in ? i : 0), in);
#pragma unroll
            for (int m = 0; m < M; ++m) cp_async16(&ahead[warp][s][m][lane], w[m] + (in ? i : 0), in);
        }
        cp_async_commit();
        cp_async_wait<0>();
#pragma unroll
        for (int s = 0; s < kAhead; ++s) {
            const uint4 av = ahead[warp][s][M][lane];
#pragma unroll
            for (int m = 0; m < M; ++m) acc[m] = dot8(ahead[warp][s][m][lane], av, acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    if (lane != 0) return;
    const float scale = GATED && p.weights != nullptr ? p.weights[pair] : 1.0f;
#pragma unroll
    for (int f = 0; f < F; ++f) {
        const int n = n0 + f;
        if (n >= p.N) break;
        if (GATED) static_cast<B16*>(p.out)[(size_t)r * p.ldo + n] = __float2bfloat16_rn(lb_gated_pair(scale * acc[f], scale * acc[F + f], p.act, p.alpha, p.limit));
        else static_cast<float*>(p.out)[(size_t)r * p.ldo + n] = acc[f];
    }
}

constexpr int kFewPairs = 64;

template <bool GATED>
int launch_product_rows(const ProductArgs& p, int n_pairs, cudaStream_t s) {
    const int features = 4 * (GATED ? 2 : 4);       // a block's four warps, F features each
    const dim3 grid((unsigned)n_pairs, (unsigned)((p.N + features - 1) / features)), block(128);
    LB_CHECK_CUDA(lb_launch_overlapped(expert_product_rows_kernel<GATED>, grid, block, 0, s, p));
    return LB_OK;
}

__global__ void expert_combine_kernel(float* __restrict__ x, int64_t ldx, const float* __restrict__ y, int64_t ldy, const int32_t* __restrict__ place,
                                      int n_rows, int width, int top, const float* __restrict__ weights, int overwrite) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const long total = (long)n_rows * width;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long t = i / width;
        const int c = (int)(i - t * width);
        float acc = 0.0f;
        if (weights != nullptr)
            for (int k = 0; k < top; ++k) acc = fmaf(weights[t * top + k], y[(size_t)place[t * top + k] * ldy + c], acc);
        else
            for (int k = 0; k < top; ++k) acc += y[(size_t)place[t * top + k] * ldy + c];
        if (overwrite) x[(size_t)t * ldx + c] = acc;
        else x[(size_t)t * ldx + c] += acc;
    }
}

template <typename T, bool GATED>
int launch_product(const ProductArgs& p, int n_pairs, cudaStream_t s) {
    // Row tiles of 16 where the pairs are few (a decode step), of 64 otherwise; no more tiles than pairs / tile + experts.
    const bool small = n_pairs <= 16 * p.E;
    const int BM = small ? 16 : 64;
    const int tiles = (n_pairs + BM - 1) / BM + min(p.E, n_pairs);
    const dim3 grid((unsigned)tiles, (unsigned)((p.N + kBN - 1) / kBN)), block(256);
    if (small) LB_CHECK_CUDA(lb_launch_overlapped(expert_product_kernel<T, 1, GATED>, grid, block, 0, s, p));
    else LB_CHECK_CUDA(lb_launch_overlapped(expert_product_kernel<T, 4, GATED>, grid, block, 0, s, p));
    return LB_OK;
}

}  // namespace

extern "C" int lb_router_topk(int dtype, const void* h, int64_t ldh, const void* router, int32_t* ids, float* weights, int n_rows, int n_experts,
                              int width, int top, int softmax, int renormalise, void* stream) {
    return lb_router_topk_biased(dtype, h, ldh, router, nullptr, ids, weights, n_rows, n_experts, width, top, softmax, renormalise, stream);
}

extern "C" int lb_router_topk_biased(int dtype, const void* h, int64_t ldh, const void* router, const float* bias, int32_t* ids, float* weights, int n_rows,
                                     int n_experts, int width, int top, int softmax, int renormalise, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && n_experts > 0 && width > 0 && top > 0 && top <= n_experts && n_experts <= 4096, "router: top %d of %d experts", top, n_experts);
    if (n_rows == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const size_t smem = (size_t)n_experts * sizeof(float);
    const int threads = 32 * max(1, min(16, n_experts));       // a warp per expert, up to sixteen
    if (dtype == LB_F32)
        LB_CHECK_CUDA(lb_launch_overlapped(router_topk_kernel<float>, dim3(n_rows), dim3(threads), smem, s, (const float*)h, ldh, (const float*)router, ids, weights,
                                           n_experts, width, top, softmax, renormalise, bias));
    else if (dtype == LB_BF16)
        LB_CHECK_CUDA(lb_launch_overlapped(router_topk_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, s, (const __nv_bfloat16*)h, ldh,
                                           (const __nv_bfloat16*)router, ids, weights, n_experts, width, top, softmax, renormalise, bias));
    else return lb_fail(LB_ERR_INVALID_ARGUMENT, "router: unknown dtype %d", dtype);
    return LB_OK;
}

extern "C" int lb_expert_plan(const int32_t* ids, int n_pairs, int n_experts, int32_t* offsets, int32_t* place, int32_t* pair_at, void* stream) {
    LB_CHECK_ARG(n_pairs >= 0 && n_experts > 0 && n_experts <= 4096, "expert plan: bad sizes");
    const int threads = 32 * max(1, min(32, n_experts));
    const int staged = (size_t)(n_experts + 1 + n_pairs) * sizeof(int) <= 48 * 1024 ? 1 : 0;
    LB_CHECK_CUDA(lb_launch_overlapped(expert_plan_kernel, dim3(1), dim3(threads), (size_t)(n_experts + 1 + (staged ? n_pairs : 0)) * sizeof(int),
                                       static_cast<cudaStream_t>(stream), const_cast<int32_t*>(ids), n_pairs, n_experts, offsets, place, pair_at, staged,
                                       (const int32_t*)nullptr, (const int32_t*)nullptr, 0, 1, (float*)nullptr));
    return LB_OK;
}

extern "C" int lb_expert_plan_table(const int32_t* tokens, const int32_t* table, int vocab, int top, int32_t* ids, float* weights, int n_rows, int n_experts,
                                    int32_t* offsets, int32_t* place, int32_t* pair_at, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && n_experts > 0 && n_experts <= 4096 && top > 0 && vocab > 0, "expert plan by table: bad sizes");
    const int n_pairs = n_rows * top;
    const int threads = 32 * max(1, min(32, n_experts));
    const int staged = (size_t)(n_experts + 1 + n_pairs) * sizeof(int) <= 48 * 1024 ? 1 : 0;
    LB_CHECK_CUDA(lb_launch_overlapped(expert_plan_kernel, dim3(1), dim3(threads), (size_t)(n_experts + 1 + (staged ? n_pairs : 0)) * sizeof(int),
                                       static_cast<cudaStream_t>(stream), ids, n_pairs, n_experts, offsets, place, pair_at, staged, tokens, table, vocab, top,
                                       weights));
    return LB_OK;
}

// Tests compare the two bfloat16 paths: non-zero keeps every product on the 32-bit units.
static int lb_expert_product_plain_only = 0;
extern "C" int lb_expert_product_set_plain(int on) {
    lb_expert_product_plain_only = on;
    return LB_OK;
}

extern "C" int lb_expert_product(int dtype, int gated, const void* a, int64_t lda, const void* w, int64_t expert_stride, const int32_t* offsets,
                                 const int32_t* pair_at, const float* weights, void* out, int64_t ldo, int n_pairs, int n_experts, int n, int k, int top,
                                 int act, void* stream) {
    return lb_expert_product_kind(dtype, gated, a, lda, w, expert_stride, offsets, pair_at, weights, out, ldo, n_pairs, n_experts, n, k, top, act, 0.0f, 0.0f,
                                  stream);
}

extern "C" int lb_expert_product_kind(int dtype, int gated, const void* a, int64_t lda, const void* w, int64_t expert_stride, const int32_t* offsets,
                                      const int32_t* pair_at, const float* weights, void* out, int64_t ldo, int n_pairs, int n_experts, int n, int k, int top,
                                      int act, float alpha, float limit, void* stream) {
    LB_CHECK_ARG(n_pairs >= 0 && n_experts > 0 && n > 0 && k > 0 && top > 0 && act >= 0 && act <= LB_GATE_CAPPED, "expert product: bad sizes");
    if (n_pairs == 0) return LB_OK;
    ProductArgs p{a, lda, w, expert_stride, offsets, pair_at, weights, out, ldo, n_experts, n, k, top, act, alpha, limit};
    auto s = static_cast<cudaStream_t>(stream);
    if (dtype == LB_F32) return gated ? launch_product<float, true>(p, n_pairs, s) : launch_product<float, false>(p, n_pairs, s);
    if (dtype == LB_BF16 && mma_takes(p) && !lb_expert_product_plain_only && n_pairs <= kFewPairs)
        return gated ? launch_product_rows<true>(p, n_pairs, s) : launch_product_rows<false>(p, n_pairs, s);
    if (dtype == LB_BF16 && mma_takes(p) && !lb_expert_product_plain_only)
        return gated ? launch_product_mma<true>(p, n_pairs, s) : launch_product_mma<false>(p, n_pairs, s);
    if (dtype == LB_BF16) return gated ? launch_product<__nv_bfloat16, true>(p, n_pairs, s) : launch_product<__nv_bfloat16, false>(p, n_pairs, s);
    return lb_fail(LB_ERR_INVALID_ARGUMENT, "expert product: unknown dtype %d", dtype);
}

extern "C" int lb_expert_combine(float* x, int64_t ldx, const float* y, int64_t ldy, const int32_t* place, int n_rows, int width, int top, void* stream) {
    return lb_expert_combine_weighted(x, ldx, y, ldy, place, nullptr, n_rows, width, top, stream);
}

extern "C" int lb_expert_combine_weighted(float* x, int64_t ldx, const float* y, int64_t ldy, const int32_t* place, const float* weights, int n_rows,
                                          int width, int top, void* stream) {
    return lb_expert_combine_into(x, ldx, y, ldy, place, weights, n_rows, width, top, 0, stream);
}

extern "C" int lb_expert_combine_into(float* x, int64_t ldx, const float* y, int64_t ldy, const int32_t* place, const float* weights, int n_rows,
                                      int width, int top, int overwrite, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && width > 0 && top > 0, "expert combine: bad sizes");
    if (n_rows == 0) return LB_OK;
    const long total = (long)n_rows * width;
    const int blocks = (int)min((total + 255) / 256, (long)148 * 16);
    LB_CHECK_CUDA(lb_launch_overlapped(expert_combine_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), x, ldx, y, ldy, place, n_rows, width,
                                       top, weights, overwrite));
    return LB_OK;
}
