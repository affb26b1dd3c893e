// Attention over latent cache rows on the tensor cores (bfloat16, mma.sync m16n8k16, 32-bit accumulation).
//
// The same computation as lb_latent_attention (latent_attention.cu): wide queries [T, H, rank + rot] against cache
// rows [rank | rot], softmax in 32-bit, the weighted sum of the rows' first `rank` values out.  All heads share the
// rows, so a block takes M = 16 * MT query rows that are (token, head) pairs of one request, HB <= 16 heads of TOK = M / HB
// consecutive tokens, and walks the visible keys in tiles of 32:
//   scores   warp w makes the 8 keys 8w .. 8w + 7 of the tile for all M rows, k over rank + rot;
//   softmax  row maxima and sums meet in shared memory; the weights go there too, as bfloat16;
//   sums     warp w owns a quarter of the rank values of all M rows and adds weights x rows to them.
// Key tiles arrive by cp.async, one tile ahead.  A request's keys may be split over several blocks (decode steps of
// few requests); the parts are merged by a second kernel.  Shapes: rank a multiple of 32 from a built list, rot a
// multiple of 16; anything else stays with the 32-bit kernel.
#include "api.h"
#include "common.cuh"

#include <math_constants.h>

namespace {

using bf16 = __nv_bfloat16;
constexpr int kKeys = 32;
constexpr int kPStride = kKeys + 8;          // weights' row stride in shared memory (elements): 80 bytes, conflict-free for ldmatrix

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// What a (token, head)'s sums are multiplied by at the end.  Without extras 1 / l.  A head's sink adds exp(sink) to the divisor (it has no
// key and no value; `m`, the running maximum, is in the scores' base-2 scale); a gate multiplies the result by sigmoid(gate[t, head]).
struct HeadExtras {
    const float* sink;
    const float* gate;
    int64_t ldg;
};
__device__ __forceinline__ float finish_factor(const HeadExtras& x, int t, int head, float m, float l) {
    float f = 1.0f;
    if (x.sink != nullptr) {
        const float sk = x.sink[head] * 1.4426950408889634f, top = fmaxf(m, sk);
        f = exp2f(m - top);
        l = l * f + exp2f(sk - top);
    }
    if (x.gate != nullptr) f *= 1.0f / (1.0f + expf(-x.gate[(size_t)t * x.ldg + head]));
    return f / l;
}

// MT: 16-row tiles of a block; RT: 8-column tiles of the rank values per warp (rank = 32 * RT).
template <int MT, int RT>
__global__ void __launch_bounds__(128)
latent_attention_mma_kernel(const bf16* __restrict__ wide, int64_t ldw, const bf16* __restrict__ cache, const int32_t* __restrict__ q_start,
                            const int32_t* __restrict__ n_past, const int32_t* __restrict__ block_table, int table_stride,
                            float* __restrict__ out, int64_t ldo, float* __restrict__ part_o, float* __restrict__ part_ml, int n_tokens,
                            int n_head, int rot, int page_size, float scale_log2, int window, int HB, int n_splits, HeadExtras extras) {
    constexpr int M = 16 * MT, RANK = 32 * RT;
    const int D = RANK + rot, DS = D + 8, chunks = D / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);               // [M][DS]
    bf16* ks = qs + (size_t)M * DS;                              // [2][kKeys][DS]
    bf16* ps = ks + (size_t)2 * kKeys * DS;                      // [M][kPStride]
    float* red_max = reinterpret_cast<float*>(ps + (size_t)M * kPStride);   // [4][M]
    float* red_sum = red_max + 4 * M;                            // [4][M]

    const int TOK = M / HB;                                      // rows beyond TOK * HB stay empty
    const int s = blockIdx.y, split = blockIdx.z % n_splits, hg = blockIdx.z / n_splits;
    const int qt = gridDim.x - 1 - blockIdx.x;                     // a request's last tiles see the most keys: they start first
    const int first = q_start[s] + qt * TOK;
    const int n_here = min(TOK, q_start[s + 1] - first);
    if (n_here <= 0) return;
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int p_first = n_past[s] + qt * TOK, p_last = p_first + n_here - 1;
    const int lo_min = window > 0 ? max(0, p_first - window + 1) : 0;
    const int32_t* table = block_table + (size_t)s * table_stride;

    // The block's tiles of keys, and this split's share of them.
    const int tile_lo = lo_min / kKeys, tile_hi = p_last / kKeys;
    const int per = (tile_hi - tile_lo + n_splits) / n_splits;
    const int my_lo = tile_lo + split * per, my_hi = min(tile_hi, my_lo + per - 1);

    auto load_tile = [&](int tile, int buf) {
        bf16* dst0 = ks + (size_t)buf * kKeys * DS;
        for (int key = warp; key < kKeys; key += 4) {
            const int j = tile * kKeys + key;
            bf16* dst = dst0 + (size_t)key * DS;
            if (j >= lo_min && j <= p_last) {
                const bf16* src = cache + ((size_t)table[j / page_size] * page_size + (j % page_size)) * D;
                for (int c = lane; c < chunks; c += 32) cp_async16(dst + c * 8, src + c * 8);
            } else {
                for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        cp_async_commit();
    };
    if (my_lo <= my_hi) load_tile(my_lo, 0);                     // on its way while the queries are staged
    // Queries: row r is token first + r / HB, head hg * HB + r % HB.
    for (int r = warp; r < M; r += 4) {
        const int tok = r / HB, head = hg * HB + r % HB;
        const bool valid = tok < n_here && head < n_head;
        const bf16* src = wide + (size_t)(first + min(tok, n_here - 1)) * ldw + (size_t)min(head, n_head - 1) * D;
        for (int c = lane; c < chunks; c += 32) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (valid) v = *reinterpret_cast<const uint4*>(src + c * 8);
            *reinterpret_cast<uint4*>(qs + (size_t)r * DS + c * 8) = v;
        }
    }

    float o[MT][RT][4];
    float m_run[MT][2], l_run[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        m_run[mt][0] = m_run[mt][1] = -CUDART_INF_F;
        l_run[mt][0] = l_run[mt][1] = 0.0f;
#pragma unroll
        for (int nt = 0; nt < RT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[mt][nt][i] = 0.0f;
    }

    for (int tile = my_lo; tile <= my_hi; ++tile) {
        const int buf = (tile - my_lo) & 1;
        cp_async_wait_all();
        __syncthreads();                                        // the tile (and, first time, the queries) is there; the step before is over
        if (tile < my_hi) load_tile(tile + 1, buf ^ 1);
        const bf16* kt = ks + (size_t)buf * kKeys * DS;

        // ---- scores of keys 8w .. 8w + 7 for all rows
        float sc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) sc[mt][i] = 0.0f;
        for (int kk = 0; kk < D; kk += 16) {
            uint32_t b[2];
            ldmatrix_x2(b, kt + (size_t)(8 * warp + (lane & 7)) * DS + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t a[4];
                ldmatrix_x4(a, qs + (size_t)(mt * 16 + (lane & 15)) * DS + kk + (lane >> 4) * 8);
                mma_bf16(sc[mt], a, b);
            }
        }
        // ---- mask, row maxima over the warp's keys
        const int j0 = tile * kKeys + 8 * warp + 2 * t4;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = mt * 16 + g + 8 * half, tok = row / HB;
                const int p_row = p_first + tok, lo_row = window > 0 ? max(0, p_row - window + 1) : 0;
                float mx = -CUDART_INF_F;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = j0 + e;
                    const bool seen = tok < n_here && j >= lo_row && j <= p_row;
                    const float v = seen ? sc[mt][2 * half + e] * scale_log2 : -CUDART_INF_F;
                    sc[mt][2 * half + e] = v;
                    mx = fmaxf(mx, v);
                }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                if (t4 == 0) red_max[warp * M + row] = mx;
            }
        __syncthreads();
        // ---- weights (to shared memory as bfloat16), row sums, rescaling of what has been summed so far
        float corr[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = mt * 16 + g + 8 * half;
                const float m_tile = fmaxf(fmaxf(red_max[row], red_max[M + row]), fmaxf(red_max[2 * M + row], red_max[3 * M + row]));
                const float m_new = fmaxf(m_run[mt][half], m_tile);
                const bool none = m_new == -CUDART_INF_F;                   // nothing seen yet in this row
                corr[mt][half] = none ? 1.0f : exp2f(m_run[mt][half] - m_new);
                const float p0 = none ? 0.0f : exp2f(sc[mt][2 * half] - m_new), p1 = none ? 0.0f : exp2f(sc[mt][2 * half + 1] - m_new);
                *reinterpret_cast<__nv_bfloat162*>(ps + (size_t)row * kPStride + 8 * warp + 2 * t4) = __floats2bfloat162_rn(p0, p1);
                float sum = p0 + p1;
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if (t4 == 0) red_sum[warp * M + row] = sum;
                m_run[mt][half] = m_new;
            }
        __syncthreads();
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = mt * 16 + g + 8 * half;
                l_run[mt][half] = l_run[mt][half] * corr[mt][half] + ((red_sum[row] + red_sum[M + row]) + (red_sum[2 * M + row] + red_sum[3 * M + row]));
            }
#pragma unroll
            for (int nt = 0; nt < RT; ++nt) {
                o[mt][nt][0] *= corr[mt][0];
                o[mt][nt][1] *= corr[mt][0];
                o[mt][nt][2] *= corr[mt][1];
                o[mt][nt][3] *= corr[mt][1];
            }
        }
        // ---- weights x rows, this warp's quarter of the rank values
#pragma unroll
        for (int k2 = 0; k2 < kKeys; k2 += 16) {
            uint32_t a[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(a[mt], ps + (size_t)(mt * 16 + (lane & 15)) * kPStride + k2 + (lane >> 4) * 8);
#pragma unroll
            for (int nt = 0; nt < RT; ++nt) {
                uint32_t b[2];
                ldmatrix_x2_trans(b, kt + (size_t)(k2 + (lane & 15)) * DS + (warp * RT + nt) * 8);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) mma_bf16(o[mt][nt], a[mt], b);
            }
        }
    }

    // ---- out: normalised, or (keys split over blocks) the part with its maximum and sum
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = mt * 16 + g + 8 * half, tok = row / HB, head = hg * HB + row % HB;
            if (tok >= n_here || head >= n_head) continue;
            const int t = first + tok;
            if (n_splits == 1) {
                const float inv = finish_factor(extras, t, head, m_run[mt][half], l_run[mt][half]);
                float* dst = out + (size_t)t * ldo + (size_t)head * RANK + warp * RT * 8 + 2 * t4;
#pragma unroll
                for (int nt = 0; nt < RT; ++nt)
                    *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[mt][nt][2 * half] * inv, o[mt][nt][2 * half + 1] * inv);
            } else {
                const size_t at = ((size_t)split * n_tokens + t) * n_head + head;
                float* dst = part_o + at * RANK + warp * RT * 8 + 2 * t4;
#pragma unroll
                for (int nt = 0; nt < RT; ++nt) *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[mt][nt][2 * half], o[mt][nt][2 * half + 1]);
                if (warp == 0 && t4 == 0) {
                    part_ml[at * 2] = m_run[mt][half];
                    part_ml[at * 2 + 1] = l_run[mt][half];
                }
            }
        }
}

// The same attention for steps with runs of tokens and latents of up to 256 values: a block takes 64 rows, every warp 16 of them with
// all 32 keys of a tile and all rank values.  Maxima and sums stay inside the warp (four lanes share a row), the weights pass from the
// score accumulators straight into the next product's operand registers, and the only block-wide meeting is the change of key tiles.
// N8: 8-column tiles of the rank values (rank = 8 * N8, N8 even).
template <int N8, typename TO>
__global__ void __launch_bounds__(128)
latent_attention_rows_kernel(const bf16* __restrict__ wide, int64_t ldw, const bf16* __restrict__ cache, const int32_t* __restrict__ q_start,
                             const int32_t* __restrict__ n_past, const int32_t* __restrict__ block_table, int table_stride, TO* __restrict__ out,
                             int64_t ldo, int n_head, int rot, int page_size, float scale_log2, int window, int HB, HeadExtras extras) {
    constexpr int M = 64, RANK = 8 * N8;
    const int D = RANK + rot, DS = D + 8, chunks = D / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);               // [M][DS]
    bf16* ks = qs + (size_t)M * DS;                              // [2][kKeys][DS]
    const int TOK = M / HB;                                      // rows beyond TOK * HB stay empty
    const int s = blockIdx.y, hg = blockIdx.z;
    const int qt = gridDim.x - 1 - blockIdx.x;                     // a request's last tiles see the most keys: they start first
    const int first = q_start[s] + qt * TOK;
    const int n_here = min(TOK, q_start[s + 1] - first);
    if (n_here <= 0) return;
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int p_first = n_past[s] + qt * TOK, p_last = p_first + n_here - 1;
    const int lo_min = window > 0 ? max(0, p_first - window + 1) : 0;
    const int32_t* table = block_table + (size_t)s * table_stride;
    const int tile_lo = lo_min / kKeys, tile_hi = p_last / kKeys;

    auto load_tile = [&](int tile, int buf) {
        bf16* dst0 = ks + (size_t)buf * kKeys * DS;
        for (int key = warp; key < kKeys; key += 4) {
            const int j = tile * kKeys + key;
            bf16* dst = dst0 + (size_t)key * DS;
            if (j >= lo_min && j <= p_last) {
                const bf16* src = cache + ((size_t)table[j / page_size] * page_size + (j % page_size)) * D;
                for (int c = lane; c < chunks; c += 32) cp_async16(dst + c * 8, src + c * 8);
            } else {
                for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        cp_async_commit();
    };
    load_tile(tile_lo, 0);                                        // on its way while the queries are staged
    for (int r = warp; r < M; r += 4) {
        const int tok = r / HB, head = hg * HB + r % HB;
        const bool valid = tok < n_here && head < n_head;
        const bf16* src = wide + (size_t)(first + min(tok, n_here - 1)) * ldw + (size_t)min(head, n_head - 1) * D;
        for (int c = lane; c < chunks; c += 32) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (valid) v = *reinterpret_cast<const uint4*>(src + c * 8);
            *reinterpret_cast<uint4*>(qs + (size_t)r * DS + c * 8) = v;
        }
    }

    // This thread's two rows (g and g + 8 of the warp's sixteen): their tokens' positions and first visible keys.
    int p_row[2], lo_row[2];
    bool live[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int tok = (warp * 16 + g + 8 * half) / HB;
        live[half] = tok < n_here;
        p_row[half] = p_first + tok;
        lo_row[half] = window > 0 ? max(0, p_row[half] - window + 1) : 0;
    }
    float o[N8][4];
#pragma unroll
    for (int nt = 0; nt < N8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[nt][i] = 0.0f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.0f, 0.0f};

    for (int tile = tile_lo; tile <= tile_hi; ++tile) {
        const int buf = (tile - tile_lo) & 1;
        cp_async_wait_all();
        __syncthreads();
        if (tile < tile_hi) load_tile(tile + 1, buf ^ 1);
        const bf16* kt = ks + (size_t)buf * kKeys * DS;

        float sc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) sc[nt][i] = 0.0f;
#pragma unroll 4
        for (int kk = 0; kk < D; kk += 16) {
            uint32_t a[4];
            ldmatrix_x4(a, qs + (size_t)(warp * 16 + (lane & 15)) * DS + kk + (lane >> 4) * 8);
#pragma unroll
            for (int pair = 0; pair < 2; ++pair) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + (size_t)(pair * 16 + ((lane >> 4) & 1) * 8 + (lane & 7)) * DS + kk + ((lane >> 3) & 1) * 8);
                const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
                mma_bf16(sc[2 * pair], a, b0);
                mma_bf16(sc[2 * pair + 1], a, b1);
            }
        }
        float corr[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float mx = -CUDART_INF_F;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = tile * kKeys + nt * 8 + 2 * t4 + e;
                    const bool seen = live[half] && j >= lo_row[half] && j <= p_row[half];
                    const float v = seen ? sc[nt][2 * half + e] * scale_log2 : -CUDART_INF_F;
                    sc[nt][2 * half + e] = v;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[half], mx);
            const bool none = m_new == -CUDART_INF_F;
            corr[half] = none ? 1.0f : exp2f(m_run[half] - m_new);
            float sum = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float p = none ? 0.0f : exp2f(sc[nt][2 * half + e] - m_new);
                    sc[nt][2 * half + e] = p;
                    sum += p;
                }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l_run[half] = l_run[half] * corr[half] + sum;
            m_run[half] = m_new;
        }
#pragma unroll
        for (int nt = 0; nt < N8; ++nt) {
            o[nt][0] *= corr[0];
            o[nt][1] *= corr[0];
            o[nt][2] *= corr[1];
            o[nt][3] *= corr[1];
        }
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) {
            const uint32_t a[4] = {pack_bf16(sc[2 * k2][0], sc[2 * k2][1]), pack_bf16(sc[2 * k2][2], sc[2 * k2][3]),
                                   pack_bf16(sc[2 * k2 + 1][0], sc[2 * k2 + 1][1]), pack_bf16(sc[2 * k2 + 1][2], sc[2 * k2 + 1][3])};
#pragma unroll
            for (int np = 0; np < N8 / 2; ++np) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, kt + (size_t)(k2 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * DS + np * 16 + ((lane >> 4) & 1) * 8);
                const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
                mma_bf16(o[2 * np], a, b0);
                mma_bf16(o[2 * np + 1], a, b1);
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = warp * 16 + g + 8 * half, tok = row / HB, head = hg * HB + row % HB;
        if (tok >= n_here || head >= n_head) continue;
        const float inv = finish_factor(extras, first + tok, head, m_run[half], l_run[half]);
        TO* dst = out + (size_t)(first + tok) * ldo + (size_t)head * RANK + 2 * t4;
#pragma unroll
        for (int nt = 0; nt < N8; ++nt) {
            if constexpr (sizeof(TO) == 4) *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][2 * half] * inv, o[nt][2 * half + 1] * inv);
            else *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) = __floats2bfloat162_rn(o[nt][2 * half] * inv, o[nt][2 * half + 1] * inv);
        }
    }
}

template <int N8, typename TO>
int launch_rows(const void* wide, int64_t ldw, const void* cache, const int32_t* q_start, const int32_t* n_past, const int32_t* block_table, int table_stride,
                TO* out, int64_t ldo, int n_seq, int max_q_len, int n_head, int rot, int page_size, float scale, int window, HeadExtras extras,
                cudaStream_t s) {
    // Up to sixteen heads of a token side by side (more heads: groups of equal size), then the next tokens.
    const int groups = (n_head + 15) / 16, HB = (n_head + groups - 1) / groups, TOK = 64 / HB, DS = 8 * N8 + rot + 8;
    const size_t smem = (size_t)(64 + 2 * kKeys) * DS * sizeof(bf16);
    if (smem > 48 * 1024) LB_CHECK_CUDA(cudaFuncSetAttribute(latent_attention_rows_kernel<N8, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const dim3 grid((max_q_len + TOK - 1) / TOK, n_seq, (n_head + HB - 1) / HB);
    LB_CHECK_CUDA(lb_launch_overlapped(latent_attention_rows_kernel<N8, TO>, grid, dim3(128), smem, s, (const bf16*)wide, ldw, (const bf16*)cache, q_start, n_past,
                                       block_table, table_stride, out, ldo, n_head, rot, page_size, scale * 1.4426950408889634f, window, HB, extras));
    return LB_OK;
}

// out[t, h, :] = sum_s 2^(m_s - m) o_s / sum_s 2^(m_s - m) l_s over the parts, in their order.
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, float* __restrict__ out, int64_t ldo,
                                    int n_tokens, int n_head, int rank, int n_splits, HeadExtras extras) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x, h = blockIdx.y;
    float m = -CUDART_INF_F;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(((size_t)s * n_tokens + t) * n_head + h) * 2]);
    float l = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
        const size_t at = ((size_t)s * n_tokens + t) * n_head + h;
        const float ms = part_ml[at * 2];
        if (ms != -CUDART_INF_F) l += exp2f(ms - m) * part_ml[at * 2 + 1];
    }
    const float inv = finish_factor(extras, t, h, m, l);
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const size_t at = ((size_t)s * n_tokens + t) * n_head + h;
            const float ms = part_ml[at * 2];
            if (ms != -CUDART_INF_F) acc = fmaf(exp2f(ms - m), part_o[at * rank + d], acc);
        }
        out[(size_t)t * ldo + (size_t)h * rank + d] = acc * inv;
    }
}

// C[t, h * c_head + n] = sum_k A[t, h * a_head + k] * B[h * b_head + k * b_k + n * b_n]: the products per head around the attention
// (the keys' maps moved onto the queries; the values' maps on the attended latents) on the tensor cores.  A is float (rounded to
// bfloat16 as it is staged), B and C bfloat16.  A block makes 64 rows x 64 columns of one head, a warp 16 of the rows; K in chunks of 32.
// KN: B's rows run along n (b_n = 1), else along k (b_k = 1).  KC: K in chunks of that many (64; 128 for steps of few rows, whose
// blocks then make fewer round trips to memory).  A is float or bfloat16.
template <bool KN, int KC, typename TA>
__global__ void __launch_bounds__(128)
head_matmul_mma_kernel(const TA* __restrict__ A, int64_t lda, int64_t a_head, const bf16* __restrict__ B, int64_t b_head, int64_t b_k, int64_t b_n,
                       bf16* __restrict__ C, int64_t ldc, int64_t c_head, int M, int N, int K) {
    __shared__ __align__(16) bf16 As[64][KC + 8];
    __shared__ __align__(16) bf16 Bs[KN ? KC : 64][KN ? 72 : KC + 8];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int h = blockIdx.z, m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const TA* a = A + (size_t)h * a_head;
    const bf16* b = B + (size_t)h * b_head;
    float acc[8][4] = {};
    for (int k0 = 0; k0 < K; k0 += KC) {
        for (int idx = threadIdx.x; idx < 64 * (KC / 4); idx += 128) {      // 64 rows x groups of four values
            const int r = idx / (KC / 4), k = (idx % (KC / 4)) * 4;
            if constexpr (sizeof(TA) == 4) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (m0 + r < M && k0 + k < K) v = *reinterpret_cast<const float4*>(a + (size_t)(m0 + r) * lda + k0 + k);
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                *reinterpret_cast<uint2*>(&As[r][k]) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            } else {
                uint2 v = make_uint2(0u, 0u);
                if (m0 + r < M && k0 + k < K) v = *reinterpret_cast<const uint2*>(a + (size_t)(m0 + r) * lda + k0 + k);
                *reinterpret_cast<uint2*>(&As[r][k]) = v;
            }
        }
        if (KN) {
            for (int idx = threadIdx.x; idx < KC * 8; idx += 128) {         // k rows x 8 pieces of eight n
                const int k = idx >> 3, n = (idx & 7) * 8;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (k0 + k < K && n0 + n < N) v = *reinterpret_cast<const uint4*>(b + (size_t)(k0 + k) * b_k + n0 + n);
                *reinterpret_cast<uint4*>(&Bs[k][n]) = v;
            }
        } else {
            for (int idx = threadIdx.x; idx < 64 * (KC / 8); idx += 128) {  // 64 n rows x pieces of eight k
                const int n = idx / (KC / 8), k = (idx % (KC / 8)) * 8;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (n0 + n < N && k0 + k < K) v = *reinterpret_cast<const uint4*>(b + (size_t)(n0 + n) * b_n + k0 + k);
                *reinterpret_cast<uint4*>(&Bs[n][k]) = v;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < KC; kk += 16) {
            if (k0 + kk >= K) break;
            uint32_t af[4];
            ldmatrix_x4(af, &As[warp * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                uint32_t bfr[2];
                if (KN) ldmatrix_x2_trans(bfr, &Bs[kk + (lane & 15)][nt * 8]);
                else ldmatrix_x2(bfr, &Bs[nt * 8 + (lane & 7)][kk + ((lane >> 3) & 1) * 8]);
                mma_bf16(acc[nt], af, bfr);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = m0 + warp * 16 + g + 8 * half;
        if (r >= M) continue;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int n = n0 + nt * 8 + 2 * t4;
            if (n < N) *reinterpret_cast<__nv_bfloat162*>(C + (size_t)r * ldc + (size_t)h * c_head + n) = __floats2bfloat162_rn(acc[nt][2 * half], acc[nt][2 * half + 1]);
        }
    }
}

size_t mma_smem_bytes(int m, int rank, int rot) {
    const int DS = rank + rot + 8;
    return ((size_t)m * DS + (size_t)2 * kKeys * DS + (size_t)m * kPStride) * sizeof(bf16) + (size_t)8 * m * sizeof(float);
}

template <int MT, int RT>
int launch_mma(const void* wide, int64_t ldw, const void* cache, const int32_t* q_start, const int32_t* n_past, const int32_t* block_table,
               int table_stride, float* out, int64_t ldo, float* part_o, float* part_ml, int n_tokens, int n_seq, int max_q_len, int n_head, int rot,
               int page_size, float scale, int window, int n_splits, bool merge_parts, HeadExtras extras, cudaStream_t s) {
    constexpr int M = 16 * MT;
    const int groups = (n_head + 15) / 16, HB = (n_head + groups - 1) / groups, TOK = M / HB;
    const size_t smem = mma_smem_bytes(M, 32 * RT, rot);
    if (smem > 48 * 1024) LB_CHECK_CUDA(cudaFuncSetAttribute(latent_attention_mma_kernel<MT, RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const dim3 grid((max_q_len + TOK - 1) / TOK, n_seq, ((n_head + HB - 1) / HB) * n_splits);
    LB_CHECK_CUDA(lb_launch_overlapped(latent_attention_mma_kernel<MT, RT>, grid, dim3(128), smem, s, (const bf16*)wide, ldw, (const bf16*)cache, q_start,
                                       n_past, block_table, table_stride, out, ldo, part_o, part_ml, n_tokens, n_head, rot, page_size,
                                       scale * 1.4426950408889634f, window, HB, n_splits, extras));
    if (n_splits > 1 && merge_parts)            // else the caller merges the parts itself (lb_latent_finish)
        LB_CHECK_CUDA(lb_launch_overlapped(latent_merge_kernel, dim3(n_tokens, n_head), dim3(128), 0, s, (const float*)part_o, (const float*)part_ml, out, ldo,
                                           n_tokens, n_head, 32 * RT, n_splits, extras));
    return LB_OK;
}

bool built_rank(int rank) {
    for (const int r : {32, 64, 96, 128, 192, 256, 384, 512})
        if (r == rank) return true;
    return false;
}

}  // namespace

// Everything the 16-byte loads and paired stores need: rows of four floats in A, pieces of eight values along B's rows, pairs in C.
extern "C" int lb_head_matmul_mma_supports(int64_t lda, int64_t a_head, int64_t b_head, int64_t b_k, int64_t b_n, int64_t ldc, int64_t c_head, int N, int K) {
    const bool kn = b_n == 1;
    if (!kn && b_k != 1) return 0;
    return lda % 4 == 0 && a_head % 4 == 0 && K % 4 == 0 && b_head % 8 == 0 && (kn ? b_k % 8 == 0 && N % 8 == 0 : b_n % 8 == 0 && K % 8 == 0) && ldc % 2 == 0 &&
                   c_head % 2 == 0 && N % 2 == 0 ? 1 : 0;
}

extern "C" int lb_head_matmul_mma(int a_dtype, const void* A, int64_t lda, int64_t a_head, const void* B, int64_t b_head, int64_t b_k, int64_t b_n, void* C, int64_t ldc,
                                  int64_t c_head, int M, int N, int K, int n_head, void* stream) {
    if (!lb_head_matmul_mma_supports(lda, a_head, b_head, b_k, b_n, ldc, c_head, N, K))
        return lb_fail(LB_ERR_UNSUPPORTED, "product per head on tensor cores: strides or sizes off its 16-byte pieces");
    LB_CHECK_ARG(M >= 0 && N > 0 && K > 0 && n_head > 0 && n_head <= 65535, "product per head: bad sizes M=%d N=%d K=%d heads=%d", M, N, K, n_head);
    if (M == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const dim3 grid((N + 63) / 64, (M + 63) / 64, n_head);
    LB_CHECK_ARG(a_dtype == LB_F32 || a_dtype == LB_BF16, "product per head: unknown dtype %d", a_dtype);
#define LB_HEADS(KN, KC)                                                                                                                                    \
    if (a_dtype == LB_F32)                                                                                                                                  \
        LB_CHECK_CUDA(lb_launch_overlapped(head_matmul_mma_kernel<KN, KC, float>, grid, dim3(128), 0, s, (const float*)A, lda, a_head, (const bf16*)B, b_head, b_k, \
                                           b_n, (bf16*)C, ldc, c_head, M, N, K));                                                                           \
    else                                                                                                                                                    \
        LB_CHECK_CUDA(lb_launch_overlapped(head_matmul_mma_kernel<KN, KC, bf16>, grid, dim3(128), 0, s, (const bf16*)A, lda, a_head, (const bf16*)B, b_head, b_k,  \
                                           b_n, (bf16*)C, ldc, c_head, M, N, K))
    if (b_n == 1) {
        if (M <= 64) { LB_HEADS(true, 128); }
        else { LB_HEADS(true, 64); }
    } else {
        if (M <= 64) { LB_HEADS(false, 128); }
        else { LB_HEADS(false, 64); }
    }
#undef LB_HEADS
    return LB_OK;
}

extern "C" int lb_latent_attention_mma_supports(int n_head, int rank, int rot, int page_size) {
    return n_head > 0 && built_rank(rank) && rot >= 0 && rot % 16 == 0 && page_size > 0 && mma_smem_bytes(32, rank, rot) <= 200 * 1024 ? 1 : 0;
}

extern "C" int lb_latent_attention_rows_supports(int n_head, int rank, int rot, int page_size) {
    return lb_latent_attention_mma_supports(n_head, rank, rot, page_size) && rank <= 256 && (size_t)(64 + 2 * kKeys) * (rank + rot + 8) * sizeof(bf16) <= 200 * 1024 ? 1 : 0;
}

// The 64-row kernel with the attended latents written as bfloat16 (what the values' product on the tensor cores reads).
extern "C" int lb_latent_attention_rows16(const void* wide, int64_t ldw, const void* cache, const int32_t* q_start, const int32_t* n_past,
                                          const int32_t* block_table, int table_stride, void* out, int64_t ldo, int n_tokens, int n_seq, int max_q_len,
                                          int n_head, int rank, int rot, int page_size, float scale, int window, void* stream) {
    return lb_latent_attention_rows16_ext(wide, ldw, cache, q_start, n_past, block_table, table_stride, out, ldo, n_tokens, n_seq, max_q_len, n_head, rank, rot,
                                          page_size, scale, window, nullptr, stream);
}

extern "C" int lb_latent_attention_rows16_ext(const void* wide, int64_t ldw, const void* cache, const int32_t* q_start, const int32_t* n_past,
                                              const int32_t* block_table, int table_stride, void* out, int64_t ldo, int n_tokens, int n_seq,
                                              int max_q_len, int n_head, int rank, int rot, int page_size, float scale, int window,
                                              const lb_latent_extras* x, void* stream) {
    const HeadExtras extras = x != nullptr ? HeadExtras{x->sink, x->gate, x->ldg} : HeadExtras{nullptr, nullptr, 0};
    if (!lb_latent_attention_rows_supports(n_head, rank, rot, page_size))
        return lb_fail(LB_ERR_UNSUPPORTED, "latent attention, 64 rows a block: rank %d, rot %d are not built", rank, rot);
    if (n_tokens == 0 || n_seq == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
#define LB_ROWS16(N8) \
    if (rank == 8 * N8) return launch_rows<N8, bf16>(wide, ldw, cache, q_start, n_past, block_table, table_stride, (bf16*)out, ldo, n_seq, max_q_len, n_head, rot, \
                                                     page_size, scale, window, extras, s)
    LB_ROWS16(4); LB_ROWS16(8); LB_ROWS16(12); LB_ROWS16(16); LB_ROWS16(24); LB_ROWS16(32);
#undef LB_ROWS16
    return lb_fail(LB_ERR_UNSUPPORTED, "latent attention, 64 rows a block: rank %d is not built", rank);
}

extern "C" int lb_latent_attention_mma(const void* wide, int64_t ldw, const void* cache, const int32_t* q_start, const int32_t* n_past,
                                       const int32_t* block_table, int table_stride, float* out, int64_t ldo, float* part_o, float* part_ml,
                                       int n_tokens, int n_seq, int max_q_len, int n_head, int rank, int rot, int page_size, float scale, int window,
                                       int n_splits, int merge_parts, void* stream) {
    return lb_latent_attention_mma_ext(wide, ldw, cache, q_start, n_past, block_table, table_stride, out, ldo, part_o, part_ml, n_tokens, n_seq, max_q_len,
                                       n_head, rank, rot, page_size, scale, window, n_splits, merge_parts, nullptr, stream);
}

// With extras: a part of split keys is left as it is (its maximum and sum travel with it); the sink and the gate act where the parts
// meet (the merge here, or lb_latent_finish_ext), or at once where the keys are not split.
extern "C" int lb_latent_attention_mma_ext(const void* wide, int64_t ldw, const void* cache, const int32_t* q_start, const int32_t* n_past,
                                           const int32_t* block_table, int table_stride, float* out, int64_t ldo, float* part_o, float* part_ml,
                                           int n_tokens, int n_seq, int max_q_len, int n_head, int rank, int rot, int page_size, float scale, int window,
                                           int n_splits, int merge_parts, const lb_latent_extras* x, void* stream) {
    const HeadExtras extras = x != nullptr ? HeadExtras{x->sink, x->gate, x->ldg} : HeadExtras{nullptr, nullptr, 0};
    if (!lb_latent_attention_mma_supports(n_head, rank, rot, page_size))
        return lb_fail(LB_ERR_UNSUPPORTED, "latent attention on tensor cores: rank %d, rot %d are not built", rank, rot);
    LB_CHECK_ARG(n_tokens >= 0 && n_seq >= 0 && max_q_len >= 0 && n_splits >= 1 && out != nullptr && (n_splits == 1 || (part_o != nullptr && part_ml != nullptr)),
                 "latent attention: bad sizes tokens=%d requests=%d splits=%d", n_tokens, n_seq, n_splits);
    if (n_tokens == 0 || n_seq == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    // Runs of tokens with a latent of up to 256 values: 64 rows a block, every warp with rows of its own.
    if (max_q_len > 1 && n_splits == 1 && rank <= 256 && (size_t)(64 + 2 * kKeys) * (rank + rot + 8) * sizeof(bf16) <= 200 * 1024) {
#define LB_ROWS(N8) \
    if (rank == 8 * N8) return launch_rows<N8, float>(wide, ldw, cache, q_start, n_past, block_table, table_stride, out, ldo, n_seq, max_q_len, n_head, rot, page_size, \
                                               scale, window, extras, s)
        LB_ROWS(4); LB_ROWS(8); LB_ROWS(12); LB_ROWS(16); LB_ROWS(24); LB_ROWS(32);
#undef LB_ROWS
    }
    // Else two 16-row tiles a block where a request brings several tokens; one otherwise.
    const bool two = max_q_len > 1;
#define LB_MMA(MT, RT) return launch_mma<MT, RT>(wide, ldw, cache, q_start, n_past, block_table, table_stride, out, ldo, part_o, part_ml, n_tokens, n_seq, \
                                                 max_q_len, n_head, rot, page_size, scale, window, n_splits, merge_parts != 0, extras, s)
#define LB_MMA_RANK(RT)            \
    if (rank == 32 * RT) {         \
        if (two) LB_MMA(2, RT);    \
        LB_MMA(1, RT);             \
    }
    LB_MMA_RANK(1) LB_MMA_RANK(2) LB_MMA_RANK(3) LB_MMA_RANK(4) LB_MMA_RANK(6) LB_MMA_RANK(8)
    LB_MMA_RANK(12) LB_MMA_RANK(16)
#undef LB_MMA_RANK
#undef LB_MMA
    return lb_fail(LB_ERR_UNSUPPORTED, "latent attention on tensor cores: rank %d is not built", rank);
}
