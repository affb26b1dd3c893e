// Mixers whose memory is a matrix per head, carried from token to token:
//     S_t = keep_t S_{t-1} + take_t k_t v_t^T,      o_t = S_t^T q_t (over a normaliser, where the mixer has one).
// Three kinds of (keep, take):
//   fixed decay    keep = decay[h], take = 1, no normaliser (retention);
//   token decay    keep = exp(f) with f <= 0 a number a token and head (the column zf holds f itself), take = 1, no normaliser:
//                  the recurrence of a state space whose step depends on the input, its step folded into the values;
//   gated          from two numbers a token and head, i (log of the input gate) and f (log of the forget gate), with a
//                  running maximum m that starts at 0: m_t = max(f_t + m_{t-1}, i_t), keep = exp(f_t + m_{t-1} - m_t),
//                  take = exp(i_t - m_t); a vector n_t follows the same recurrence with k alone, and
//                  o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6).  The gates arrive as pre-activations:
//                  i = cap tanh(zi / cap), f = logsigmoid(cap tanh(zf / cap)).
// Queries and keys may be rotated first (the first rot_dims values of a head in pairs (j, j + rot_dims/2), angle =
// position * freq[j]) and scaled.  `qk_share` heads in a row may share one query and one key row (a group's).  State,
// gates, angles and every sum are 32-bit.
//
// State of a request: [head][value tile][D x VT | D | 1] floats (S for the tile's VT value columns, n, m); every tile
// keeps its own n and m, so that the blocks of a launch share nothing.
//
// lb_matrix_memory_pieces is the form for long prompts: every piece a block of its own, in three launches (see the kernels).
// lb_matrix_memory walks a request's rows one after the other (a block per (request, head, value tile)); a decode step
// is one such row.  With `chunked` it does the same in pieces of 32 rows: inside a piece the rows' sums are products of
// small matrices (scores q_t . k_j weighted by the decay between j and t, then the values), and the state moves once per
// piece.
#include "api.h"
#include "common.cuh"

#include <math_constants.h>

namespace {

struct MemoryArgs {
    const float* q;            // [T, ld] rows, head h at columns (h / qk_share) * D
    const float* k;
    const float* v;            // head h at columns h * E
    const float* zi;           // [T, ld] gate pre-activations, head h at column h (gated kind), else null
    const float* zf;           // the same; without zi and without decay: the log of keep itself (token decay)
    int64_t ld;
    const float* decay;        // [H] (fixed kind), else null
    const float* freq;         // [rot_dims / 2] or null
    const int32_t* positions;  // [T]
    const int32_t* q_start;    // [S + 1]
    const int32_t* slots;      // [S]
    float* state;              // [slot][H][NV][D * VT + D + 1]
    int64_t slot_stride;       // floats per slot
    float* out;                // [T, ldo], head h at columns h * E
    int64_t ldo;
    int H, D, E, VT, NV, rot_dims;
    float q_scale, k_scale, cap;
    int qk_share;              // heads that read one query and key row; 1: every head its own
    int qkv_act;               // an activation on queries, keys and values as they arrive (0 sigmoid, 1 silu, 2 GELU tanh form, 3 relu); -1: none
};

// Scratch of the three-launch form for long prompts, in which every piece of 32 rows is a block of its own.
struct PieceArgs {
    float* sums;        // [piece][head][tile][D * VT + D]: a piece's own sum; after the scan, the state before the piece
    float* scalars;     // [piece][head][2]: the piece's sum of log forget gates, and the maximum its own rows would reach from minus infinity
    float* before;      // [piece][head]: the running maximum before the piece
};

// Piece g of the step (pieces of 32 rows, request after request): its request and its number inside the request; false past the last.
__device__ __forceinline__ bool find_piece(const int32_t* q_start, int n_seq, int g, int* seq, int* piece) {
    for (int s = 0; s < n_seq; ++s) {
        const int pieces = (q_start[s + 1] - q_start[s] + 31) >> 5;
        if (g < pieces) {
            *seq = s;
            *piece = g;
            return true;
        }
        g -= pieces;
    }
    return false;
}

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ float arriving(float z, int act) {
    if (act < 0) return z;
    const float sg = 1.0f / (1.0f + expf(-z));
    return act == LB_GATE_SILU ? z * sg : act == LB_GATE_GELU_TANH ? lb_gelu_tanh(z) : act == LB_GATE_RELU ? fmaxf(z, 0.0f) : sg;
}

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }

// Value d of a head's query or key row for the token at `pos`, rotated and scaled.
__device__ __forceinline__ float rotated(const float* row, int d, int rot_dims, const float* freq, int pos, float scale) {
    float v = row[d];
    if (d < rot_dims) {
        const int half = rot_dims >> 1, j = d < half ? d : d - half;
        float sn, cs;
        sincosf((float)pos * freq[j], &sn, &cs);
        const float lo = row[j], hi = row[j + half];
        v = d < half ? lo * cs - hi * sn : hi * cs + lo * sn;
    }
    return v * scale;
}

// The two gates of a token and head and the maximum after them.
__device__ __forceinline__ void gates(const MemoryArgs& a, int row, int h, float m_prev, float* keep, float* take, float* m_new) {
    if (a.decay != nullptr) {
        *keep = a.decay[h];
        *take = 1.0f;
        *m_new = 0.0f;
        return;
    }
    if (a.zi == nullptr) {
        *keep = expf(a.zf[(size_t)row * a.ld + h]);
        *take = 1.0f;
        *m_new = 0.0f;
        return;
    }
    const float gi = a.cap * tanhf(a.zi[(size_t)row * a.ld + h] / a.cap);
    const float gf = log_sigmoid(a.cap * tanhf(a.zf[(size_t)row * a.ld + h] / a.cap));
    const float m = fmaxf(gf + m_prev, gi);
    *keep = expf(gf + m_prev - m);
    *take = expf(gi - m);
    *m_new = m;
}

// ---------------------------------------------------------------- row by row
// 256 threads: thread (c, ds) owns rows ds, ds + DS, .. of column c of the tile's S (in shared memory).  The state and the first
// row's queries, keys and values are asked for together (4-byte cp.async), and every further row a row ahead, so that a decode
// step is one round trip to memory and a short portion one per row.
__global__ void __launch_bounds__(256) matrix_memory_rows_kernel(MemoryArgs a, int vt_pow2) {
    extern __shared__ float smem[];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int seq = blockIdx.x, h = blockIdx.y, nv = blockIdx.z;
    const int row0 = a.q_start[seq], row1 = a.q_start[seq + 1];
    if (row1 <= row0) return;
    const int D = a.D, VT = a.VT, E = a.E;
    const int c = threadIdx.x & (vt_pow2 - 1), ds = threadIdx.x / vt_pow2, DS = blockDim.x / vt_pow2;
    const int col = nv * VT + c;
    const bool live = c < VT && col < E;
    float* S = smem;                       // [D][VT]
    float* ns = S + (size_t)D * VT;        // [D]
    float* qs = ns + D;                    // [D] rotated and scaled
    float* ks = qs + D;                    // [D]
    float* red = ks + D;                   // [DS][vt_pow2]
    float* raw = red + 256;                // [2][2 D + VT]: a row's queries, keys and values as they arrive, two rows in turn
    const int raw_row = 2 * D + VT;
    float* st = a.state + (size_t)a.slots[seq] * a.slot_stride + ((size_t)h * a.NV + nv) * ((size_t)D * VT + D + 1);
    const bool gated = a.zi != nullptr;
    auto ask = [&](int row, int buffer) {
        float* dst = raw + buffer * raw_row;
        const float* q_row = a.q + (size_t)row * a.ld + (size_t)(h / a.qk_share) * D;
        const float* k_row = a.k + (size_t)row * a.ld + (size_t)(h / a.qk_share) * D;
        const float* v_row = a.v + (size_t)row * a.ld + (size_t)h * E + nv * VT;
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            cp_async4(dst + d, q_row + d);
            cp_async4(dst + D + d, k_row + d);
        }
        for (int x = threadIdx.x; x < VT; x += blockDim.x) {
            if (nv * VT + x < E) cp_async4(dst + 2 * D + x, v_row + x);
            else dst[2 * D + x] = 0.0f;
        }
    };
    for (int i = threadIdx.x; i < D * VT + D; i += blockDim.x) cp_async4(S + i, st + i);       // S and n lie one after the other
    ask(row0, 0);
    cp_async_commit();
    float m = st[(size_t)D * VT + D];
    for (int row = row0; row < row1; ++row) {
        const int buffer = (row - row0) & 1;
        const int pos = a.positions[row];
        float keep, take, m_new;
        gates(a, row, h, m, &keep, &take, &m_new);
        m = m_new;
        cp_async_wait_all();
        __syncthreads();                   // the row has arrived; everyone is done with the row before
        if (row + 1 < row1) ask(row + 1, buffer ^ 1);
        cp_async_commit();
        float* mine = raw + buffer * raw_row;
        if (a.qkv_act >= 0) {              // the row's queries, keys and (real) values pass the activation where they landed
            for (int i = threadIdx.x; i < raw_row; i += blockDim.x)
                if (i < 2 * D || nv * VT + (i - 2 * D) < E) mine[i] = arriving(mine[i], a.qkv_act);
            __syncthreads();
        }
        for (int d = threadIdx.x; d < 2 * D; d += blockDim.x) {
            const bool is_k = d >= D;
            const int dd = is_k ? d - D : d;
            (is_k ? ks : qs)[dd] = rotated(mine + (is_k ? D : 0), dd, a.rot_dims, a.freq, pos, is_k ? a.k_scale : a.q_scale);
        }
        __syncthreads();
        float acc = 0.0f;
        if (live) {
            const float tv = take * mine[2 * D + c];
            for (int d = ds; d < D; d += DS) {
                const float s = fmaf(keep, S[d * VT + c], ks[d] * tv);
                S[d * VT + c] = s;
                acc = fmaf(s, qs[d], acc);
            }
        }
        red[ds * vt_pow2 + c] = acc;
        if (gated)
            for (int d = threadIdx.x; d < D; d += blockDim.x) ns[d] = fmaf(keep, ns[d], take * ks[d]);
        __syncthreads();
        if (ds == 0 && live) {
            float o = 0.0f;
            for (int i = 0; i < DS; ++i) o += red[i * vt_pow2 + c];
            if (gated) {
                float nq = 0.0f;
                for (int d = 0; d < D; ++d) nq = fmaf(ns[d], qs[d], nq);
                o /= fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
            }
            a.out[(size_t)row * a.ldo + (size_t)h * E + col] = o;
        }
    }
    cp_async_wait_all();
    __syncthreads();
    for (int i = threadIdx.x; i < D * VT + D; i += blockDim.x) st[i] = S[i];
    if (threadIdx.x == 0) st[(size_t)D * VT + D] = m;
}

// S[d][c] = keep S[d][c] + sum_j u_j k_j[d] v_j[c] for this thread's column c and its values d = tg, tg + DS, .., N of them at a time.
template <int N, int DS>
__device__ __forceinline__ void state_after_piece(float* S, const float* ks, const float* vs, const float* uj, float keep, int tg, int c, int cc, bool live,
                                                  int n, int D, int VT, int LDQ) {
    for (int d0 = tg; d0 < D; d0 += N * DS) {
        float add[N];
#pragma unroll
        for (int i = 0; i < N; ++i) add[i] = 0.0f;
        for (int j = 0; j < n; ++j) {
            const float v = uj[j] * vs[j * VT + cc];
#pragma unroll
            for (int i = 0; i < N; ++i) {
                const int d = d0 + i * DS;
                if (d < D) add[i] = fmaf(ks[j * LDQ + d], v, add[i]);
            }
        }
        if (live) {
#pragma unroll
            for (int i = 0; i < N; ++i) {
                const int d = d0 + i * DS;
                if (d < D) S[d * VT + c] = fmaf(keep, S[d * VT + c], add[i]);
            }
        }
    }
}

// ---------------------------------------------------------------- in pieces of 32 rows
// With b_t the sum of the log forget gates from the piece's start to row t, and m_t the running maximum (by the same recursion
// as row by row):  w(t, j) = exp(i_j + b_t - b_j - m_t) for j <= t,  alpha_t = exp(b_t + m_prev - m_t),
//     o_t = alpha_t S_prev^T q_t + sum_{j <= t} w(t, j) (q_t . k_j) v_j,      n_t . q_t likewise with n_prev and without v,
//     S_new = exp(b_last + m_prev - m_last) S_prev + sum_j exp(i_j + b_last - b_j - m_last) k_j v_j^T.
// Every exponent is at most 0.  A fixed decay is the case i = 0, f = log(decay), m = 0.  The piece's rows are asked for together
// (three round trips to memory a piece instead of three a row); thread (c, g) owns column c of the tile for rows g, g + DS, ..
constexpr int kPiece = 32;

// MODE 0: a block walks a request's pieces one after the other from the state in its slot.  For long prompts three launches instead:
// MODE 1, a block per piece: the piece's own sum, as if its state began at zero and its maximum at minus infinity; then the scan
// (matrix_memory_scan_kernel) leaves the state before every piece in the sum's place; MODE 2, a block per piece: the piece's outputs
// from that state.
template <int VTP, int NT, int MODE>
__global__ void __launch_bounds__(NT) matrix_memory_chunks_kernel(MemoryArgs a, PieceArgs w, int n_seq) {
    constexpr int vt_pow2 = VTP, DS = NT / VTP, R = kPiece / DS, kWarps = NT / 32;      // thread (c, tg) owns column c for the R rows tg, tg + DS, ..
    extern __shared__ float smem[];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int h = blockIdx.y, nv = blockIdx.z;
    int seq = blockIdx.x, piece = 0;
    if (MODE != 0 && !find_piece(a.q_start, n_seq, blockIdx.x, &seq, &piece)) return;
    const int row0 = a.q_start[seq] + piece * kPiece, row1 = MODE == 0 ? a.q_start[seq + 1] : min(a.q_start[seq + 1], row0 + kPiece);
    if (row1 <= row0) return;
    const int D = a.D, VT = a.VT, E = a.E, LDQ = D + 1, LDP = kPiece + 1;
    const int c = threadIdx.x & (vt_pow2 - 1), tg = threadIdx.x / vt_pow2, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = nv * VT + c;
    const bool live = c < VT && col < E;
    const int cc = live ? c : 0;           // threads without a column read column 0 and store nothing
    float* S = smem;                       // [D][VT]
    float* ns = S + (size_t)D * VT;        // [D]
    float* qs = ns + D;                    // [kPiece][LDQ]
    float* ks = qs + kPiece * LDQ;         // [kPiece][LDQ]
    float* vs = ks + kPiece * LDQ;         // [kPiece][VT]
    float* P = vs + kPiece * VT;           // [kPiece][LDP]
    float* gi = P + kPiece * LDP;          // log input gate of row t
    float* gb = gi + kPiece;               // b_t
    float* gm = gb + kPiece;               // m_t
    float* al = gm + kPiece;               // alpha_t
    float* uj = al + kPiece;               // row j's factor in the new state
    float* den = uj + kPiece;              // what divides row t
    float* sc = den + kPiece;              // [0] the old state's factor in the new one, [1] m_last
    int* pos_s = reinterpret_cast<int*>(sc + 2);      // the rows' positions
    const bool gated = a.zi != nullptr, token = a.decay == nullptr && !gated;
    const float logd = a.decay == nullptr ? 0.0f : logf(a.decay[h]);       // -inf for a decay of 0: exp gives 0
    float* st = MODE == 0 ? a.state + (size_t)a.slots[seq] * a.slot_stride + ((size_t)h * a.NV + nv) * ((size_t)D * VT + D + 1)
                          : w.sums + (((size_t)blockIdx.x * a.H + h) * a.NV + nv) * ((size_t)D * VT + D);
    float m;
    if (MODE == 1) {
        for (int i = threadIdx.x; i < D * VT + D; i += blockDim.x) S[i] = 0.0f;
        m = gated ? -CUDART_INF_F : 0.0f;
    } else {
        for (int i = threadIdx.x; i < D * VT + D; i += blockDim.x) S[i] = st[i];
        m = MODE == 0 ? st[(size_t)D * VT + D] : w.before[(size_t)blockIdx.x * a.H + h];
    }
    for (int p0 = row0; p0 < row1; p0 += kPiece) {
        const int n = min(kPiece, row1 - p0);
        // The piece's rows as they are, all asked for at once (4-byte cp.async, one round trip), and the gates.
        for (int t = warp; t < n; t += kWarps) {          // a warp per row, lanes over the row's values
            const float* q_row = a.q + (size_t)(p0 + t) * a.ld + (size_t)(h / a.qk_share) * D;
            const float* k_row = a.k + (size_t)(p0 + t) * a.ld + (size_t)(h / a.qk_share) * D;
            for (int d = lane; d < D; d += 32) {
                if (MODE != 1) cp_async4(qs + t * LDQ + d, q_row + d);       // a piece's own sum needs no queries
                cp_async4(ks + t * LDQ + d, k_row + d);
            }
            const float* v_row = a.v + (size_t)(p0 + t) * a.ld + (size_t)h * E + nv * VT;
            for (int x = lane; x < VT; x += 32) {
                if (nv * VT + x < E) cp_async4(vs + t * VT + x, v_row + x);
                else vs[t * VT + x] = 0.0f;
            }
        }
        cp_async_commit();
        if (threadIdx.x < kPiece) {
            const int t = threadIdx.x, row = p0 + t;
            float i_log = -CUDART_INF_F, f_log = 0.0f;
            if (t < n) {
                pos_s[t] = a.positions[row];
                if (gated) {
                    i_log = a.cap * tanhf(a.zi[(size_t)row * a.ld + h] / a.cap);
                    f_log = log_sigmoid(a.cap * tanhf(a.zf[(size_t)row * a.ld + h] / a.cap));
                } else if (token) {
                    f_log = a.zf[(size_t)row * a.ld + h];
                }
            }
            // b_t by a running sum over the lanes.
            float b = f_log;
            if (gated || token) {
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float up = __shfl_up_sync(0xffffffffu, b, o);
                    if (t >= o) b += up;
                }
                gb[t] = b;
            }
            if (gated) {
                // m_t = b_t + max(m_prev, max_{j <= t} (i_j - b_j)), which is the recursion m_t = max(f_t + m_{t-1}, i_t) written out.
                float best = i_log - b;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float up = __shfl_up_sync(0xffffffffu, best, o);
                    if (t >= o) best = fmaxf(best, up);
                }
                gi[t] = i_log;
                gm[t] = b + fmaxf(m, best);
            }
        }
        cp_async_wait_all();
        __syncthreads();
        if (a.qkv_act >= 0) {              // queries, keys and (real) values pass the activation where they landed
            for (int t = warp; t < n; t += kWarps) {
                for (int d = lane; d < D; d += 32) {
                    if (MODE != 1) qs[t * LDQ + d] = arriving(qs[t * LDQ + d], a.qkv_act);
                    ks[t * LDQ + d] = arriving(ks[t * LDQ + d], a.qkv_act);
                }
                for (int x = lane; x < VT; x += 32)
                    if (nv * VT + x < E) vs[t * VT + x] = arriving(vs[t * VT + x], a.qkv_act);
            }
            __syncwarp();                  // the warp that activated a row is the one that rotates it below
        }
        // Rotation and scales, in place.
        {
            const int half = a.rot_dims >> 1;
            for (int t = warp; t < n; t += kWarps) {
                float* q_row = qs + t * LDQ;
                float* k_row = ks + t * LDQ;
                for (int d = lane; d < half; d += 32) {
                    float sn, cs;
                    sincosf((float)pos_s[t] * a.freq[d], &sn, &cs);
                    const float ql = MODE != 1 ? q_row[d] : 0.0f, qh = MODE != 1 ? q_row[d + half] : 0.0f, kl = k_row[d], kh = k_row[d + half];
                    q_row[d] = (ql * cs - qh * sn) * a.q_scale;
                    q_row[d + half] = (qh * cs + ql * sn) * a.q_scale;
                    k_row[d] = (kl * cs - kh * sn) * a.k_scale;
                    k_row[d + half] = (kh * cs + kl * sn) * a.k_scale;
                }
                for (int d = a.rot_dims + lane; d < D; d += 32) {
                    q_row[d] *= a.q_scale;
                    k_row[d] *= a.k_scale;
                }
            }
        }
        __syncthreads();
        if (threadIdx.x < n) {
            const int t = threadIdx.x;
            if (gated) {
                al[t] = expf(gb[t] + m - gm[t]);
                uj[t] = expf(gi[t] + gb[n - 1] - gb[t] - gm[n - 1]);
            } else if (token) {
                al[t] = expf(gb[t]);
                uj[t] = t == n - 1 ? 1.0f : expf(gb[n - 1] - gb[t]);
            } else {
                al[t] = expf((float)(t + 1) * logd);
                uj[t] = t == n - 1 ? 1.0f : expf((float)(n - 1 - t) * logd);
            }
            if (t == 0) {
                sc[0] = gated ? expf(gb[n - 1] + m - gm[n - 1]) : token ? expf(gb[n - 1]) : expf((float)n * logd);
                sc[1] = gated ? gm[n - 1] : 0.0f;
                if (MODE == 1 && nv == 0) {
                    w.scalars[((size_t)blockIdx.x * a.H + h) * 2] = gated || token ? gb[n - 1] : (float)n * logd;
                    w.scalars[((size_t)blockIdx.x * a.H + h) * 2 + 1] = sc[1];
                }
            }
        }
        // Weighted scores: a warp per row t, lane j.
        if (MODE != 1)
        for (int t = warp; t < kPiece; t += kWarps) {
            const int j = lane;
            float p = 0.0f;
            const float* q_row = qs + t * LDQ;
            if (t < n && j <= t) {
                const float* k_row = ks + j * LDQ;
                float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
                int d = 0;
                for (; d + 3 < D; d += 4) {
                    d0 = fmaf(q_row[d], k_row[d], d0);
                    d1 = fmaf(q_row[d + 1], k_row[d + 1], d1);
                    d2 = fmaf(q_row[d + 2], k_row[d + 2], d2);
                    d3 = fmaf(q_row[d + 3], k_row[d + 3], d3);
                }
                for (; d < D; ++d) d0 = fmaf(q_row[d], k_row[d], d0);
                const float w = gated ? expf(gi[j] + gb[t] - gb[j] - gm[t]) : t == j ? 1.0f : token ? expf(gb[t] - gb[j]) : expf((float)(t - j) * logd);
                p = ((d0 + d1) + (d2 + d3)) * w;
            }
            P[t * LDP + j] = p;
            // What divides the row: the old n's share (lanes over its values) and the piece's (the row's weighted scores).
            if (t < n) {
                float divisor = 1.0f;
                if (gated) {
                    float old = 0.0f;
                    for (int x = lane; x < D; x += 32) old = fmaf(ns[x], q_row[x], old);
                    const float nq = expf(gb[t] + m - gm[t]) * lb_warp_sum(old) + lb_warp_sum(p);
                    divisor = fmaxf(fabsf(nq), expf(-gm[t])) + 1e-6f;
                }
                if (lane == 0) den[t] = divisor;
            }
        }
        __syncthreads();
        const float m_next = sc[1];
        // Outputs: this thread's rows tg, tg + DS, .. (up to eight) of column c.
        if (MODE != 1) {
            float from_state[R], from_piece[R];
#pragma unroll
            for (int r = 0; r < R; ++r) from_state[r] = from_piece[r] = 0.0f;
            const float* q_rows = qs + tg * LDQ;
            const float* p_rows = P + tg * LDP;
#pragma unroll 2
            for (int d = 0; d < D; ++d) {
                const float s = S[d * VT + cc];
#pragma unroll
                for (int r = 0; r < R; ++r) from_state[r] = fmaf(q_rows[r * DS * LDQ + d], s, from_state[r]);
            }
#pragma unroll 2
            for (int j = 0; j < n; ++j) {
                const float v = vs[j * VT + cc];
#pragma unroll
                for (int r = 0; r < R; ++r) from_piece[r] = fmaf(p_rows[r * DS * LDP + j], v, from_piece[r]);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int t = tg + r * DS;
                if (t < n && live) a.out[(size_t)(p0 + t) * a.ldo + (size_t)h * E + col] = (al[t] * from_state[r] + from_piece[r]) / den[t];
            }
        }
        __syncthreads();
        // The state after the piece.
        if (MODE == 2) break;
        const float keep = sc[0];
        if (D <= 2 * DS) state_after_piece<2, DS>(S, ks, vs, uj, keep, tg, c, cc, live, n, D, VT, LDQ);
        else if (D <= 4 * DS) state_after_piece<4, DS>(S, ks, vs, uj, keep, tg, c, cc, live, n, D, VT, LDQ);
        else state_after_piece<8, DS>(S, ks, vs, uj, keep, tg, c, cc, live, n, D, VT, LDQ);
        if (gated)
            for (int d = threadIdx.x; d < D; d += blockDim.x) {
                float add = 0.0f;
                for (int j = 0; j < n; ++j) add = fmaf(uj[j], ks[j * LDQ + d], add);
                ns[d] = fmaf(keep, ns[d], add);
            }
        m = m_next;
        __syncthreads();
    }
    if constexpr (MODE != 2) {
        for (int i = threadIdx.x; i < D * VT + D; i += blockDim.x) st[i] = S[i];
        if (MODE == 0 && threadIdx.x == 0) st[(size_t)D * VT + D] = m;
    }
}

// The scan between the two launches of the per-piece form: a block per (request, head, value tile) walks the request's pieces.  With
// (b, m_own) the piece's scalars: m_new = max(b + m, m_own), S_new = exp(b + m - m_new) S + exp(m_own - m_new) sum; a fixed decay has
// m = 0 throughout and b = rows x log(decay).  The state before the piece takes the sum's place; the next piece's sum travels (cp.async)
// while this one is added.
__global__ void __launch_bounds__(256) matrix_memory_scan_kernel(MemoryArgs a, PieceArgs w) {
    extern __shared__ float smem[];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int seq = blockIdx.x, h = blockIdx.y, nv = blockIdx.z;
    const int len = a.q_start[seq + 1] - a.q_start[seq], pieces = (len + 31) >> 5;
    if (pieces <= 0) return;
    int g0 = 0;
    for (int s = 0; s < seq; ++s) g0 += (a.q_start[s + 1] - a.q_start[s] + 31) >> 5;
    const int count = a.D * a.VT + a.D;
    float* S = smem;                    // [count]
    float* buf = S + count;             // [2][count]
    float* st = a.state + (size_t)a.slots[seq] * a.slot_stride + ((size_t)h * a.NV + nv) * ((size_t)count + 1);
    const bool gated = a.zi != nullptr;
    auto sum_of = [&](int g) { return w.sums + (((size_t)g * a.H + h) * a.NV + nv) * (size_t)count; };
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
        cp_async4(S + i, st + i);
        cp_async4(buf + i, sum_of(g0) + i);
    }
    cp_async_commit();
    float m = st[count];
    float b_next = w.scalars[((size_t)g0 * a.H + h) * 2], own_next = w.scalars[((size_t)g0 * a.H + h) * 2 + 1];
    for (int p = 0; p < pieces; ++p) {
        const int g = g0 + p;
        float* mine = buf + (p & 1) * count;
        const float b = b_next, m_own = own_next;
        cp_async_wait_all();
        __syncthreads();
        if (p + 1 < pieces) {              // the next piece's sum and scalars travel while this one is added
            float* next = buf + ((p + 1) & 1) * count;
            for (int i = threadIdx.x; i < count; i += blockDim.x) cp_async4(next + i, sum_of(g + 1) + i);
            b_next = w.scalars[((size_t)(g + 1) * a.H + h) * 2];
            own_next = w.scalars[((size_t)(g + 1) * a.H + h) * 2 + 1];
        }
        cp_async_commit();
        const float m_new = gated ? fmaxf(b + m, m_own) : 0.0f;
        const float keep = gated ? expf(b + m - m_new) : expf(b), take = gated ? expf(m_own - m_new) : 1.0f;
        float* out = sum_of(g);
        for (int i = threadIdx.x; i < count; i += blockDim.x) {
            const float before = S[i];
            out[i] = before;
            S[i] = fmaf(keep, before, take * mine[i]);
        }
        if (nv == 0 && threadIdx.x == 0) w.before[(size_t)g * a.H + h] = m;
        m = m_new;
    }
    for (int i = threadIdx.x; i < count; i += blockDim.x) st[i] = S[i];
    if (threadIdx.x == 0) st[count] = m;
}

}  // namespace

namespace {
struct PieceScratch {
    float* sums;
    float* scalars;
    float* before;
    int max_pieces;
};
}  // namespace

static int matrix_memory_run(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                             const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state,
                             int64_t slot_stride, float* out, int64_t ldo, int n_seq, int n_head, int dim, int vdim, int value_tile, float q_scale,
                             float k_scale, float cap, int chunked, const PieceScratch* pieces, int qk_share, int qkv_act, void* stream) {
    LB_CHECK_ARG(qkv_act >= -1 && qkv_act <= LB_GATE_RELU, "matrix memory: activation %d on queries, keys and values (-1 none, 0 sigmoid, 1 silu, 2 gelu_tanh, 3 relu)", qkv_act);
    LB_CHECK_ARG(n_seq >= 0 && n_head > 0 && dim > 0 && vdim > 0 && value_tile > 0 && value_tile <= 64, "matrix memory: bad sizes heads=%d dim=%d vdim=%d tile=%d",
                 n_head, dim, vdim, value_tile);
    LB_CHECK_ARG(decay != nullptr ? (zi == nullptr && zf == nullptr) : zf != nullptr, "matrix memory: a fixed decay, or the two gates, or the log of a decay a token");
    LB_CHECK_ARG(qk_share >= 1 && n_head % qk_share == 0, "matrix memory: %d heads do not share queries and keys in groups of %d", n_head, qk_share);
    LB_CHECK_ARG(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || freq != nullptr), "matrix memory: %d of %d values to rotate", rot_dims, dim);
    if (n_seq == 0) return LB_OK;
    MemoryArgs a{};
    a.q = q; a.k = k; a.v = v; a.zi = zi; a.zf = zf; a.ld = ld; a.decay = decay; a.freq = freq; a.positions = positions; a.q_start = q_start;
    a.slots = slots; a.state = state; a.slot_stride = slot_stride; a.out = out; a.ldo = ldo;
    a.H = n_head; a.D = dim; a.E = vdim; a.VT = value_tile; a.NV = (vdim + value_tile - 1) / value_tile; a.rot_dims = rot_dims;
    a.q_scale = q_scale; a.k_scale = k_scale; a.cap = cap; a.qk_share = qk_share; a.qkv_act = qkv_act;
    LB_CHECK_ARG(slot_stride >= (int64_t)n_head * a.NV * ((int64_t)dim * value_tile + dim + 1), "matrix memory: the state slots are too small");
    int p2 = 1;
    while (p2 < value_tile) p2 <<= 1;
    auto s = static_cast<cudaStream_t>(stream);
    if (chunked) {
        const size_t bytes = ((size_t)dim * value_tile + dim + 2 * (size_t)kPiece * (dim + 1) + (size_t)kPiece * value_tile + kPiece * (kPiece + 1) + 7 * kPiece + 2) *
                             sizeof(float);
        LB_CHECK_ARG(bytes <= 200 * 1024, "matrix memory: a tile of %d x %d floats does not fit shared memory", dim, value_tile);
        auto launch = [&](auto kernel, int threads, int blocks, const PieceArgs& w) -> int {
            if (bytes > 48 * 1024) LB_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
            LB_CHECK_CUDA(lb_launch_overlapped(kernel, dim3(blocks, n_head, a.NV), dim3(threads), bytes, s, a, w, n_seq));
            return LB_OK;
        };
#define LB_MEMORY_MODE(MODE, blocks, w)                                                                   \
    (p2 <= 8    ? launch(matrix_memory_chunks_kernel<8, 256, MODE>, 256, blocks, w)                      \
     : p2 == 16 ? launch(matrix_memory_chunks_kernel<16, 512, MODE>, 512, blocks, w)                     \
     : p2 == 32 ? launch(matrix_memory_chunks_kernel<32, 512, MODE>, 512, blocks, w)                     \
                : launch(matrix_memory_chunks_kernel<64, 512, MODE>, 512, blocks, w))
        if (pieces == nullptr) return LB_MEMORY_MODE(0, n_seq, PieceArgs{});
        // Every piece a block of its own: the pieces' own sums, the scan over them, the pieces' outputs.
        const PieceArgs w{pieces->sums, pieces->scalars, pieces->before};
        if (int rc = LB_MEMORY_MODE(1, pieces->max_pieces, w)) return rc;
        const size_t scan_bytes = 3 * ((size_t)dim * value_tile + dim) * sizeof(float);
        LB_CHECK_ARG(scan_bytes <= 200 * 1024, "matrix memory: a tile of %d x %d floats does not fit shared memory", dim, value_tile);
        if (scan_bytes > 48 * 1024) LB_CHECK_CUDA(cudaFuncSetAttribute(matrix_memory_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)scan_bytes));
        LB_CHECK_CUDA(lb_launch_overlapped(matrix_memory_scan_kernel, dim3(n_seq, n_head, a.NV), dim3(256), scan_bytes, s, a, w));
        return LB_MEMORY_MODE(2, pieces->max_pieces, w);
#undef LB_MEMORY_MODE
    }
    const size_t smem = ((size_t)dim * value_tile + 3 * (size_t)dim + 256 + 2 * (2 * (size_t)dim + value_tile)) * sizeof(float);
    LB_CHECK_ARG(smem <= 200 * 1024, "matrix memory: a tile of %d x %d floats does not fit shared memory", dim, value_tile);
    if (smem > 48 * 1024) LB_CHECK_CUDA(cudaFuncSetAttribute(matrix_memory_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LB_CHECK_CUDA(lb_launch_overlapped(matrix_memory_rows_kernel, dim3(n_seq, n_head, a.NV), dim3(256), smem, s, a, p2));
    return LB_OK;
}

extern "C" int lb_matrix_memory(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                                const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state,
                                int64_t slot_stride, float* out, int64_t ldo, int n_seq, int n_head, int dim, int vdim, int value_tile, float q_scale,
                                float k_scale, float cap, int chunked, void* stream) {
    return matrix_memory_run(q, k, v, zi, zf, ld, decay, freq, rot_dims, positions, q_start, slots, state, slot_stride, out, ldo, n_seq, n_head, dim, vdim,
                             value_tile, q_scale, k_scale, cap, chunked, nullptr, 1, -1, stream);
}

extern "C" int lb_matrix_memory_shared(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                                       const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state,
                                       int64_t slot_stride, float* out, int64_t ldo, int n_seq, int n_head, int dim, int vdim, int value_tile, float q_scale,
                                       float k_scale, float cap, int chunked, int qk_share, void* stream) {
    return lb_matrix_memory_activated(q, k, v, zi, zf, ld, decay, freq, rot_dims, positions, q_start, slots, state, slot_stride, out, ldo, n_seq, n_head, dim,
                                      vdim, value_tile, q_scale, k_scale, cap, chunked, qk_share, -1, stream);
}

extern "C" int lb_matrix_memory_activated(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                                          const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots,
                                          float* state, int64_t slot_stride, float* out, int64_t ldo, int n_seq, int n_head, int dim, int vdim, int value_tile,
                                          float q_scale, float k_scale, float cap, int chunked, int qk_share, int qkv_act, void* stream) {
    return matrix_memory_run(q, k, v, zi, zf, ld, decay, freq, rot_dims, positions, q_start, slots, state, slot_stride, out, ldo, n_seq, n_head, dim, vdim,
                             value_tile, q_scale, k_scale, cap, chunked, nullptr, qk_share, qkv_act, stream);
}

extern "C" int64_t lb_matrix_memory_pieces_floats(int n_tokens, int n_seq, int n_head, int dim, int vdim, int value_tile) {
    const int64_t pieces = n_tokens / 32 + n_seq, tiles = (vdim + value_tile - 1) / value_tile;
    return pieces * n_head * (tiles * ((int64_t)dim * value_tile + dim) + 3);
}

extern "C" int lb_matrix_memory_pieces_shared(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                                              const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots,
                                              float* state, int64_t slot_stride, float* out, int64_t ldo, int n_tokens, int n_seq, int n_head, int dim, int vdim,
                                              int value_tile, float q_scale, float k_scale, float cap, float* scratch, int qk_share, void* stream) {
    return lb_matrix_memory_pieces_activated(q, k, v, zi, zf, ld, decay, freq, rot_dims, positions, q_start, slots, state, slot_stride, out, ldo, n_tokens, n_seq,
                                             n_head, dim, vdim, value_tile, q_scale, k_scale, cap, scratch, qk_share, -1, stream);
}

extern "C" int lb_matrix_memory_pieces_activated(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld,
                                                 const float* decay, const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start,
                                                 const int32_t* slots, float* state, int64_t slot_stride, float* out, int64_t ldo, int n_tokens, int n_seq,
                                                 int n_head, int dim, int vdim, int value_tile, float q_scale, float k_scale, float cap, float* scratch,
                                                 int qk_share, int qkv_act, void* stream) {
    LB_CHECK_ARG(scratch != nullptr && n_tokens >= 0 && value_tile > 0, "matrix memory in pieces: no scratch");
    const int64_t pieces = n_tokens / 32 + n_seq, tiles = (vdim + value_tile - 1) / value_tile;
    const int64_t sums = pieces * n_head * tiles * ((int64_t)dim * value_tile + dim);
    const PieceScratch ps{scratch, scratch + sums, scratch + sums + pieces * n_head * 2, (int)pieces};
    return matrix_memory_run(q, k, v, zi, zf, ld, decay, freq, rot_dims, positions, q_start, slots, state, slot_stride, out, ldo, n_seq, n_head, dim, vdim,
                             value_tile, q_scale, k_scale, cap, 1, &ps, qk_share, qkv_act, stream);
}

extern "C" int lb_matrix_memory_pieces(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                                       const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots,
                                       float* state, int64_t slot_stride, float* out, int64_t ldo, int n_tokens, int n_seq, int n_head, int dim, int vdim,
                                       int value_tile, float q_scale, float k_scale, float cap, float* scratch, void* stream) {
    return lb_matrix_memory_pieces_shared(q, k, v, zi, zf, ld, decay, freq, rot_dims, positions, q_start, slots, state, slot_stride, out, ldo, n_tokens, n_seq,
                                          n_head, dim, vdim, value_tile, q_scale, k_scale, cap, scratch, 1, stream);
}
