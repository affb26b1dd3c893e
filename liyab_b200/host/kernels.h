// C++ faces of the CUDA kernels (csrc/api.h) and the choice between them.
//
// Each function passes raw device pointers and the step's stream to the kernel
// library's C interface and turns a non-zero status into an `Error` carrying the
// library's message.  Nothing here computes: there is no CPU path and no library
// fallback.  The functions that choose a kernel by type and size (`linear`,
// `gemm_splits`, `decode_splits`, `attend`) are pure functions of the shapes, so a
// captured step and an eager one choose alike.
#pragma once

#include <atomic>
#include <cstdint>
#include <string>
#include <vector>

#include "device.h"
#include "spec.h"

namespace liyab::kernels {

// Kernel launches issued through this module (a replayed graph adds its own count).
extern std::atomic<uint64_t> launches;

void check(int status, const char* what);

// kXielu: the activation's two learned numbers ride behind the bias (a bias of N + 2 floats: bias[N] = p, bias[N + 1] = q).
enum Activation : int { kNone = 0, kGeluTanh = 1, kGeluErf = 2, kXielu = 3, kRelu2 = 4 };      // kRelu2: max(z, 0)^2
int activation_from_name(const std::string& name);      // UNSUPPORTED when unknown

// Keys and values of a fused projection that go straight to a layer's cache pages.
struct KvDestination {
    void* cache = nullptr;
    const int32_t* slot_mapping = nullptr;
    int q_dim = 0, n_kv_head = 0, head_dim = 0, page_size = 0;
};

void embed_positions(cudaStream_t s, const int32_t* tokens, const int32_t* positions, const Tensor& table,
                     const Tensor* pos_table, const Rows& x, int n_tokens, float scale);
// x[t] = table[token t] * scale + the sinusoid of the token's position (entry 2i sin(p w_i), entry 2i + 1 cos(p w_i); freq2 holds every w_i
// as two floats, leading part and rest); with `gain` [width] the row is then divided by its root mean square and multiplied by it.
void embed_sinusoid(cudaStream_t s, const int32_t* tokens, const int32_t* positions, const Tensor& table, const float* freq2, const float* gain,
                    const Rows& x, int n_tokens, float scale, float eps);
void gather_tokens(cudaStream_t s, int32_t* dst, const int32_t* src, const int32_t* map, int n);
void layernorm(cudaStream_t s, const Rows& x, const int32_t* rows, const float* weight, const float* bias, const Rows& out,
               int n_rows, float eps);
void kv_append(cudaStream_t s, const Rows& k, const Rows& v, const int32_t* slot_mapping, void* cache, DType cache_dtype,
               int n_tokens, int n_kv_head, int head_dim, int page_size);
void scale_softcap(cudaStream_t s, float* logits, int64_t count, float scale, float soft_cap);

// out[:m] = act(a[:m] . w^T + bias) + residual; w is [n, k] in the type of `a`; bias float32 or null.
bool tcgen05_accepts(const Rows& a, const Tensor& w);
int gemm_splits(int m, int n, int k);
void gemm_ffma(cudaStream_t s, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m, int act,
               const Rows* residual);
void gemm_tcgen05(cudaStream_t s, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m, int act,
                  const Rows* residual, float* partial, int n_splits);
// Products of up to 64 tokens take the one-launch kernel on mma.sync while every block can afford to fetch all
// activations: a reduction length of up to 1024 (measured: with K = 1600 or 3072 the tcgen05 kernel with K split over
// blocks and a second half wins, at 8 tokens as at 64).
inline constexpr int kRowsMaxK = 1024;
// Up to 16 tokens the kernel keeps all columns of the activations, so a longer reduction (up to 4096) is worth it too
// where a block then asks for all its weights at once: one pass over its feature groups (GPT-2 small's and medium's
// down projections; GPT-2 XL's projections would take three passes and stay with the split product: 2.30 against 2.16 ms).
bool gemm_rows_takes(int m, int n, int k, int sm_count);
bool gemm_rows_supports(const Rows& a, const Tensor& w, int m);
// The same product with the rows of the float32 matrix x normalised inside the kernel (LayerNorm: gain, offset or
// null, eps; with `rms` no mean is taken off and gain_offset is added to every gain): up to 16 tokens, K up to 1024,
// bfloat16 weights.
bool gemm_rows_normed_supports(const Runtime& rt, const Rows& x, const Tensor& w, int m);
void gemm_rows_normed(cudaStream_t s, const Rows& x, const float* gain, const float* offset, float eps, const Tensor& w, const float* bias,
                      const Rows& out, int m, int act, const Rows* residual, const KvDestination* kv, bool rms = false, float gain_offset = 0.0f);
void gemm_rows(cudaStream_t s, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m, int act,
               const Rows* residual, const KvDestination* kv);
int gemm_persistent_tile(const Rows& a, const Tensor& w, const Rows& out, int m, const Rows* residual);
bool gemm_persistent_kv_supports(const Tensor& w, const Rows& out, const KvDestination& kv);
void gemm_persistent(cudaStream_t s, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m, int act,
                     const Rows* residual, const KvDestination* kv);
// The product with the kernel chosen by type and size; `ws` lends scratch for products of few tokens.
void linear(const Runtime& rt, Workspace* ws, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m,
            int act, const Rows* residual);
// A fused projection of few tokens (at most 64) whose keys and values should also reach the cache: true when the
// chosen kernel did both (the split product's second half scatters them); false when nothing was launched and the
// caller should run the product and the cache write separately.
bool linear_with_cache(const Runtime& rt, Workspace* ws, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m,
                       const KvDestination& kv);

struct AttentionShape {
    int n_head = 0, n_kv_head = 0, head_dim = 0, page_size = 0;
    float scale = 1.0f;
    int window = 0;          // w > 0: a query sees the w latest keys
    int chunk = 0;           // c > 0: a query sees the earlier keys of its own chunk of c positions, counted from position 0
    // A penalty by distance: device floats r1 [n_head] then r2 [n_head]; the score of the key d positions back loses r1 ln(1 + r2 d).
    const float* distance = nullptr;
    // A sink a head: device floats [n_head]; exp(sink[h]) joins the divisor of the head's softmax as it is, with no key and no value.
    const float* sink = nullptr;
    // One number for the kernels: 0 all earlier keys, w > 0 a window, -c a chunk (a shape has one of the two at most).
    int mask() const { return chunk > 0 ? -chunk : window; }
};
bool decode_scalar_supports(const AttentionShape& a);
bool decode_mma_supports(const AttentionShape& a);
bool prefill_supports(const AttentionShape& a);
bool prefill_tc_supports(const AttentionShape& a);
int decode_splits(int n_seq, int n_kv_head, int max_context, bool tensor_cores);
void attention_generic(cudaStream_t s, DType dtype, const Rows& q, const void* cache, const int32_t* tok_seq,
                       const int32_t* positions, const int32_t* block_table, int table_width, const Rows& out, int n_tokens,
                       const AttentionShape& a);
void decode_attention(cudaStream_t s, bool tensor_cores, const Rows& q, const void* cache, int n_pages, const int32_t* positions,
                      const int32_t* block_table, int table_width, const Rows& out, float* partial, int* counters, int n_seq,
                      const AttentionShape& a, int n_splits);
void prefill_attention(const Runtime& rt, const Rows& q, int n_tokens, const void* cache, int n_pages, const int32_t* q_start,
                       const int32_t* n_past, const int32_t* block_table, int table_width, const Rows& out, int n_seq,
                       int max_q_len, const AttentionShape& a);

// ---- row-wise pieces between the products: RMS norm in groups, token shift, xIELU, gated side input ----
// out[r] = x[rows ? rows[r] : r] cut into `groups` equal parts, each over its own root mean square, times weight.
void rms_groups(cudaStream_t s, const Rows& x, const int32_t* rows, const float* weight, const Rows& out, int n_rows, int groups, float eps,
                float gain_offset = 0.0f);      // gain_offset: added to every gain (1 for gains stored around zero)
// The step's layout as the shift kernels need it.
struct ShiftLayout {
    const int32_t* tok_seq = nullptr;
    const int32_t* q_start = nullptr;
    const int32_t* slots = nullptr;
    int n_tokens = 0, n_seq = 0;
    bool decode_only = false;
};
// m[t] = h[t] + (h[t - 1] - h[t]) * mix, the row before a request's first row taken from (and its last row left in) `state`.
void token_shift(cudaStream_t s, const Rows& h, const float* mix, const Rows& m, void* state, const ShiftLayout& l);
// h = rms_groups(x) and m = token_shift(h) in one pass over x.
void rms_shift(cudaStream_t s, const Rows& x, const float* weight, const float* mix, const Rows& h, const Rows& m, void* state,
               const ShiftLayout& l, int groups, float eps);
// In place over z[:n_rows]: the xIELU with its two learned numbers pq (float, on the device).
void xielu(cudaStream_t s, const Rows& z, int n_rows, const float* pq);
// x[t] += rms(proj (gelu_tanh(gate x[t]) * table[tokens[t]])) * weight.
// Steps of more than 64 tokens in bfloat16 run the two maps as library products (x rounded to bfloat16 first); all others as two
// kernels of their own with 32-bit rows.  `ws` lends the scratch.
void token_side(const Runtime& rt, Workspace* ws, const Rows& x, const int32_t* tokens, const Tensor& table, const Tensor& gate, const Tensor& proj,
                const float* weight, int n_tokens, float eps);

// ---- attention over a cache of latent rows [c (rank) | r (rot)] ----
struct LatentShape {
    int n_head = 0, dim = 0, rot = 0, rot_dims = 0, vdim = 0, rank = 0, page_size = 0;
    float scale = 1.0f;
    int window = 0;
    const float* sink = nullptr;     // device floats [n_head]: exp(sink[h]) joins the divisor of the head's softmax (no key, no value)
    bool interleaved = false;        // the rotation pairs value 2i with 2i + 1 instead of i with i + rot_dims / 2
};
void latent_store(cudaStream_t s, const Rows& d, const float* gain, const float* freq, const int32_t* positions, const int32_t* slot_mapping,
                  void* cache, DType cache_dtype, int n_tokens, const LatentShape& a, float eps);
void rope_heads(cudaStream_t s, const Rows& q, const float* freq, const int32_t* positions, const Rows& wide, int n_tokens, const LatentShape& a);
// C[t, h * c_head + n] = sum_k A[t, h * a_head + k] * B[h * b_head + k * b_k + n * b_n].
// Float rows, bfloat16 maps and output whose strides fit 16-byte pieces go to the tensor cores; everything else to the 32-bit units.
void head_matmul(cudaStream_t s, const Rows& a, int64_t a_head, const Tensor& b, int64_t b_head, int64_t b_k, int64_t b_n, const Rows& c,
                 int64_t c_head, int m, int n, int k, int n_head);
// Steps of few tokens in bfloat16: rotation, keys' map and cache row in one launch; merge of the attention's parts and values' map in one.
bool latent_few_supports(const LatentShape& a);
void latent_prepare(cudaStream_t s, const Rows& qd, const Tensor& uk, const float* gain, const float* freq, const int32_t* positions,
                    const int32_t* slot_mapping, void* cache, const Rows& wide, int n_tokens, const LatentShape& a, float eps,
                    const Rows* latent = nullptr);      // latent: the rows [latent | rotated key] where they do not follow the queries in qd
void latent_finish(cudaStream_t s, const Rows& attended, const float* part_o, const float* part_ml, const Tensor& uv, const Rows& values, int n_tokens,
                   const LatentShape& a, int n_splits, const Rows* gate = nullptr);      // gate: one float a (token, head); the head's values times its sigmoid
// The tensor-core kernel (bfloat16 wide queries and cache): whether it takes the shape, into how many parts a decode step's keys are cut
// (a function of the step's shape and the longest span a query can see, so a recorded step and an eager one cut alike), and the launch.
bool latent_mma_supports(const LatentShape& a);
// Runs of tokens, latents of up to 256 values: 64 rows a block, the attended latents out as bfloat16 for the values' product.
bool latent_rows_supports(const LatentShape& a);
void latent_attention_rows16(cudaStream_t s, const Rows& wide, const void* cache, const int32_t* q_start, const int32_t* n_past, const int32_t* block_table,
                             int table_width, const Rows& out, int n_tokens, int n_seq, int max_q_len, const LatentShape& a, const Rows* gate = nullptr);
int latent_splits(int n_seq, int n_head, int span);
void latent_attention_mma(cudaStream_t s, const Rows& wide, const void* cache, const int32_t* q_start, const int32_t* n_past, const int32_t* block_table,
                          int table_width, const Rows& out, float* part_o, float* part_ml, int n_tokens, int n_seq, int max_q_len, const LatentShape& a,
                          int n_splits, bool merge = true, const Rows* gate = nullptr);       // merge false: the parts are left for latent_finish
void latent_attention(cudaStream_t s, DType cache_dtype, const Rows& wide, const void* cache, const int32_t* tok_seq, const int32_t* positions,
                      const int32_t* block_table, int table_width, const Rows& out, int n_tokens, const LatentShape& a, const Rows* gate = nullptr);

// ---- pieces around gated mixers and mixers of several branches ----
// x[r, :] += v (float [width]) for the first n_rows rows.
void add_row(cudaStream_t s, const Rows& x, const float* v, int n_rows);
// x[r, :] += scale * sum_i rms(y_i[r, :]) * weight_i over up to four branches (float rows; a weight may be null).
// With `rounded` (bfloat16 rows) the new rows of x are also left there, rounded once, for the part that reads the stream next.
void rms_sum_add(cudaStream_t s, const Rows& x, const std::vector<Rows>& y, const std::vector<const float*>& weight, int n_rows, float scale, float eps,
                 const Rows* rounded = nullptr);
// Queries, keys and values of a float projection on their way to attention: per-head RMS norm of queries and keys (gains may be null),
// queries into q_out [T, n_head * padded], keys and values into the cache pages (heads padded with zeros to `padded` values).
struct QkvColumns {
    int q_off = 0, k_off = 0, v_off = 0, n_head = 0, n_kv_head = 0, dim = 0, vdim = 0, padded = 0, page_size = 0;
};
// With temp_every > 0 the queries of the token at position p are multiplied by 1 + temp_coef ln(floor((p + 1) / temp_every) + 1).
void qk_norm_store(cudaStream_t s, const Rows& proj, const QkvColumns& c, const float* q_weight, const float* k_weight, const Rows& q_out, void* cache,
                   const int32_t* slot_mapping, int n_tokens, bool norm, float eps, const int32_t* positions = nullptr, float temp_coef = 0.0f,
                   int temp_every = 0);
// The same for queries and keys that are normed over the whole projection and rotated, and for values that blend with an earlier layer's:
// norm_mode 0 none, 1 a head (gains [dim]), 2 all of q and all of k each over one root mean square (gains [n_head * dim], [n_kv_head * dim]);
// the first rot_dims values of a head rotated in pairs (i, i + rot_dims / 2) by positions[t] * freq[i]; with v_first_in the values become
// (1 - lambda) v + lambda v_first_in[t], with v_first_out the row's own values are left there (float [T, n_kv_head * vdim]).
void qkv_rotary_store(cudaStream_t s, const Rows& proj, const QkvColumns& c, const float* q_weight, const float* k_weight, const Rows& q_out, void* cache,
                      const int32_t* slot_mapping, int n_tokens, int norm_mode, float eps, const int32_t* positions, const float* freq, int rot_dims,
                      const Rows* v_first_in, const Rows* v_first_out, const float* lambda);
// out = o over the root mean square of the whole row, times gain (or null), times gate(g) (rows g without data: no gate).
void row_norm_gate(cudaStream_t s, const Rows& o, const Rows& g, const float* gain, const Rows& out, int n_rows, int gate, float eps);
// In place over the float rows x[:n_rows]: sigmoid, silu, gelu_tanh or relu (a Gate code).
void activate_columns(cudaStream_t s, const Rows& x, int n_rows, int gate);
// A row's experts looked up by its token id in an int32 table [vocab, top]; every weight 1 / top.
void router_table(cudaStream_t s, const int32_t* tokens, const Tensor& table, int32_t* ids, float* weights, int n_rows, int top, int n_experts);
// router_table and expert_plan in one launch.
void expert_plan_table(cudaStream_t s, const int32_t* tokens, const Tensor& table, int32_t* ids, float* weights, int n_rows, int top, int n_experts,
                       int32_t* offsets, int32_t* place, int32_t* pair_at);
void rows_to_bf16(cudaStream_t s, const Rows& x, const Rows& y, int n_rows);
// kCapped has two numbers (alpha, limit): g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(alpha g') (u' + 1).
enum Gate : int { kSigmoid = 0, kSilu = 1, kGeluGate = 2, kRelu = 3, kCapped = 4 };
int gate_from_name(const std::string& name);
// out[t, h * vdim + c] = f(o[t, h * o_head + c]) * gain * gate(g[t, h * vdim + c]); f: over the head's root mean square when `norm`;
// rows g without data: no gate.
void head_gate(cudaStream_t s, const Rows& o, int o_head, const Rows& g, const float* gain, const Rows& out, int n_tokens, int n_head, int vdim, bool norm,
               int gate, float eps);
// mid[r, c] = gate(gu[r, c]) * gu[r, inner + c]; gu float [rows, 2 * inner].
void gated_act(cudaStream_t s, const Rows& gu, const Rows& mid, int n_rows, int gate, float alpha = 0.0f, float limit = 0.0f);

// ---- a matrix memory per head, carried from token to token (retention with a fixed decay; gated with a running maximum) ----
struct MemoryShape {
    int n_head = 0, dim = 0, vdim = 0, value_tile = 0, rot_dims = 0;
    float q_scale = 1.0f, k_scale = 1.0f, cap = 0.0f;
    int qk_share = 1;                // heads that read one query and key row (a group's); 1: every head its own
    int qkv_act = -1;                // an activation on queries, keys and values as the kernels read them (a Gate code up to kRelu); -1: none
    int64_t slot_stride = 0;         // floats between two requests' states; 0: slot_floats() (a mixer may keep more in its slot)
    int64_t stride() const { return slot_stride > 0 ? slot_stride : slot_floats(); }
    int tiles() const { return (vdim + value_tile - 1) / value_tile; }
    int64_t slot_floats() const { return static_cast<int64_t>(n_head) * tiles() * (static_cast<int64_t>(dim) * value_tile + dim + 1); }
};
// The value tile a shape gets (the state's layout depends on it, so it is chosen once per part).
int memory_value_tile(int dim, int vdim);
// q, k, v, zi, zf: column blocks of one float buffer (same stride); decay [n_head], or the two gates, or zf alone: the log of keep itself,
// a number a token and head (take = 1, no normaliser).
void matrix_memory(cudaStream_t s, const Rows& q, const Rows& k, const Rows& v, const Rows* zi, const Rows* zf, const float* decay, const float* freq,
                   const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state, const Rows& out, int n_seq, const MemoryShape& m,
                   bool chunked);
// The form for long portions (every piece of 32 rows a block of its own, three launches); `scratch` holds memory_pieces_floats(..) floats.
int64_t memory_pieces_floats(int n_tokens, int n_seq, const MemoryShape& m);
void matrix_memory_pieces(cudaStream_t s, const Rows& q, const Rows& k, const Rows& v, const Rows* zi, const Rows* zf, const float* decay, const float* freq,
                          const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state, const Rows& out, int n_tokens, int n_seq,
                          const MemoryShape& m, float* scratch);

// ---- routed experts ----
void router_topk(cudaStream_t s, const Rows& h, const Tensor& router, int32_t* ids, float* weights, int n_rows, int top, bool softmax, bool renormalise,
                 const float* bias = nullptr);
void expert_plan(cudaStream_t s, const int32_t* ids, int n_pairs, int n_experts, int32_t* offsets, int32_t* place, int32_t* pair_at);
void expert_product(cudaStream_t s, bool gated, const Rows& a, const Tensor& w, int n_experts, const int32_t* offsets, const int32_t* pair_at,
                    const float* weights, const Rows& out, int n_pairs, int n, int k, int top, int gate, float alpha = 0.0f, float limit = 0.0f);
// With `weights` [rows, top] every result is multiplied by its weight as it is added.
// `overwrite`: the sums are written to x instead of added.
void expert_combine(cudaStream_t s, const Rows& x, const Rows& y, const int32_t* place, int n_rows, int top, const float* weights = nullptr, bool overwrite = false);

// ---- the pieces around a state space per head whose step depends on the input (the recurrence is the matrix memory's) ----
struct StateSpaceShape {
    int n_head = 0, vdim = 0, n_state = 0, groups = 0, taps = 0;
    int64_t inner() const { return static_cast<int64_t>(n_head) * vdim; }
    int64_t group_values() const { return 2 * static_cast<int64_t>(groups) * n_state; }
    int64_t channels() const { return inner() + group_values(); }
    int64_t conv_floats() const { return static_cast<int64_t>(taps - 1) * channels(); }
    int64_t prepared_cols() const { return 2 * inner() + group_values() + n_head; }
};
// proj: float rows [z | x B C | dt]; out: float rows [x | B | C | dt x | log keep]; conv_state: the slots' [taps - 1][channels] floats.
void ssm_prepare(cudaStream_t s, const Rows& proj, const float* taps, const float* tap_bias, const float* dt_bias, const float* a_log, float* conv_state,
                 int64_t slot_stride, const int32_t* tok_seq, const int32_t* q_start, const int32_t* slots, const Rows& out, int n_tokens, int n_seq,
                 const StateSpaceShape& m, bool decode_only);
// out = (o + skip_gain[head] * skip) * silu(z) in `groups` equal parts, each over its root mean square, times weight.
void gated_group_norm(cudaStream_t s, const Rows& o, const Rows* skip, const float* skip_gain, int head, const Rows* z, const float* weight, const Rows& out,
                      int n_rows, int groups, float eps);

void sample(cudaStream_t s, const float* logits, int64_t row_stride, int n_rows, int vocab, const float* temperature,
            const int32_t* top_k, const float* top_p, const double* uniform, int32_t* out_ids);

// The two device status words (tcgen05/TMA bounded waits; the fused step's grid barrier): an asynchronous
// copy into `host2` (pinned, two ints) on `s`, and their reset.
void status_words_fetch(cudaStream_t s, int* host2);
void status_words_clear(cudaStream_t s);

}  // namespace liyab::kernels
