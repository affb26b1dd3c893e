/* The C interface of the kernel library (libliyab_b200.so).
 *
 * Plain C types only, one status return per call in the reference's numbering
 * (0 = ok; include/liyab/liyab_c_api.h:41-53), the message of the last failure on
 * the calling thread from lb_last_error().  Pointers are device pointers unless a
 * name says otherwise; `stream` is a cudaStream_t passed as void*.  Element types
 * are LB_F32 = 0 and LB_BF16 = 1.  Nothing here allocates device memory unless its
 * comment says so.
 */
#pragma once

#include <stdint.h>

#define LB_ABI_VERSION 5

#ifdef __cplusplus
extern "C" {
#endif

const char* lb_last_error(void);
int lb_abi_version(void);

/* x[t,:] = table[tokens[t],:] * scale + pos_table[positions[t],:] in 32-bit;
 * pos_table may be null.  Tables are `dtype`; x is float. */
int lb_embed_positions(int dtype, const int32_t* tokens, const int32_t* positions, const void* table,
                       const void* pos_table, float* x, int n_tokens, int width, float scale, void* stream);

/* dst[i] = src[map[i]] where map[i] >= 0; other entries of dst are left alone. */
int lb_gather_tokens(int32_t* dst, const int32_t* src, const int32_t* map, int n, void* stream);

/* y[r,:] = LayerNorm(x[rows ? rows[r] : r, :]) with 32-bit statistics; weight and
 * bias are float and may be null; y is `out_dtype`. */
int lb_layernorm(int out_dtype, const float* x, const int32_t* rows, const float* weight, const float* bias, void* y,
                 int n_rows, int width, float eps, void* stream);

/* Copies each token's key and value rows (row_stride elements apart) into the
 * layer's cache [page][K|V][kv_head][slot][head_dim] at slot_mapping[t] =
 * page * page_size + slot; a negative entry skips the token. */
int lb_kv_append(int dtype, const void* k, const void* v, int64_t row_stride, const int32_t* slot_mapping, void* cache,
                 int n_tokens, int n_kv_head, int head_dim, int page_size, void* stream);

/* Activations of the products' epilogues (`act`): 0 none, 1 GELU (tanh form), 2 GELU (erf form), 3 xIELU (z > 0: a z^2 + z/2, else
 * b (exp(z) - 1 - z) + z/2 with a = softplus(p), b = 1/2 + softplus(q)); with 3 the bias holds N + 2 floats, bias[N] = p, bias[N + 1] = q. */
/* out[M,N] = act(A[M,K] . W[N,K]^T + bias) + residual on the 32-bit units; bias
 * and residual (float, row stride ldr) may be null; out may alias residual. */
int lb_gemm_ffma(int in_dtype, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias,
                 const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act,
                 void* stream);

/* The same product for bfloat16 operands on the tcgen05 tensor cores (TMA-fed,
 * accumulator in tensor memory).  Needs K, lda and ldw to be multiples of 8 and
 * 16-byte aligned bases, else LB_ERR_UNSUPPORTED (4).  token_tile 0 picks the tile
 * (lb_gemm_tcgen05_token_tile): 16, 32, 64 put the weights on the accumulator's
 * lanes and that many tokens on its columns; 128 and 256 put 128 tokens on the
 * lanes and that many features on the columns.  out is LB_BF16 or LB_F32.
 * n_splits > 1 (at most 64 tokens only) splits K over that many blocks per tile, so
 * that a product with few output tiles still uses the whole GPU; it needs `partial`
 * (n_splits * M * N floats; `counters` is unused and may be null): the blocks write
 * their partial sums there and a second small kernel adds them in order and applies
 * the epilogue.  At most 16 splits. */
int lb_gemm_tcgen05(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias,
                    const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act,
                    int token_tile, float* partial, int* counters, int n_splits, void* stream);
int lb_gemm_tcgen05_token_tile(int M, int N);
/* The split product as a fused projection of queries, keys and values (bias only): its second half also puts the
 * features from q_dim on into the tokens' cache slots (bfloat16 pages of one layer; token i at slot_mapping[i];
 * negative: nowhere), as lb_kv_append would.  Needs a real split: lb_gemm_tcgen05_splits(M, K, n_splits) > 1. */
int lb_gemm_tcgen05_splits(int M, int K, int n_splits);
int lb_gemm_tcgen05_kv(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, void* out,
                       int64_t ldo, int M, int N, int K, float* partial, int n_splits, void* kv_cache,
                       const int32_t* slot_mapping, int q_dim, int n_kv_head, int head_dim, int page_size, void* stream);
/* lb_gemm_rows for up to 16 tokens and K up to 1024 with the activations made in the kernel: every block normalises the
 * float32 rows x itself (LayerNorm with two-pass 32-bit statistics, eps, gain and offset or null), which saves the
 * LayerNorm's launch.  Everything else as lb_gemm_rows. */
int lb_gemm_rows_normed_supports(const void* x, int64_t ldx, const void* W, int64_t ldw, int M, int N, int K);
int lb_gemm_rows_normed(int out_dtype, const float* x, int64_t ldx, const float* gain, const float* offset, float eps, const void* W,
                        int64_t ldw, const float* bias, const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N,
                        int K, int act, void* kv_cache, const int32_t* slot_mapping, int q_dim, int n_kv_head, int head_dim,
                        int page_size, void* stream);
/* The same product for 1 to 64 tokens in one launch on mma.sync (weights streamed once, no split of K over blocks,
 * no second kernel): lb_gemm_rows_supports tells whether it takes the product.  With kv_cache given (bfloat16 pages
 * of one layer), features from q_dim on are the keys and values of a fused projection and are also written to the
 * tokens' cache slots (as lb_kv_append would). */
int lb_gemm_rows_supports(const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N, int K);
int lb_gemm_rows(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias,
                 const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act, void* kv_cache,
                 const int32_t* slot_mapping, int q_dim, int n_kv_head, int head_dim, int page_size, void* stream);
/* The same product for more than 64 tokens as a persistent kernel: one block per SM walks tiles of 128 tokens x
 * feature_tile features, operands, residual and result all moved by TMA, the epilogue of a tile under the products
 * of the next.  lb_gemm_persistent_tile returns the feature tile it would choose, or 0 where the kernel does not
 * take the product (64 tokens or fewer; a row stride or base off TMA's 16-byte rule; a residual with bfloat16
 * output).  feature_tile 0 = that choice; else a multiple of 32 (float32 out) or 64 (bfloat16 out) up to 256. */
int lb_gemm_persistent_tile(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* residual,
                            int64_t ldr, const void* out, int64_t ldo, int M, int N, int K);
/* Profiling aid: from now on every launch writes eight time stamps per block (nanoseconds) to `buffer` (device
 * memory, 8 * number of SMs 64-bit words); null switches it off. */
int lb_gemm_persistent_timing(unsigned long long* buffer);
/* With kv_cache (else null and zeros): the product is a fused query/key/value projection whose features from
 * q_dim on go to the pages of the cache (token i at slot_mapping[i]; negative: nowhere) instead of `out`;
 * lb_gemm_persistent_kv_supports says for which shapes. */
int lb_gemm_persistent(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias,
                       const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act,
                       int feature_tile, void* kv_cache, const int32_t* slot_mapping, int q_dim, int n_kv_head, int head_dim,
                       int page_size, void* stream);
int lb_gemm_persistent_kv_supports(int out_dtype, int N, int act, int has_residual, int q_dim, int n_kv_head, int head_dim,
                                   int page_size);
/* Reads and clears the status word that a bounded wait sets when it runs out
 * (0: none did).  Synchronises the device. */
int lb_gemm_tcgen05_status(int* status);

/* Causal attention of every token of the step over its request's pages.
 * q: [n_tokens, n_head*head_dim] with row stride q_stride; tok_seq[t] is the row
 * of block_table (stride table_stride) of the token's request; positions[t] its
 * absolute position.  `window` says which earlier keys a query sees, here and in the four attention kernels below:
 * 0 all of them; w > 0 the w latest; -c those of the query's own chunk of c positions (chunks counted from position 0). */
int lb_paged_attention_generic(int dtype, const void* q, int64_t q_stride, const void* cache, const int32_t* tok_seq,
                               const int32_t* positions, const int32_t* block_table, int table_stride, void* out,
                               int64_t out_stride, int n_tokens, int n_head, int n_kv_head, int head_dim,
                               int page_size, float scale, int window, void* stream);

/* Decode attention, bfloat16: token i is the one new token of request i (row i of
 * positions and of block_table).  The keys are split n_splits ways; with more than
 * one split, `partial` (lb_decode_attention_scratch_floats floats) and `counters`
 * (n_seq * n_kv_head ints, zero before the first call; the kernel leaves them zero)
 * are scratch that launches on one stream may share.  lb_decode_attention_supports
 * says whether a shape is taken (head_dim 16..256 in powers of two, 1/2/4/8 query
 * heads per key/value head, page_size a power of two). */
int lb_decode_attention(const void* q, int64_t q_stride, const void* cache, const int32_t* positions,
                        const int32_t* block_table, int table_stride, void* out, int64_t out_stride, float* partial,
                        int* counters, int n_seq, int n_head, int n_kv_head, int head_dim, int page_size, float scale,
                        int window, int n_splits, void* stream);
int lb_decode_attention_supports(int n_head, int n_kv_head, int head_dim, int page_size);
/* lb_decode_attention with a penalty by distance: `distance` holds r1 [n_head] then r2 [n_head], and the score of the key d
 * positions back loses r1 ln(1 + r2 d); null: none. */
int lb_decode_attention_biased(const void* q, int64_t q_stride, const void* cache, const int32_t* positions, const int32_t* block_table,
                               int table_stride, void* out, int64_t out_stride, float* partial, int* counters, int n_seq, int n_head,
                               int n_kv_head, int head_dim, int page_size, float scale, int window, int n_splits, const float* distance,
                               void* stream);
/* The same with scores and weighted values on the tensor cores (head_dim 64 or 128, up to 16 query heads per
 * key/value head, pages of 16 positions or more); same arguments, scratch and split semantics. */
int lb_decode_attention_mma(const void* q, int64_t q_stride, const void* cache, int n_pages, const int32_t* positions,
                            const int32_t* block_table, int table_stride, void* out, int64_t out_stride, float* partial,
                            int* counters, int n_seq, int n_head, int n_kv_head, int head_dim, int page_size, float scale,
                            int window, int n_splits, void* stream);
int lb_decode_attention_mma_supports(int n_head, int n_kv_head, int head_dim, int page_size);
int lb_decode_attention_mma_biased(const void* q, int64_t q_stride, const void* cache, int n_pages, const int32_t* positions,
                                   const int32_t* block_table, int table_stride, void* out, int64_t out_stride, float* partial, int* counters,
                                   int n_seq, int n_head, int n_kv_head, int head_dim, int page_size, float scale, int window, int n_splits,
                                   const float* distance, void* stream);
int64_t lb_decode_attention_scratch_floats(int n_seq, int n_head, int head_dim, int n_splits);

/* Prefill attention, bfloat16, products on the tensor cores: request i brings the
 * tokens of rows q_start[i] .. q_start[i+1]-1 (q_start has n_seq + 1 entries), the
 * first of them at position n_past[i]; max_q_len is the longest such run.  Keys
 * and values, those of this step included, are read from the pages.
 * lb_prefill_attention_supports: head_dim 16..128 in steps of 16, page_size a
 * power of two. */
int lb_prefill_attention(const void* q, int64_t q_stride, const void* cache, const int32_t* q_start,
                         const int32_t* n_past, const int32_t* block_table, int table_stride, void* out,
                         int64_t out_stride, int n_seq, int max_q_len, int n_head, int n_kv_head, int head_dim,
                         int page_size, float scale, int window, void* stream);
int lb_prefill_attention_supports(int n_head, int n_kv_head, int head_dim, int page_size);
/* lb_prefill_attention and lb_prefill_attention_tc with a penalty by distance (`distance` as for lb_decode_attention_biased; the tcgen05
 * kernel applies it to the raw scores and so needs scale != 0). */
int lb_prefill_attention_biased(const void* q, int64_t q_stride, const void* cache, const int32_t* q_start, const int32_t* n_past,
                                const int32_t* block_table, int table_stride, void* out, int64_t out_stride, int n_seq, int max_q_len,
                                int n_head, int n_kv_head, int head_dim, int page_size, float scale, int window, const float* distance,
                                void* stream);
int lb_prefill_attention_tc_biased(const void* q, int64_t q_stride, int n_tokens, const void* cache, int n_pages, const int32_t* q_start,
                                   const int32_t* n_past, const int32_t* block_table, int table_stride, void* out, int64_t out_stride,
                                   int n_seq, int max_q_len, int n_head, int n_kv_head, int head_dim, int page_size, float scale, int window,
                                   const float* distance, void* stream);
/* The same on the tcgen05 tensor cores (head size 64, pages of 16 positions or more): TMA-fed, scores and output
 * accumulated in tensor memory.  n_tokens is the number of rows of q (and out), n_pages the number of pages of the
 * layer's cache (both bound the tensor maps). */
int lb_prefill_attention_tc(const void* q, int64_t q_stride, int n_tokens, const void* cache, int n_pages,
                            const int32_t* q_start, const int32_t* n_past, const int32_t* block_table, int table_stride,
                            void* out, int64_t out_stride, int n_seq, int max_q_len, int n_head, int n_kv_head, int head_dim,
                            int page_size, float scale, int window, void* stream);
int lb_prefill_attention_tc_supports(int n_head, int n_kv_head, int head_dim, int page_size);

/* y[r,:] = x[rows ? rows[r] : r, :] cut into `groups` equal consecutive parts, each divided by its own
 * sqrt(mean(part^2) + eps), the whole times weight (float, may be null); statistics in 32-bit; y is `out_dtype`. */
int lb_rms_groups(int out_dtype, const float* x, int64_t ldx, const int32_t* rows, const float* weight, void* y, int64_t ldy,
                  int n_rows, int width, int groups, float eps, void* stream);
/* Token shift: m[t] = h[t] + (prev - h[t]) * mix, where prev is h[t - 1] within a request's run of rows and the
 * request's state (row slots[s] of `state`, [slot, width] of `dtype`) for the run's first row; afterwards the state
 * holds the run's last row of h.  tok_seq[t] is the request of row t, q_start[s] .. q_start[s + 1] - 1 its rows.
 * decode_only: every request brings one row (the second launch, which saves longer runs' last rows, is left out). */
int lb_token_shift(int dtype, const void* h, int64_t ldh, const float* mix, void* m, int64_t ldm, void* state,
                   const int32_t* tok_seq, const int32_t* q_start, const int32_t* slots, int n_tokens, int n_seq, int decode_only,
                   int width, void* stream);
/* lb_rms_groups (to h) and lb_token_shift (to m) in one pass over the float rows x. */
int lb_rms_shift(int dtype, const float* x, int64_t ldx, const float* weight, const float* mix, void* h, int64_t ldh, void* m,
                 int64_t ldm, void* state, const int32_t* tok_seq, const int32_t* q_start, const int32_t* slots, int n_tokens,
                 int n_seq, int decode_only, int width, int groups, float eps, void* stream);
/* In place: z > 0 -> a z^2 + z/2, else b (exp(z) - 1 - z) + z/2, a = softplus(pq[0]), b = 1/2 + softplus(pq[1]). */
int lb_xielu(int dtype, void* z, int64_t ldz, int n_rows, int cols, const float* pq, void* stream);
/* x[t,:] += rms(y) * weight with y = proj . (gelu_tanh(gate . x[t,:]) * table[tokens[t],:]); gate [dim, width], proj
 * [width, dim] and table [vocab, dim] are `dtype`, x and weight float; rms divides by sqrt(mean(y^2) + eps).  g: scratch of
 * n_tokens * dim floats (two launches: the gate spread over the GPU, then a block per token). */
int lb_token_side(int dtype, float* x, int64_t ldx, const int32_t* tokens, const void* table, const void* gate, const void* proj,
                  const float* weight, float* g, int n_tokens, int width, int dim, float eps, void* stream);
/* The pieces of the same for many tokens, around two library products (x16 . gate^T and g16 . proj^T):
 * y[r, :] = bfloat16(x[r, :]);  g16[t, :] = bfloat16(gelu_tanh(pre[t, :]) * table[tokens[t], :]);  x[t, :] += rms(y[t, :]) * weight. */
int lb_rows_to_bf16(const float* x, int64_t ldx, void* y, int64_t ldy, int n_rows, int cols, void* stream);
int lb_side_gate_finish(const float* pre, int64_t ldp, const int32_t* tokens, const void* table, void* g16, int64_t ldg, int n_tokens, int dim, void* stream);
int lb_rms_add(float* x, int64_t ldx, const float* y, int64_t ldy, const float* weight, int n_rows, int width, float eps, void* stream);

/* Attention over a cache of latent rows [c (rank) | r (rot)], one row per position: pages [page][slot][rank + rot].
 * lb_latent_store: row t of d (float, [rank | rot]) -> c = d[:rank] / sqrt(mean^2 + eps) * gain; r = the last rot values
 * with the first rot_dims of them rotated (value i pairs with i + rot_dims/2, angle position * freq[i]); written at
 * slot_mapping[t] (negative: nowhere). */
int lb_latent_store(int cache_dtype, const float* d, int64_t ldd, const float* gain, const float* freq, const int32_t* positions,
                    const int32_t* slot_mapping, void* cache, int n_tokens, int rank, int rot, int rot_dims, float eps, void* stream);
/* Queries [T, H * (dim + rot)], head by head [dim | rot]: the rot part, rotated as above, goes to columns
 * h * (rank + rot) + rank .. of the wide queries (built: float queries to float or bfloat16 wide queries). */
int lb_rope_heads(int q_dtype, int wide_dtype, const void* q, int64_t ldq, const float* freq, const int32_t* positions, void* wide, int64_t ldw,
                  int n_tokens, int n_head, int dim, int rot, int rot_dims, int rank, void* stream);
/* C[t, h * c_head + n] = sum_k A[t, h * a_head + k] * B[h * b_head + k * b_k + n * b_n], n < N, k < K, for every head h;
 * 32-bit FMA whatever the element types (built: f32 f32 f32; bf16 bf16 f32; f32 bf16 bf16; f32 bf16 f32). */
int lb_head_matmul(int a_dtype, int b_dtype, int c_dtype, const void* A, int64_t lda, int64_t a_head, const void* B, int64_t b_head,
                   int64_t b_k, int64_t b_n, void* C, int64_t ldc, int64_t c_head, int M, int N, int K, int n_head, void* stream);
/* out[t, h * rank + :] = sum_j p_j c_j with p = softmax_j((wide[t, h, :] . row_j) * scale) over the rows j of the token's
 * request with 0 <= position - j < window (window 0: all j <= position). */
int lb_latent_attention(int cache_dtype, const float* wide, int64_t ldw, const void* cache, const int32_t* tok_seq,
                        const int32_t* positions, const int32_t* block_table, int table_stride, float* out, int64_t ldo, int n_tokens,
                        int n_head, int rank, int rot, int page_size, float scale, int window, void* stream);
/* Steps of few tokens, bfloat16 weights, cache and wide queries: lb_rope_heads, the keys' product per head (uk: [n_head * dim, rank]) and,
 * with cache given, lb_latent_store in one launch; qd rows are [queries | latent row] floats (the latent row only with cache). */
int lb_latent_few_supports(int dim, int rot, int rank, int vdim, int n_splits);
int lb_latent_prepare(const float* qd, int64_t ldq, const void* uk, const float* gain, const float* freq, const int32_t* positions,
                      const int32_t* slot_mapping, void* cache, void* wide, int64_t ldw, int n_tokens, int n_head, int dim, int rot, int rot_dims,
                      int rank, float eps, void* stream);
/* The merge of a split attention's parts (n_splits > 1; else `attended` is read) and the values' product per head (uv: [n_head * vdim, rank])
 * in one launch; values bfloat16. */
int lb_latent_finish(const float* attended, int64_t lda, const float* part_o, const float* part_ml, const void* uv, void* values, int64_t ldv,
                     int n_tokens, int n_head, int rank, int vdim, int n_splits, void* stream);
/* lb_head_matmul on the tensor cores: A float (rounded to bfloat16 on the way in) or bfloat16, B and C bfloat16; lb_head_matmul_mma_supports says
 * whether the strides fit its 16-byte pieces (one of b_k, b_n is 1). */
int lb_head_matmul_mma_supports(int64_t lda, int64_t a_head, int64_t b_head, int64_t b_k, int64_t b_n, int64_t ldc, int64_t c_head, int N, int K);
int lb_head_matmul_mma(int a_dtype, const void* A, int64_t lda, int64_t a_head, const void* B, int64_t b_head, int64_t b_k, int64_t b_n, void* C, int64_t ldc,
                       int64_t c_head, int M, int N, int K, int n_head, void* stream);
/* The same attention on the tensor cores for bfloat16 wide queries and cache rows (lb_latent_attention_mma_supports: rank one of
 * 32, 64, 96, 128, 192, 256, 384, 512; rot a multiple of 16).  Request i brings rows q_start[i] .. q_start[i + 1] - 1, the first at
 * position n_past[i]; max_q_len is the longest such run.  n_splits > 1 cuts every request's keys over that many blocks; it needs
 * part_o (n_splits * n_tokens * n_head * rank floats) and part_ml (n_splits * n_tokens * n_head * 2 floats), merged by a second launch
 * (or, with merge_parts 0, left for lb_latent_finish; one part is always written to out as it is). */
int lb_latent_attention_mma_supports(int n_head, int rank, int rot, int page_size);
/* The kernel for runs of tokens (64 rows a block, rank up to 256) by itself, with the attended latents out as bfloat16. */
int lb_latent_attention_rows_supports(int n_head, int rank, int rot, int page_size);
int lb_latent_attention_rows16(const void* wide, int64_t ldw, const void* cache, const int32_t* q_start, const int32_t* n_past,
                               const int32_t* block_table, int table_stride, void* out, int64_t ldo, int n_tokens, int n_seq, int max_q_len,
                               int n_head, int rank, int rot, int page_size, float scale, int window, void* stream);
int lb_latent_attention_mma(const void* wide, int64_t ldw, const void* cache, const int32_t* q_start, const int32_t* n_past,
                            const int32_t* block_table, int table_stride, float* out, int64_t ldo, float* part_o, float* part_ml,
                            int n_tokens, int n_seq, int max_q_len, int n_head, int rank, int rot, int page_size, float scale, int window,
                            int n_splits, int merge_parts, void* stream);

/* One token id per row of logits.  temperature[r] <= 0: the first maximum.
 * Otherwise top_k[r] (<= 0 or >= vocab: off), top_p[r] (>= 1: off) and the draw
 * uniform[r] in [0,1).  out_probs (optional, [n_rows, vocab]) receives the
 * distribution drawn from. */
int lb_sample(const float* logits, int64_t row_stride, int n_rows, int vocab, const float* temperature,
              const int32_t* top_k, const float* top_p, const double* uniform, int32_t* out_ids, float* out_probs,
              void* stream);

/* logits[i] = logits[i] * scale, then soft_cap * tanh(logits[i] / soft_cap) when soft_cap > 0. */
int lb_scale_softcap(float* logits, int64_t count, float scale, float soft_cap, void* stream);

/* A whole decode step of up to 16 tokens as one cooperative kernel (bfloat16, head size 64 or 128): embedding,
 * every layer (LayerNorm, fused projection with cache write, attention over the pages, output projection,
 * LayerNorm, feed-forward) and the head.  `layers_dev` holds n_layers records of lb_decode_stack_layer_bytes()
 * bytes each on the device: thirteen pointers (norm 1 gain and bias, norm 2 gain and bias, projection weight and
 * bias, output weight and bias, up weight and bias, down weight and bias, the layer's cache pages), three floats
 * (the norms' eps, the score factor), six ints (heads, key/value heads, head size, inner width, activation,
 * window) and four bytes of padding.  x, q, att, inner, partial, counters and logits are scratch of 16 rows;
 * `barrier` points at one of a pair of zeroed counters that alternate launches use in turn. */
int lb_decode_stack_layer_bytes(void);
int64_t lb_decode_stack_scratch_floats(int n_tokens, int n_head, int head_dim, int n_splits);
int lb_decode_stack(const void* layers_dev, int n_layers, int n_tokens, int width, int vocab, const void* embedding,
                    const void* pos_table, float embed_scale, const float* lnf_w, const float* lnf_b, float lnf_eps,
                    const void* head_w, const float* head_b, const int32_t* tokens, const int32_t* positions,
                    const int32_t* block_table, int table_stride, const int32_t* slot_mapping, int page_size, float* x, void* q,
                    void* att, void* inner, float* partial, int* counters, float* logits, unsigned* barrier, int max_k,
                    int head_dim, int n_splits, int unit_warps, unsigned long long* timing, void* stream);
/* Reads and clears the status word of the fused step's grid barrier.  Synchronises the device. */
int lb_decode_stack_status(int* status);

/* The two status words without a device synchronisation: an asynchronous copy into pinned host memory on
 * `stream`, and a reset on `stream`. */
int lb_gemm_tcgen05_status_async(int* host, void* stream);
int lb_gemm_tcgen05_status_clear(void* stream);
int lb_decode_stack_status_async(int* host, void* stream);
int lb_decode_stack_status_clear(void* stream);
/* Writes a status word, as a kernel whose bounded wait ran out would (for tests of the host's handling). */
int lb_gemm_tcgen05_status_set(int value);
int lb_decode_stack_status_set(int value);
/* Makes the NEXT launch meet a wait that nothing ends, once: the one-tile tcgen05 product leaves its
 * accumulator-ready barrier unsignalled; the fused step's block 0 is not counted at its first grid barrier.
 * The waits run to their limit (about two seconds), set the status word and the kernel returns. */
int lb_gemm_tcgen05_withhold_next(int on);
int lb_decode_stack_withhold_next(int on);

/* lb_gemm_rows_normed with the kind of norm as an argument: rms != 0: y = x / sqrt(mean(x^2) + eps) * (gain + gain_offset) + offset. */
int lb_gemm_rows_normed_kind(int out_dtype, const float* x, int64_t ldx, const float* gain, const float* offset, float eps, int rms, float gain_offset,
                             const void* W, int64_t ldw, const float* bias, const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N,
                             int K, int act, void* kv_cache, const int32_t* slot_mapping, int q_dim, int n_kv_head, int head_dim, int page_size,
                             void* stream);
/* lb_rms_groups with `gain_offset` added to every gain (1 for gains stored around zero). */
int lb_rms_groups_offset(int out_dtype, const float* x, int64_t ldx, const int32_t* rows, const float* weight, float gain_offset, void* y, int64_t ldy,
                         int n_rows, int width, int groups, float eps, void* stream);
/* x[r,:] += v for every row. */
int lb_add_row(float* x, int64_t ldx, const float* v, int n_rows, int width, void* stream);
/* x[r,:] += scale * sum_i y_i[r,:] / sqrt(mean(y_i[r,:]^2) + eps) * weight_i over 1 to 4 branches; `y`, `ldy`, `weight` are host
 * arrays of device pointers and strides (a weight, or the whole array, may be null). */
int lb_rms_sum_add(float* x, int64_t ldx, int n_branches, const float* const* y, const int64_t* ldy, const float* const* weight, int n_rows, int width,
                   float scale, float eps, void* stream);
/* From the float rows proj [T, ld] holding q (n_head x dim at column q_off), k (n_kv_head x dim at k_off) and v (n_kv_head x vdim at
 * v_off): with `norm`, every query and key head over its root mean square times q_weight / k_weight (float [dim], may be null).
 * Queries go to q_out [T, n_head x padded], keys and values into the cache [page][K|V][kv_head][slot][padded] at slot_mapping[t]
 * (negative: skipped; cache null: queries only); values beyond dim or vdim are zeros. */
int lb_qk_norm_store(int dtype, const float* proj, int64_t ld, int q_off, int k_off, int v_off, const float* q_weight, const float* k_weight, void* q_out,
                     int64_t ldq, void* cache, const int32_t* slot_mapping, int n_tokens, int n_head, int n_kv_head, int dim, int vdim, int padded,
                     int page_size, int norm, float eps, void* stream);
/* out[t, h * vdim + c] = f(o[t, h * o_head + c]) * gain[h * vdim + c] * act(g[t, h * vdim + c]); with `norm`, f divides a head's vdim values
 * by their root mean square; gain may be null; act 0 sigmoid, 1 silu; g float. */
int lb_head_gate(int in_dtype, int out_dtype, const void* o, int64_t ldo, int o_head, const float* g, int64_t ldg, const float* gain, void* out,
                 int64_t ld_out, int n_tokens, int n_head, int vdim, int norm, int act, float eps, void* stream);
/* mid[r, c] = act(gu[r, c]) * gu[r, inner + c]; act 0 sigmoid, 1 silu, 2 GELU (tanh form). */
int lb_gated_act(int out_dtype, const float* gu, int64_t ld, void* mid, int64_t ldm, int n_rows, int inner, int act, void* stream);

/* A matrix memory per head carried from row to row of every request: S = keep S + take k v^T, out = S^T q (see matrix_memory.cu).
 * q, k, v (and the gates' pre-activations zi, zf, one column a head) are columns of float rows `ld` apart; either `decay` [n_head]
 * (keep = decay, take = 1) or zi and zf with `cap`.  freq [rot_dims / 2] rotates the first rot_dims values of queries and keys.
 * state: [slot][n_head][tiles][dim * value_tile + dim + 1] floats, slot_stride floats a slot; tiles = ceil(vdim / value_tile).
 * chunked != 0: rows in pieces (prompt portions); 0: row by row. */
int lb_matrix_memory(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay, const float* freq,
                     int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state, int64_t slot_stride, float* out,
                     int64_t ldo, int n_seq, int n_head, int dim, int vdim, int value_tile, float q_scale, float k_scale, float cap, int chunked,
                     void* stream);

/* The same for steps with long portions, every piece of 32 rows a block of its own (three launches: the pieces' own sums, a scan over them,
 * the pieces' outputs); scratch: lb_matrix_memory_pieces_floats(..) floats. */
int64_t lb_matrix_memory_pieces_floats(int n_tokens, int n_seq, int n_head, int dim, int vdim, int value_tile);
int lb_matrix_memory_pieces(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                            const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state,
                            int64_t slot_stride, float* out, int64_t ldo, int n_tokens, int n_seq, int n_head, int dim, int vdim, int value_tile,
                            float q_scale, float k_scale, float cap, float* scratch, void* stream);

/* Routed experts (see routed_experts.cu).  ids and weights: [rows, top]. */
int lb_router_topk(int dtype, const void* h, int64_t ldh, const void* router, int32_t* ids, float* weights, int n_rows, int n_experts, int width, int top,
                   int softmax, int renormalise, void* stream);
int lb_expert_plan(const int32_t* ids, int n_pairs, int n_experts, int32_t* offsets, int32_t* place, int32_t* pair_at, void* stream);
/* gated: mid[place, :n] = act(W_e[:n] . a) * (W_e[n:2n] . a) with a = weights[pair] * h[pair / top]; else y[place, :n] = W_e . mid[place] (float). */
int lb_expert_product(int dtype, int gated, const void* a, int64_t lda, const void* w, int64_t expert_stride, const int32_t* offsets,
                      const int32_t* pair_at, const float* weights, void* out, int64_t ldo, int n_pairs, int n_experts, int n, int k, int top, int act,
                      void* stream);
/* Non-zero: bfloat16 products stay on the 32-bit units instead of the tensor cores (for comparisons). */
int lb_expert_product_set_plain(int on);
int lb_expert_combine(float* x, int64_t ldx, const float* y, int64_t ldy, const int32_t* place, int n_rows, int width, int top, void* stream);

/* lb_matrix_memory / lb_matrix_memory_pieces for heads that share queries and keys in groups: head h reads the query and key row
 * (h / qk_share); both also take the third kind of recurrence: decay, zi null and zf the log of keep itself, a number a token and head
 * (take = 1, no normaliser). */
int lb_matrix_memory_shared(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                            const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state,
                            int64_t slot_stride, float* out, int64_t ldo, int n_seq, int n_head, int dim, int vdim, int value_tile, float q_scale,
                            float k_scale, float cap, int chunked, int qk_share, void* stream);
int lb_matrix_memory_pieces_shared(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                                   const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state,
                                   int64_t slot_stride, float* out, int64_t ldo, int n_tokens, int n_seq, int n_head, int dim, int vdim, int value_tile,
                                   float q_scale, float k_scale, float cap, float* scratch, int qk_share, void* stream);

/* x[t,:] = table[tokens[t],:] * scale + e(positions[t]) with e[2i] = sin(pos w_i), e[2i+1] = cos(pos w_i), w_i = freq2[2i] + freq2[2i+1]
 * (a frequency as the sum of two floats); with `gain` (float [width]) the row is then divided by its root mean square and multiplied by it. */
int lb_embed_sinusoid(int dtype, const int32_t* tokens, const int32_t* positions, const void* table, const float* freq2, const float* gain, float* x,
                      int n_tokens, int width, float scale, float eps, void* stream);

/* lb_paged_attention_generic with a penalty by distance: `distance` holds r1 [n_head] then r2 [n_head], and the score of the key at
 * distance d loses r1 ln(1 + r2 d); null: none. */
int lb_paged_attention_generic_biased(int dtype, const void* q, int64_t q_stride, const void* cache, const int32_t* tok_seq, const int32_t* positions,
                                      const int32_t* block_table, int table_stride, void* out, int64_t out_stride, int n_tokens, int n_head,
                                      int n_kv_head, int head_dim, int page_size, float scale, int window, const float* distance, void* stream);

/* lb_qk_norm_store with a temperature on the queries: with temp_every > 0 every query value of the token at position p is multiplied by
 * 1 + temp_coef ln(floor((p + 1) / temp_every) + 1). */
int lb_qk_norm_store_tempered(int dtype, const float* proj, int64_t ld, int q_off, int k_off, int v_off, const float* q_weight, const float* k_weight,
                              void* q_out, int64_t ldq, void* cache, const int32_t* slot_mapping, int n_tokens, int n_head, int n_kv_head, int dim,
                              int vdim, int padded, int page_size, int norm, float eps, const int32_t* positions, float temp_coef, int temp_every,
                              void* stream);

/* lb_gated_act with every kind of gate: 0 sigmoid, 1 silu, 2 GELU (tanh form), 3 relu, 4 the capped form with (alpha, limit):
 * g' = min(g, limit), u' = clamp(u, -limit, limit), mid = g' sigmoid(alpha g') (u' + 1). */
int lb_gated_act_kind(int out_dtype, const float* gu, int64_t ld, void* mid, int64_t ldm, int n_rows, int inner, int act, float alpha, float limit,
                      void* stream);

/* The router with a bias (float [n_experts], added to the sums before the choice); the experts' products with every kind of gate and,
 * with `weights` null, no weight on the experts' input; the sum of a row's results each times its weight. */
int lb_router_topk_biased(int dtype, const void* h, int64_t ldh, const void* router, const float* bias, int32_t* ids, float* weights, int n_rows,
                          int n_experts, int width, int top, int softmax, int renormalise, void* stream);
int lb_expert_product_kind(int dtype, int gated, const void* a, int64_t lda, const void* w, int64_t expert_stride, const int32_t* offsets,
                           const int32_t* pair_at, const float* weights, void* out, int64_t ldo, int n_pairs, int n_experts, int n, int k, int top, int act,
                           float alpha, float limit, void* stream);
int lb_expert_combine_weighted(float* x, int64_t ldx, const float* y, int64_t ldy, const int32_t* place, const float* weights, int n_rows, int width,
                               int top, void* stream);

/* The pieces around a state space per head (see state_space.cu).  proj: float rows [z | x B C | dt] with the convolution's channels at
 * column xbc_off and dt at dt_off; taps [channels, n_taps]; state: + slot * slot_stride floats, [n_taps - 1][channels];
 * out rows: [x (n_head vdim) | B C (group_values) | dt x (n_head vdim) | -exp(a_log) dt (n_head)].  decode_only: every request brings one
 * row, whose inputs enter the state in the same launch. */
int lb_ssm_prepare(const float* proj, int64_t ld, int xbc_off, int dt_off, const float* taps, const float* tap_bias, const float* dt_bias,
                   const float* a_log, float* state, int64_t slot_stride, const int32_t* tok_seq, const int32_t* q_start, const int32_t* slots, float* out,
                   int64_t ldo, int n_tokens, int n_seq, int n_head, int vdim, int group_values, int n_taps, int decode_only, void* stream);
/* out = (o + skip_gain[c / head] * skip) * silu(z), cut into `groups` equal parts each over its own root mean square, times weight;
 * skip, z and weight may be null. */
int lb_gated_group_norm(int out_dtype, const float* o, int64_t ldo, const float* skip, int64_t lds, const float* skip_gain, int head, const float* z,
                        int64_t ldz, const float* weight, void* out, int64_t ld_out, int n_rows, int width, int groups, float eps, void* stream);

/* lb_paged_attention_generic_biased with a sink a head: `sink` [n_head] (or null); exp(sink[h]) joins the divisor of head h's softmax as it is
 * (not scaled), with no key and no value. */
int lb_paged_attention_generic_sink(int dtype, const void* q, int64_t q_stride, const void* cache, const int32_t* tok_seq, const int32_t* positions,
                                    const int32_t* block_table, int table_stride, void* out, int64_t out_stride, int n_tokens, int n_head,
                                    int n_kv_head, int head_dim, int page_size, float scale, int window, const float* distance, const float* sink,
                                    void* stream);

/* The bfloat16 attention kernels with a sink a head (`sink` [n_head] or null, as lb_paged_attention_generic_sink's): it joins the divisor once,
 * where a row's keys (or a request's key ranges) have all been summed. */
int lb_decode_attention_sink(const void* q, int64_t q_stride, const void* cache, const int32_t* positions, const int32_t* block_table,
                             int table_stride, void* out, int64_t out_stride, float* partial, int* counters, int n_seq, int n_head,
                             int n_kv_head, int head_dim, int page_size, float scale, int window, int n_splits, const float* distance,
                             const float* sink, void* stream);
int lb_decode_attention_mma_sink(const void* q, int64_t q_stride, const void* cache, int n_pages, const int32_t* positions,
                                 const int32_t* block_table, int table_stride, void* out, int64_t out_stride, float* partial, int* counters,
                                 int n_seq, int n_head, int n_kv_head, int head_dim, int page_size, float scale, int window, int n_splits,
                                 const float* distance, const float* sink, void* stream);
int lb_prefill_attention_sink(const void* q, int64_t q_stride, const void* cache, const int32_t* q_start, const int32_t* n_past,
                              const int32_t* block_table, int table_stride, void* out, int64_t out_stride, int n_seq, int max_q_len,
                              int n_head, int n_kv_head, int head_dim, int page_size, float scale, int window, const float* distance,
                              const float* sink, void* stream);
int lb_prefill_attention_tc_sink(const void* q, int64_t q_stride, int n_tokens, const void* cache, int n_pages, const int32_t* q_start,
                                 const int32_t* n_past, const int32_t* block_table, int table_stride, void* out, int64_t out_stride,
                                 int n_seq, int max_q_len, int n_head, int n_kv_head, int head_dim, int page_size, float scale, int window,
                                 const float* distance, const float* sink, void* stream);

/* What attention over latent rows may have besides its sizes.  sink [n_head]: exp(sink[h]) joins the divisor of head h's softmax (no key, no
 * value, not scaled).  gate: one float a (token, head) at gate[t * ldg + h]; the head's result is multiplied by sigmoid of it.  interleaved:
 * the rotation pairs value 2i with 2i + 1 instead of i with i + rot_dims / 2.  latent (lb_latent_prepare_ext): the rows [latent | rotated key],
 * ldl floats apart, where they do not follow the queries in qd.  A null pointer to the struct means none of it. */
typedef struct lb_latent_extras {
    const float* sink;
    const float* gate;
    int64_t ldg;
    int interleaved;
    const float* latent;
    int64_t ldl;
} lb_latent_extras;
int lb_latent_store_ext(int cache_dtype, const float* d, int64_t ldd, const float* gain, const float* freq, const int32_t* positions,
                        const int32_t* slot_mapping, void* cache, int n_tokens, int rank, int rot, int rot_dims, float eps, const lb_latent_extras* extras,
                        void* stream);
int lb_rope_heads_ext(int q_dtype, int wide_dtype, const void* q, int64_t ldq, const float* freq, const int32_t* positions, void* wide, int64_t ldw,
                      int n_tokens, int n_head, int dim, int rot, int rot_dims, int rank, int interleaved, void* stream);
int lb_latent_prepare_ext(const float* qd, int64_t ldq, const void* uk, const float* gain, const float* freq, const int32_t* positions,
                          const int32_t* slot_mapping, void* cache, void* wide, int64_t ldw, int n_tokens, int n_head, int dim, int rot, int rot_dims,
                          int rank, float eps, const lb_latent_extras* extras, void* stream);
/* Sink and gate act here where the keys were split (n_splits > 1); with one part only the gate does (the attention applied the sink). */
int lb_latent_finish_ext(const float* attended, int64_t lda, const float* part_o, const float* part_ml, const void* uv, void* values, int64_t ldv,
                         int n_tokens, int n_head, int rank, int vdim, int n_splits, const lb_latent_extras* extras, void* stream);
int lb_latent_attention_ext(int cache_dtype, const float* wide, int64_t ldw, const void* cache, const int32_t* tok_seq, const int32_t* positions,
                            const int32_t* block_table, int table_stride, float* out, int64_t ldo, int n_tokens, int n_head, int rank, int rot,
                            int page_size, float scale, int window, const lb_latent_extras* extras, void* stream);
int lb_latent_attention_rows16_ext(const void* wide, int64_t ldw, const void* cache, const int32_t* q_start, const int32_t* n_past,
                                   const int32_t* block_table, int table_stride, void* out, int64_t ldo, int n_tokens, int n_seq, int max_q_len,
                                   int n_head, int rank, int rot, int page_size, float scale, int window, const lb_latent_extras* extras, void* stream);
int lb_latent_attention_mma_ext(const void* wide, int64_t ldw, const void* cache, const int32_t* q_start, const int32_t* n_past,
                                const int32_t* block_table, int table_stride, float* out, int64_t ldo, float* part_o, float* part_ml, int n_tokens,
                                int n_seq, int max_q_len, int n_head, int rank, int rot, int page_size, float scale, int window, int n_splits,
                                int merge_parts, const lb_latent_extras* extras, void* stream);

/* lb_matrix_memory_shared / lb_matrix_memory_pieces_shared with an activation on queries, keys and values as the kernels read them
 * (qkv_act: -1 none, 0 sigmoid, 1 silu, 2 GELU tanh form, 3 relu), before rotation and scales. */
int lb_matrix_memory_activated(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                               const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state,
                               int64_t slot_stride, float* out, int64_t ldo, int n_seq, int n_head, int dim, int vdim, int value_tile, float q_scale,
                               float k_scale, float cap, int chunked, int qk_share, int qkv_act, void* stream);
int lb_matrix_memory_pieces_activated(const float* q, const float* k, const float* v, const float* zi, const float* zf, int64_t ld, const float* decay,
                                      const float* freq, int rot_dims, const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state,
                                      int64_t slot_stride, float* out, int64_t ldo, int n_tokens, int n_seq, int n_head, int dim, int vdim, int value_tile,
                                      float q_scale, float k_scale, float cap, float* scratch, int qk_share, int qkv_act, void* stream);

/* lb_rms_sum_add that also leaves the new rows of x rounded to bfloat16 in x16 (rows ld16 apart; null: as lb_rms_sum_add), for the part that
 * reads the stream next. */
int lb_rms_sum_add_rounded(float* x, int64_t ldx, int n_branches, const float* const* y, const int64_t* ldy, const float* const* weight, int n_rows,
                           int width, float scale, float eps, void* x16, int64_t ld16, void* stream);
/* lb_router_table and lb_expert_plan in one launch: ids and weights [n_rows, top] are filled from the table, then the plan is made from them. */
int lb_expert_plan_table(const int32_t* tokens, const int32_t* table, int vocab, int top, int32_t* ids, float* weights, int n_rows, int n_experts,
                         int32_t* offsets, int32_t* place, int32_t* pair_at, void* stream);
/* lb_expert_combine_weighted that, with `overwrite`, writes the rows' sums to x instead of adding them. */
int lb_expert_combine_into(float* x, int64_t ldx, const float* y, int64_t ldy, const int32_t* place, const float* weights, int n_rows, int width, int top,
                           int overwrite, void* stream);

/* Queries, keys and values of a float projection on their way to attention (see rotary_rows.cu).  norm_mode 0 none, 1 every head over its
 * root mean square (gains [dim]), 2 all of q and all of k each over one root mean square (gains [n_head * dim], [n_kv_head * dim]); then the
 * first rot_dims values of every query and key head rotated (value i with i + rot_dims / 2, angle positions[t] * freq[i]).  Values: with
 * v_first_in, v = (1 - lambda[0]) v + lambda[0] v_first_in[t]; with v_first_out the row's own values are left there (rows ldv floats apart,
 * n_kv_head * vdim values).  Destinations as lb_qk_norm_store's. */
int lb_qkv_rotary_store(int dtype, const float* proj, int64_t ld, int q_off, int k_off, int v_off, const float* q_weight, const float* k_weight,
                        void* q_out, int64_t ldq, void* cache, const int32_t* slot_mapping, int n_tokens, int n_head, int n_kv_head, int dim, int vdim,
                        int padded, int page_size, int norm_mode, float eps, const int32_t* positions, const float* freq, int rot_dims,
                        const float* v_first_in, float* v_first_out, int64_t ldv, const float* lambda, void* stream);
/* out[r, c] = o[r, c] / sqrt(mean(o[r, :]^2) + eps) * gain[c] * act(g[r, c]); gain and g may be null; act 0 sigmoid, 1 silu. */
int lb_row_norm_gate(int out_dtype, const float* o, int64_t ldo, const float* g, int64_t ldg, const float* gain, void* out, int64_t ld_out, int n_rows,
                     int width, int act, float eps, void* stream);
/* x[r, c] = act(x[r, c]) for c < cols, in place; act 0 sigmoid, 1 silu, 2 GELU (tanh form), 3 relu. */
int lb_activate_columns(float* x, int64_t ld, int n_rows, int cols, int act, void* stream);
/* ids[r, j] = table[tokens[r], j] and weights[r, j] = 1 / top: a row's experts looked up by its token id (table int32 [vocab, top]). */
int lb_router_table(const int32_t* tokens, const int32_t* table, int32_t* ids, float* weights, int n_rows, int top, int n_experts, int vocab, void* stream);

#ifdef __cplusplus
}
#endif
