#include "kernels.h"

#include <cstdlib>
#include <algorithm>

#include "../csrc/api.h"

namespace liyab::kernels {

std::atomic<uint64_t> launches{0};

void check(int status, const char* what) {
    launches.fetch_add(1, std::memory_order_relaxed);
    if (status == 0) return;
    Code code = Code::Internal;
    if (status >= 1 && status <= 10) code = static_cast<Code>(status);
    throw Error(code, std::format("{}: {}", what, lb_last_error()));
}

int activation_from_name(const std::string& name) {
    if (name == "none") return kNone;
    if (name == "gelu_tanh") return kGeluTanh;
    if (name == "gelu_erf") return kGeluErf;
    if (name == "xielu") return kXielu;
    if (name == "relu2") return kRelu2;
    throw unsupported("activation '{}' is not supported; supported: gelu_tanh, gelu_erf, xielu, relu2, none", name);
}

namespace {
// Which of the bfloat16 attention kernels run heads with a sink: 1 scalar decode, 2 tensor-core decode, 4 prefill on mma.sync, 8 prefill on
// tcgen05 (all of them; LIYAB_B200_SINK_KERNELS in the environment, read once, sends such heads to the generic kernel instead, for comparisons).
const int kSinkKernels = [] {
    const char* v = std::getenv("LIYAB_B200_SINK_KERNELS");
    return v != nullptr ? std::atoi(v) : 15;
}();
// The latent attention's extras as the kernels take them; `gate`: one float a (token, head), or null.
lb_latent_extras latent_extras(const LatentShape& a, const Rows* gate, bool with_sink = true, const Rows* latent = nullptr) {
    lb_latent_extras x{};
    x.sink = with_sink ? a.sink : nullptr;
    if (gate != nullptr && gate->data != nullptr) {
        if (gate->dtype != DType::F32 || gate->cols != a.n_head) throw invalid_argument("latent attention: the gate is one float a head");
        x.gate = gate->f32();
        x.ldg = gate->stride;
    }
    x.interleaved = a.interleaved ? 1 : 0;
    if (latent != nullptr && latent->data != nullptr) {
        if (latent->dtype != DType::F32 || latent->cols != a.rank + a.rot) throw invalid_argument("latent attention: the latent rows must be float32 [tokens, rank + rot]");
        x.latent = latent->f32();
        x.ldl = latent->stride;
    }
    return x;
}
int code(DType t, const char* what) {
    if (t == DType::F32) return 0;
    if (t == DType::BF16) return 1;
    throw invalid_argument("{} has dtype {}; the kernels take float32 and bfloat16", what, dtype_name(t));
}
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
void check_product(const Rows& a, const Tensor& w, const Rows& out, const Rows* residual) {
    if (w.shape.size() != 2 || a.cols != w.dim(1) || out.cols != w.dim(0))
        throw invalid_argument("gemm: shapes do not fit: a [{}, {}], w {}, out [{}, {}]", a.rows, a.cols, shape_text(w.shape),
                               out.rows, out.cols);
    if (a.dtype != w.dtype) throw invalid_argument("gemm: a is {} but w is {}", dtype_name(a.dtype), dtype_name(w.dtype));
    if (residual != nullptr && (residual->cols != w.dim(0) || residual->dtype != DType::F32))
        throw invalid_argument("gemm: residual has the wrong shape or type");
}
}  // namespace



void embed_positions(cudaStream_t s, const int32_t* tokens, const int32_t* positions, const Tensor& table,
                     const Tensor* pos_table, const Rows& x, int n_tokens, float scale) {
    const int width = static_cast<int>(table.dim(1));
    if (pos_table != nullptr && (pos_table->dtype != table.dtype || pos_table->dim(1) != width))
        throw invalid_argument("embed: the position table does not match the embedding table");
    if (x.cols != width || x.stride != width || x.dtype != DType::F32 || x.rows < n_tokens)
        throw invalid_argument("embed: output buffer has the wrong shape");
    check(lb_embed_positions(code(table.dtype, "table"), tokens, positions, table.data, pos_table ? pos_table->data : nullptr,
                             x.f32(), n_tokens, width, scale, s), "embed_positions");
}

void embed_sinusoid(cudaStream_t s, const int32_t* tokens, const int32_t* positions, const Tensor& table, const float* freq2, const float* gain,
                    const Rows& x, int n_tokens, float scale, float eps) {
    if (x.dtype != DType::F32 || table.shape.size() != 2 || table.dim(1) != x.cols || x.stride != x.cols) throw invalid_argument("embed: the stream does not fit the table");
    check(lb_embed_sinusoid(code(table.dtype, "table"), tokens, positions, table.data, freq2, gain, x.f32(), n_tokens, static_cast<int>(x.cols), scale, eps, s),
          "embed_sinusoid");
}

void gather_tokens(cudaStream_t s, int32_t* dst, const int32_t* src, const int32_t* map, int n) {
    check(lb_gather_tokens(dst, src, map, n, s), "gather_tokens");
}

void layernorm(cudaStream_t s, const Rows& x, const int32_t* rows, const float* weight, const float* bias, const Rows& out,
               int n_rows, float eps) {
    if (x.dtype != DType::F32 || x.stride != x.cols || out.stride != out.cols || out.cols != x.cols || out.rows < n_rows)
        throw invalid_argument("layernorm: buffers must be contiguous [rows, width]");
    check(lb_layernorm(code(out.dtype, "out"), x.f32(), rows, weight, bias, out.data, n_rows, static_cast<int>(x.cols), eps, s),
          "layernorm");
}

void kv_append(cudaStream_t s, const Rows& k, const Rows& v, const int32_t* slot_mapping, void* cache, DType cache_dtype,
               int n_tokens, int n_kv_head, int head_dim, int page_size) {
    if (k.stride != v.stride || k.dtype != cache_dtype || v.dtype != cache_dtype)
        throw invalid_argument("kv_append: k and v must share a row stride and match the cache type");
    check(lb_kv_append(code(cache_dtype, "cache"), k.data, v.data, k.stride, slot_mapping, cache, n_tokens, n_kv_head, head_dim,
                       page_size, s), "kv_append");
}

void scale_softcap(cudaStream_t s, float* logits, int64_t count, float scale, float soft_cap) {
    check(lb_scale_softcap(logits, count, scale, soft_cap, s), "scale_softcap");
}

bool tcgen05_accepts(const Rows& a, const Tensor& w) {
    return a.dtype == DType::BF16 && w.dtype == DType::BF16 && w.shape.size() == 2 && w.dim(1) % 8 == 0 && a.stride % 8 == 0 &&
           aligned16(a.data) && aligned16(w.data);
}

bool gemm_rows_normed_supports(const Runtime& rt, const Rows& x, const Tensor& w, int m) {
    return rt.dtype == DType::BF16 && x.dtype == DType::F32 && w.dtype == DType::BF16 && x.cols == w.dim(1) &&
           lb_gemm_rows_normed_supports(x.data, x.stride, w.data, w.dim(1), m, static_cast<int>(w.dim(0)), static_cast<int>(w.dim(1))) != 0;
}

void gemm_rows_normed(cudaStream_t s, const Rows& x, const float* gain, const float* offset, float eps, const Tensor& w, const float* bias,
                      const Rows& out, int m, int act, const Rows* residual, const KvDestination* kv, bool rms, float gain_offset) {
    check(lb_gemm_rows_normed_kind(code(out.dtype, "out"), x.f32(), x.stride, gain, offset, eps, rms ? 1 : 0, gain_offset, w.data, w.dim(1), bias,
                              residual ? residual->f32() : nullptr, residual ? residual->stride : 0, out.data, out.stride, m,
                              static_cast<int>(w.dim(0)), static_cast<int>(w.dim(1)), act, kv ? kv->cache : nullptr,
                              kv ? kv->slot_mapping : nullptr, kv ? kv->q_dim : 0, kv ? kv->n_kv_head : 0, kv ? kv->head_dim : 0,
                              kv ? kv->page_size : 0, s),
          "gemm_rows_normed");
}

bool gemm_rows_takes(int m, int n, int k, int sm_count) {
    if (m < 1 || m > 64) return false;
    if (k <= kRowsMaxK) return true;
    if (m > 16 || k > 4096) return false;
    const int groups = (n + 7) / 8, blocks = std::min(groups, std::max(1, sm_count)), per_block = (groups + blocks - 1) / blocks;
    return per_block <= (k <= 2048 ? 2 : 1);          // the groups a block holds in its registers at that K
}

int gemm_splits(int m, int n, int k) {
    // How many ways K is split for a product of few tokens: enough blocks for most of the GPU's SMs.
    if (m > 64 || m <= 0) return 1;
    const int tiles = (n + 127) / 128, k_blocks = (k + 63) / 64;
    return std::max(1, std::min({k_blocks, 16, (96 + tiles - 1) / tiles}));
}

void gemm_ffma(cudaStream_t s, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m, int act,
               const Rows* residual) {
    check_product(a, w, out, residual);
    check(lb_gemm_ffma(code(a.dtype, "a"), code(out.dtype, "out"), a.data, a.stride, w.data, w.dim(1), bias,
                       residual ? residual->f32() : nullptr, residual ? residual->stride : 0, out.data, out.stride, m,
                       static_cast<int>(w.dim(0)), static_cast<int>(w.dim(1)), act, s), "gemm_ffma");
}

void gemm_tcgen05(cudaStream_t s, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m, int act,
                  const Rows* residual, float* partial, int n_splits) {
    check_product(a, w, out, residual);
    check(lb_gemm_tcgen05(code(out.dtype, "out"), a.data, a.stride, w.data, w.dim(1), bias, residual ? residual->f32() : nullptr,
                          residual ? residual->stride : 0, out.data, out.stride, m, static_cast<int>(w.dim(0)),
                          static_cast<int>(w.dim(1)), act, 0, partial, nullptr, n_splits, s), "gemm_tcgen05");
}

bool gemm_rows_supports(const Rows& a, const Tensor& w, int m) {
    if (!tcgen05_accepts(a, w)) return false;
    return lb_gemm_rows_supports(a.data, a.stride, w.data, w.dim(1), m, static_cast<int>(w.dim(0)), static_cast<int>(w.dim(1))) != 0;
}

void gemm_rows(cudaStream_t s, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m, int act,
               const Rows* residual, const KvDestination* kv) {
    check_product(a, w, out, residual);
    const KvDestination none;
    const KvDestination& d = kv ? *kv : none;
    check(lb_gemm_rows(code(out.dtype, "out"), a.data, a.stride, w.data, w.dim(1), bias, residual ? residual->f32() : nullptr,
                       residual ? residual->stride : 0, out.data, out.stride, m, static_cast<int>(w.dim(0)),
                       static_cast<int>(w.dim(1)), act, d.cache, d.slot_mapping, d.q_dim, d.n_kv_head, d.head_dim, d.page_size, s),
          "gemm_rows");
}

int gemm_persistent_tile(const Rows& a, const Tensor& w, const Rows& out, int m, const Rows* residual) {
    if (!tcgen05_accepts(a, w)) return 0;
    return lb_gemm_persistent_tile(code(out.dtype, "out"), a.data, a.stride, w.data, w.dim(1), residual ? residual->f32() : nullptr,
                                   residual ? residual->stride : 0, out.data, out.stride, m, static_cast<int>(w.dim(0)),
                                   static_cast<int>(w.dim(1)));
}

bool gemm_persistent_kv_supports(const Tensor& w, const Rows& out, const KvDestination& kv) {
    return lb_gemm_persistent_kv_supports(code(out.dtype, "out"), static_cast<int>(w.dim(0)), kNone, 0, kv.q_dim, kv.n_kv_head,
                                          kv.head_dim, kv.page_size) != 0;
}

void gemm_persistent(cudaStream_t s, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m, int act,
                     const Rows* residual, const KvDestination* kv) {
    check_product(a, w, out, residual);
    const KvDestination none;
    const KvDestination& d = kv ? *kv : none;
    check(lb_gemm_persistent(code(out.dtype, "out"), a.data, a.stride, w.data, w.dim(1), bias, residual ? residual->f32() : nullptr,
                             residual ? residual->stride : 0, out.data, out.stride, m, static_cast<int>(w.dim(0)),
                             static_cast<int>(w.dim(1)), act, 0, d.cache, d.slot_mapping, d.q_dim, d.n_kv_head, d.head_dim,
                             d.page_size, s), "gemm_persistent");
}

void linear(const Runtime& rt, Workspace* ws, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m,
            int act, const Rows* residual) {
    if (tcgen05_accepts(a, w)) {
        const int n = static_cast<int>(w.dim(0)), k = static_cast<int>(w.dim(1));
        if (m > 64 && gemm_persistent_tile(a, w, out, m, residual) > 0)
            return gemm_persistent(rt.stream, a, w, bias, out, m, act, residual, nullptr);
        // Up to 64 tokens: one launch on mma.sync where every block can afford to fetch all activations (measured on
        // B200, 64 tokens: 6-7 us against 8-9 us for K = 768; for K = 3072 the 393 KB of activations per block cost
        // more than the split of K saves: 13 us against 8 us).
        if (gemm_rows_takes(m, n, k, rt.sm_count) && gemm_rows_supports(a, w, m))
            return gemm_rows(rt.stream, a, w, bias, out, m, act, residual, nullptr);
        const int splits = ws != nullptr ? gemm_splits(m, n, k) : 1;
        float* partial = nullptr;
        if (splits > 1) partial = static_cast<float*>(ws->flat("gemm.partial", static_cast<int64_t>(splits) * m * n, DType::F32));
        return gemm_tcgen05(rt.stream, a, w, bias, out, m, act, residual, partial, splits);
    }
    gemm_ffma(rt.stream, a, w, bias, out, m, act, residual);
}

bool linear_with_cache(const Runtime& rt, Workspace* ws, const Rows& a, const Tensor& w, const float* bias, const Rows& out, int m,
                       const KvDestination& kv) {
    if (ws == nullptr || m > 64 || !tcgen05_accepts(a, w)) return false;
    const int n = static_cast<int>(w.dim(0)), k = static_cast<int>(w.dim(1));
    if (gemm_rows_takes(m, n, k, rt.sm_count) && gemm_rows_supports(a, w, m)) return false;          // that kernel has a cache epilogue of its own
    const int splits = gemm_splits(m, n, k);
    if (lb_gemm_tcgen05_splits(m, k, splits) <= 1) return false;
    check_product(a, w, out, nullptr);
    float* partial = static_cast<float*>(ws->flat("gemm.partial", static_cast<int64_t>(splits) * m * n, DType::F32));
    check(lb_gemm_tcgen05_kv(code(out.dtype, "out"), a.data, a.stride, w.data, w.dim(1), bias, out.data, out.stride, m, n, k, partial, splits,
                             kv.cache, kv.slot_mapping, kv.q_dim, kv.n_kv_head, kv.head_dim, kv.page_size, rt.stream),
          "gemm_tcgen05_kv");
    return true;
}

// Heads with a sink run on the kernels that take one (kSinkKernels says which); the others decline such a shape.
bool decode_scalar_supports(const AttentionShape& a) { return (a.sink == nullptr || (kSinkKernels & 1)) && lb_decode_attention_supports(a.n_head, a.n_kv_head, a.head_dim, a.page_size) != 0; }
bool decode_mma_supports(const AttentionShape& a) { return (a.sink == nullptr || (kSinkKernels & 2)) && lb_decode_attention_mma_supports(a.n_head, a.n_kv_head, a.head_dim, a.page_size) != 0; }
bool prefill_supports(const AttentionShape& a) { return (a.sink == nullptr || (kSinkKernels & 4)) && lb_prefill_attention_supports(a.n_head, a.n_kv_head, a.head_dim, a.page_size) != 0; }
bool prefill_tc_supports(const AttentionShape& a) { return (a.sink == nullptr || (kSinkKernels & 8)) && lb_prefill_attention_tc_supports(a.n_head, a.n_kv_head, a.head_dim, a.page_size) != 0; }

int decode_splits(int n_seq, int n_kv_head, int max_context, bool tensor_cores) {
    // How many ways each request's keys are split.  Scalar kernel: enough blocks for about four full waves of
    // the GPU, but no ranges shorter than 128 keys at the longest context.  Tensor-core kernel: a block gets through
    // its keys far faster, so fewer and longer ranges (about 450 blocks, 96 keys or more each; up to eight ranges merge
    // inside a cluster, which made shorter ranges pay: GPT-2 small, one request, 278 -> 270 us a step); from 32 requests
    // of 12 heads on, none.  A function of the batch's shape only, so a captured step and an eager one split alike.
    const int work = std::max(1, n_seq * n_kv_head);
    if (tensor_cores) {
        const int cap = max_context ? std::max(1, max_context / 96) : 32;
        const int n = std::max(1, std::min({32, cap, 444 / work}));
        return n > 8 && n < 16 ? 8 : n;          // eight ranges that merge inside a cluster beat a few more that cannot
    }
    const int cap = max_context ? std::max(1, max_context / 128) : 32;
    return std::max(1, std::min({32, cap, (2960 + work - 1) / work}));
}

void attention_generic(cudaStream_t s, DType dtype, const Rows& q, const void* cache, const int32_t* tok_seq,
                       const int32_t* positions, const int32_t* block_table, int table_width, const Rows& out, int n_tokens,
                       const AttentionShape& a) {
    if (q.dtype != dtype || out.dtype != dtype) throw invalid_argument("attention: q, cache and out must have one element type");
    check(lb_paged_attention_generic_sink(code(dtype, "cache"), q.data, q.stride, cache, tok_seq, positions, block_table, table_width,
                                          out.data, out.stride, n_tokens, a.n_head, a.n_kv_head, a.head_dim, a.page_size, a.scale,
                                          a.mask(), a.distance, a.sink, s), "paged_attention_generic");
}

void decode_attention(cudaStream_t s, bool tensor_cores, const Rows& q, const void* cache, int n_pages, const int32_t* positions,
                      const int32_t* block_table, int table_width, const Rows& out, float* partial, int* counters, int n_seq,
                      const AttentionShape& a, int n_splits) {
    if (q.dtype != DType::BF16 || out.dtype != DType::BF16) throw invalid_argument("decode attention takes bfloat16 only");
    if (q.stride % 8 != 0 || !aligned16(q.data))
        throw invalid_argument("decode attention: q rows must be 16-byte aligned and a multiple of 8 elements apart");
    if (n_splits > 1 && (partial == nullptr || counters == nullptr))
        throw invalid_argument("decode attention: scratch buffers are missing");
    if (tensor_cores)
        check(lb_decode_attention_mma_sink(q.data, q.stride, cache, n_pages, positions, block_table, table_width, out.data, out.stride,
                                           partial, counters, n_seq, a.n_head, a.n_kv_head, a.head_dim, a.page_size, a.scale, a.mask(),
                                           n_splits, a.distance, a.sink, s), "decode_attention_mma");
    else
        check(lb_decode_attention_sink(q.data, q.stride, cache, positions, block_table, table_width, out.data, out.stride, partial,
                                       counters, n_seq, a.n_head, a.n_kv_head, a.head_dim, a.page_size, a.scale, a.mask(), n_splits, a.distance, a.sink, s),
              "decode_attention");
}

void prefill_attention(const Runtime& rt, const Rows& q, int n_tokens, const void* cache, int n_pages, const int32_t* q_start,
                       const int32_t* n_past, const int32_t* block_table, int table_width, const Rows& out, int n_seq,
                       int max_q_len, const AttentionShape& a) {
    if (q.dtype != DType::BF16 || out.dtype != DType::BF16) throw invalid_argument("prefill attention takes bfloat16 only");
    // Measured on B200: the tcgen05 kernel walks a long tile's keys about 1.4x faster, but runs one block per SM,
    // so it wins while the launch is bound by its longest blocks (up to four blocks per SM) and loses to the
    // mma.sync kernel's several blocks per SM beyond that.
    const int64_t blocks = static_cast<int64_t>(n_seq) * a.n_head * ((max_q_len + 127) / 128);
    const bool tc = prefill_tc_supports(a) && q.stride % 8 == 0 && out.stride % 8 == 0 && aligned16(q.data) &&
                    aligned16(out.data) && blocks <= 4 * static_cast<int64_t>(rt.sm_count) && a.scale > 0;     // it takes the maximum of the raw scores
    if (tc)
        check(lb_prefill_attention_tc_sink(q.data, q.stride, n_tokens, cache, n_pages, q_start, n_past, block_table, table_width,
                                           out.data, out.stride, n_seq, max_q_len, a.n_head, a.n_kv_head, a.head_dim, a.page_size,
                                           a.scale, a.mask(), a.distance, a.sink, rt.stream), "prefill_attention_tc");
    else
        check(lb_prefill_attention_sink(q.data, q.stride, cache, q_start, n_past, block_table, table_width, out.data, out.stride, n_seq,
                                        max_q_len, a.n_head, a.n_kv_head, a.head_dim, a.page_size, a.scale, a.mask(), a.distance, a.sink, rt.stream),
              "prefill_attention");
}

void rms_groups(cudaStream_t s, const Rows& x, const int32_t* rows, const float* weight, const Rows& out, int n_rows, int groups, float eps, float gain_offset) {
    if (x.dtype != DType::F32 || out.cols != x.cols || out.rows < n_rows) throw invalid_argument("rms norm: buffers must be [rows, width], the input float32");
    check(lb_rms_groups_offset(code(out.dtype, "out"), x.f32(), x.stride, rows, weight, gain_offset, out.data, out.stride, n_rows, static_cast<int>(x.cols),
                               groups, eps, s), "rms_groups");
}

void add_row(cudaStream_t s, const Rows& x, const float* v, int n_rows) {
    if (x.dtype != DType::F32 || x.rows < n_rows) throw invalid_argument("add_row: the rows must be float32");
    check(lb_add_row(x.f32(), x.stride, v, n_rows, static_cast<int>(x.cols), s), "add_row");
}

void rms_sum_add(cudaStream_t s, const Rows& x, const std::vector<Rows>& y, const std::vector<const float*>& weight, int n_rows, float scale, float eps,
                 const Rows* rounded) {
    if (rounded != nullptr && (rounded->dtype != DType::BF16 || rounded->cols != x.cols)) throw invalid_argument("rms_sum_add: the rounded rows are bfloat16 of the stream's width");
    if (y.empty() || y.size() > 4 || weight.size() != y.size() || x.dtype != DType::F32) throw invalid_argument("rms_sum_add: one to four float branches with a weight each");
    const float* ys[4];
    int64_t ld[4];
    for (size_t i = 0; i < y.size(); ++i) {
        if (y[i].dtype != DType::F32 || y[i].cols != x.cols || y[i].rows < n_rows) throw invalid_argument("rms_sum_add: branch {} does not fit the rows", i);
        ys[i] = y[i].f32();
        ld[i] = y[i].stride;
    }
    check(lb_rms_sum_add_rounded(x.f32(), x.stride, static_cast<int>(y.size()), ys, ld, weight.data(), n_rows, static_cast<int>(x.cols), scale, eps,
                                 rounded != nullptr ? rounded->data : nullptr, rounded != nullptr ? rounded->stride : 0, s), "rms_sum_add");
}

void qk_norm_store(cudaStream_t s, const Rows& proj, const QkvColumns& c, const float* q_weight, const float* k_weight, const Rows& q_out, void* cache,
                   const int32_t* slot_mapping, int n_tokens, bool norm, float eps, const int32_t* positions, float temp_coef, int temp_every) {
    if (proj.dtype != DType::F32 || q_out.cols != static_cast<int64_t>(c.n_head) * c.padded) throw invalid_argument("qk_norm_store: buffers do not fit");
    check(lb_qk_norm_store_tempered(code(q_out.dtype, "q_out"), proj.f32(), proj.stride, c.q_off, c.k_off, c.v_off, q_weight, k_weight, q_out.data, q_out.stride,
                                    cache, slot_mapping, n_tokens, c.n_head, c.n_kv_head, c.dim, c.vdim, c.padded, c.page_size, norm ? 1 : 0, eps, positions,
                                    temp_coef, temp_every, s), "qk_norm_store");
}

int gate_from_name(const std::string& name) {
    if (name == "sigmoid") return kSigmoid;
    if (name == "silu") return kSilu;
    if (name == "gelu_tanh") return kGeluGate;
    if (name == "relu") return kRelu;
    if (name == "capped") return kCapped;
    throw unsupported("gate '{}' is not supported; supported: sigmoid, silu, gelu_tanh, relu, capped", name);
}

void head_gate(cudaStream_t s, const Rows& o, int o_head, const Rows& g, const float* gain, const Rows& out, int n_tokens, int n_head, int vdim, bool norm,
               int gate, float eps) {
    if (out.cols != static_cast<int64_t>(n_head) * vdim || (g.data != nullptr && (g.dtype != DType::F32 || g.cols != out.cols))) throw invalid_argument("head_gate: buffers do not fit");
    check(lb_head_gate(code(o.dtype, "o"), code(out.dtype, "out"), o.data, o.stride, o_head, g.f32(), g.stride, gain, out.data, out.stride, n_tokens, n_head,
                       vdim, norm ? 1 : 0, gate, eps, s), "head_gate");
}

void gated_act(cudaStream_t s, const Rows& gu, const Rows& mid, int n_rows, int gate, float alpha, float limit) {
    if (gu.dtype != DType::F32 || gu.cols != 2 * mid.cols) throw invalid_argument("gated_act: buffers do not fit");
    check(lb_gated_act_kind(code(mid.dtype, "mid"), gu.f32(), gu.stride, mid.data, mid.stride, n_rows, static_cast<int>(mid.cols), gate, alpha, limit, s), "gated_act");
}

void qkv_rotary_store(cudaStream_t s, const Rows& proj, const QkvColumns& c, const float* q_weight, const float* k_weight, const Rows& q_out, void* cache,
                      const int32_t* slot_mapping, int n_tokens, int norm_mode, float eps, const int32_t* positions, const float* freq, int rot_dims,
                      const Rows* v_first_in, const Rows* v_first_out, const float* lambda) {
    if (proj.dtype != DType::F32 || q_out.cols != static_cast<int64_t>(c.n_head) * c.padded) throw invalid_argument("qkv_rotary_store: buffers do not fit");
    const int64_t vcols = static_cast<int64_t>(c.n_kv_head) * c.vdim;
    const Rows* shared = v_first_in != nullptr ? v_first_in : v_first_out;
    if (shared != nullptr && (shared->dtype != DType::F32 || shared->cols != vcols || shared->rows < n_tokens))
        throw invalid_argument("qkv_rotary_store: the shared values are float32 [tokens, {}]", vcols);
    check(lb_qkv_rotary_store(code(q_out.dtype, "q_out"), proj.f32(), proj.stride, c.q_off, c.k_off, c.v_off, q_weight, k_weight, q_out.data, q_out.stride, cache,
                              slot_mapping, n_tokens, c.n_head, c.n_kv_head, c.dim, c.vdim, c.padded, c.page_size, norm_mode, eps, positions, freq, rot_dims,
                              v_first_in != nullptr ? v_first_in->f32() : nullptr, v_first_out != nullptr ? v_first_out->f32() : nullptr,
                              shared != nullptr ? shared->stride : 0, lambda, s), "qkv_rotary_store");
}

void row_norm_gate(cudaStream_t s, const Rows& o, const Rows& g, const float* gain, const Rows& out, int n_rows, int gate, float eps) {
    if (o.dtype != DType::F32 || out.cols != o.cols || (g.data != nullptr && (g.dtype != DType::F32 || g.cols != o.cols))) throw invalid_argument("row_norm_gate: buffers do not fit");
    check(lb_row_norm_gate(code(out.dtype, "out"), o.f32(), o.stride, g.f32(), g.stride, gain, out.data, out.stride, n_rows, static_cast<int>(o.cols), gate, eps, s),
          "row_norm_gate");
}

void activate_columns(cudaStream_t s, const Rows& x, int n_rows, int gate) {
    if (x.dtype != DType::F32) throw invalid_argument("activate_columns: the rows are float32");
    check(lb_activate_columns(x.f32(), x.stride, n_rows, static_cast<int>(x.cols), gate, s), "activate_columns");
}

void router_table(cudaStream_t s, const int32_t* tokens, const Tensor& table, int32_t* ids, float* weights, int n_rows, int top, int n_experts) {
    if (table.dtype != DType::I32 || table.shape.size() != 2 || table.dim(1) != top) throw invalid_argument("router table: an int32 table [vocab, top]");
    check(lb_router_table(tokens, static_cast<const int32_t*>(table.data), ids, weights, n_rows, top, n_experts, static_cast<int>(table.dim(0)), s), "router_table");
}

void expert_plan_table(cudaStream_t s, const int32_t* tokens, const Tensor& table, int32_t* ids, float* weights, int n_rows, int top, int n_experts,
                       int32_t* offsets, int32_t* place, int32_t* pair_at) {
    if (table.dtype != DType::I32 || table.shape.size() != 2 || table.dim(1) != top) throw invalid_argument("router table: an int32 table [vocab, top]");
    check(lb_expert_plan_table(tokens, static_cast<const int32_t*>(table.data), static_cast<int>(table.dim(0)), top, ids, weights, n_rows, n_experts, offsets,
                               place, pair_at, s), "expert_plan_table");
}

void rows_to_bf16(cudaStream_t s, const Rows& x, const Rows& y, int n_rows) {
    if (x.dtype != DType::F32 || y.dtype != DType::BF16 || x.cols != y.cols) throw invalid_argument("rows_to_bf16: float32 rows into bfloat16 rows of the same width");
    check(lb_rows_to_bf16(x.f32(), x.stride, y.data, y.stride, n_rows, static_cast<int>(x.cols), s), "rows_to_bf16");
}

int memory_value_tile(int dim, int vdim) {
    // Tiles of up to 32 value columns, equal in size (more tiles, more blocks: a memory's rows of one request and head follow one
    // another, so the tiles are what fills the GPU); fewer columns where dim x tile floats would not fit a block's shared memory.
    int cap = 32;
    while (cap > 8 && static_cast<int64_t>(dim) * cap * 4 > 96 * 1024) cap /= 2;
    const int tiles = (vdim + cap - 1) / cap;
    return (vdim + tiles - 1) / tiles;
}

void matrix_memory(cudaStream_t s, const Rows& q, const Rows& k, const Rows& v, const Rows* zi, const Rows* zf, const float* decay, const float* freq,
                   const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state, const Rows& out, int n_seq, const MemoryShape& m,
                   bool chunked) {
    if (q.dtype != DType::F32 || out.dtype != DType::F32 || k.stride != q.stride || v.stride != q.stride || (zi != nullptr && zi->stride != q.stride) ||
        (zf != nullptr && zf->stride != q.stride))
        throw invalid_argument("matrix memory: queries, keys, values and gates are column blocks of one float buffer");
    check(lb_matrix_memory_activated(q.f32(), k.f32(), v.f32(), zi != nullptr ? zi->f32() : nullptr, zf != nullptr ? zf->f32() : nullptr, q.stride, decay, freq,
                                     m.rot_dims, positions, q_start, slots, state, m.stride(), out.f32(), out.stride, n_seq, m.n_head, m.dim, m.vdim,
                                     m.value_tile, m.q_scale, m.k_scale, m.cap, chunked ? 1 : 0, m.qk_share, m.qkv_act, s), "matrix_memory");
}

int64_t memory_pieces_floats(int n_tokens, int n_seq, const MemoryShape& m) {
    return lb_matrix_memory_pieces_floats(n_tokens, n_seq, m.n_head, m.dim, m.vdim, m.value_tile);
}

void matrix_memory_pieces(cudaStream_t s, const Rows& q, const Rows& k, const Rows& v, const Rows* zi, const Rows* zf, const float* decay, const float* freq,
                          const int32_t* positions, const int32_t* q_start, const int32_t* slots, float* state, const Rows& out, int n_tokens, int n_seq,
                          const MemoryShape& m, float* scratch) {
    if (q.dtype != DType::F32 || out.dtype != DType::F32 || k.stride != q.stride || v.stride != q.stride || (zi != nullptr && zi->stride != q.stride) ||
        (zf != nullptr && zf->stride != q.stride))
        throw invalid_argument("matrix memory: queries, keys, values and gates are column blocks of one float buffer");
    check(lb_matrix_memory_pieces_activated(q.f32(), k.f32(), v.f32(), zi != nullptr ? zi->f32() : nullptr, zf != nullptr ? zf->f32() : nullptr, q.stride, decay,
                                            freq, m.rot_dims, positions, q_start, slots, state, m.stride(), out.f32(), out.stride, n_tokens, n_seq, m.n_head,
                                            m.dim, m.vdim, m.value_tile, m.q_scale, m.k_scale, m.cap, scratch, m.qk_share, m.qkv_act, s), "matrix_memory_pieces");
    launches.fetch_add(2, std::memory_order_relaxed);
}

void router_topk(cudaStream_t s, const Rows& h, const Tensor& router, int32_t* ids, float* weights, int n_rows, int top, bool softmax, bool renormalise,
                 const float* bias) {
    if (router.shape.size() != 2 || router.dim(1) != h.cols || router.dtype != h.dtype) throw invalid_argument("router: the matrix does not fit the rows");
    check(lb_router_topk_biased(code(h.dtype, "h"), h.data, h.stride, router.data, bias, ids, weights, n_rows, static_cast<int>(router.dim(0)),
                                static_cast<int>(h.cols), top, softmax ? 1 : 0, renormalise ? 1 : 0, s), "router_topk");
}

void expert_plan(cudaStream_t s, const int32_t* ids, int n_pairs, int n_experts, int32_t* offsets, int32_t* place, int32_t* pair_at) {
    check(lb_expert_plan(ids, n_pairs, n_experts, offsets, place, pair_at, s), "expert_plan");
}

void expert_product(cudaStream_t s, bool gated, const Rows& a, const Tensor& w, int n_experts, const int32_t* offsets, const int32_t* pair_at,
                    const float* weights, const Rows& out, int n_pairs, int n, int k, int top, int gate, float alpha, float limit) {
    if (a.dtype != w.dtype || w.numel() != static_cast<int64_t>(n_experts) * (gated ? 2 : 1) * n * k || a.cols != k || out.cols != n)
        throw invalid_argument("expert product: shapes do not fit");
    if (out.dtype != (gated ? a.dtype : DType::F32)) throw invalid_argument("expert product: the output has the wrong type");
    check(lb_expert_product_kind(code(a.dtype, "a"), gated ? 1 : 0, a.data, a.stride, w.data, static_cast<int64_t>(gated ? 2 : 1) * n * k, offsets, pair_at,
                                 weights, out.data, out.stride, n_pairs, n_experts, n, k, top, gate, alpha, limit, s), "expert_product");
}

void expert_combine(cudaStream_t s, const Rows& x, const Rows& y, const int32_t* place, int n_rows, int top, const float* weights, bool overwrite) {
    if (x.dtype != DType::F32 || y.dtype != DType::F32 || x.cols != y.cols) throw invalid_argument("expert combine: buffers do not fit");
    check(lb_expert_combine_into(x.f32(), x.stride, y.f32(), y.stride, place, weights, n_rows, static_cast<int>(x.cols), top, overwrite ? 1 : 0, s), "expert_combine");
}

void ssm_prepare(cudaStream_t s, const Rows& proj, const float* taps, const float* tap_bias, const float* dt_bias, const float* a_log, float* conv_state,
                 int64_t slot_stride, const int32_t* tok_seq, const int32_t* q_start, const int32_t* slots, const Rows& out, int n_tokens, int n_seq,
                 const StateSpaceShape& m, bool decode_only) {
    if (proj.dtype != DType::F32 || out.dtype != DType::F32 || proj.cols != m.inner() + m.channels() + m.n_head || out.cols != m.prepared_cols())
        throw invalid_argument("state space: the projection's or the prepared rows do not fit the shape");
    check(lb_ssm_prepare(proj.f32(), proj.stride, static_cast<int>(m.inner()), static_cast<int>(m.inner() + m.channels()), taps, tap_bias, dt_bias, a_log,
                         conv_state, slot_stride, tok_seq, q_start, slots, out.f32(), out.stride, n_tokens, n_seq, m.n_head, m.vdim,
                         static_cast<int>(m.group_values()), m.taps, decode_only ? 1 : 0, s), "ssm_prepare");
    if (!decode_only && m.taps > 1) launches.fetch_add(1, std::memory_order_relaxed);
}

void gated_group_norm(cudaStream_t s, const Rows& o, const Rows* skip, const float* skip_gain, int head, const Rows* z, const float* weight, const Rows& out,
                      int n_rows, int groups, float eps) {
    if (o.dtype != DType::F32 || out.cols != o.cols || (skip != nullptr && (skip->dtype != DType::F32 || skip->cols != o.cols)) ||
        (z != nullptr && (z->dtype != DType::F32 || z->cols != o.cols)))
        throw invalid_argument("gated group norm: buffers do not fit");
    check(lb_gated_group_norm(code(out.dtype, "out"), o.f32(), o.stride, skip != nullptr ? skip->f32() : nullptr, skip != nullptr ? skip->stride : 0, skip_gain,
                              head, z != nullptr ? z->f32() : nullptr, z != nullptr ? z->stride : 0, weight, out.data, out.stride, n_rows,
                              static_cast<int>(o.cols), groups, eps, s), "gated_group_norm");
}

void token_shift(cudaStream_t s, const Rows& h, const float* mix, const Rows& m, void* state, const ShiftLayout& l) {
    if (h.dtype != m.dtype || h.cols != m.cols) throw invalid_argument("token shift: input and output differ in type or width");
    check(lb_token_shift(code(h.dtype, "h"), h.data, h.stride, mix, m.data, m.stride, state, l.tok_seq, l.q_start, l.slots, l.n_tokens, l.n_seq,
                         l.decode_only ? 1 : 0, static_cast<int>(h.cols), s), "token_shift");
    if (!l.decode_only) launches.fetch_add(1, std::memory_order_relaxed);
}

void rms_shift(cudaStream_t s, const Rows& x, const float* weight, const float* mix, const Rows& h, const Rows& m, void* state,
               const ShiftLayout& l, int groups, float eps) {
    if (x.dtype != DType::F32 || h.dtype != m.dtype || h.cols != x.cols || m.cols != x.cols) throw invalid_argument("rms norm with token shift: buffers do not fit");
    check(lb_rms_shift(code(h.dtype, "h"), x.f32(), x.stride, weight, mix, h.data, h.stride, m.data, m.stride, state, l.tok_seq, l.q_start, l.slots,
                       l.n_tokens, l.n_seq, l.decode_only ? 1 : 0, static_cast<int>(x.cols), groups, eps, s), "rms_shift");
    if (!l.decode_only) launches.fetch_add(1, std::memory_order_relaxed);
}

void xielu(cudaStream_t s, const Rows& z, int n_rows, const float* pq) {
    check(lb_xielu(code(z.dtype, "z"), z.data, z.stride, n_rows, static_cast<int>(z.cols), pq, s), "xielu");
}

void token_side(const Runtime& rt, Workspace* ws, const Rows& x, const int32_t* tokens, const Tensor& table, const Tensor& gate, const Tensor& proj,
                const float* weight, int n_tokens, float eps) {
    const int64_t dim = gate.dim(0), width = gate.dim(1);
    if (x.dtype != DType::F32 || x.cols != width || proj.dim(0) != width || proj.dim(1) != dim || table.dim(1) != dim || gate.dtype != proj.dtype ||
        gate.dtype != table.dtype)
        throw invalid_argument("token side input: tensors do not fit");
    cudaStream_t s = rt.stream;
    if (gate.dtype == DType::BF16 && n_tokens > 64 && width % 8 == 0 && dim % 8 == 0) {
        const Rows x16 = ws->get("side.x16", n_tokens, width, DType::BF16);
        check(lb_rows_to_bf16(x.f32(), x.stride, x16.data, x16.stride, n_tokens, static_cast<int>(width), s), "rows_to_bf16");
        const Rows pre = ws->get("side.pre", n_tokens, dim, DType::F32);
        linear(rt, ws, x16, gate, nullptr, pre, n_tokens, kNone, nullptr);
        const Rows g16 = ws->get("side.g16", n_tokens, dim, DType::BF16);
        check(lb_side_gate_finish(pre.f32(), pre.stride, tokens, table.data, g16.data, g16.stride, n_tokens, static_cast<int>(dim), s), "side_gate_finish");
        const Rows y = ws->get("side.y", n_tokens, width, DType::F32);
        linear(rt, ws, g16, proj, nullptr, y, n_tokens, kNone, nullptr);
        check(lb_rms_add(x.f32(), x.stride, y.f32(), y.stride, weight, n_tokens, static_cast<int>(width), eps, s), "rms_add");
        return;
    }
    const Rows g = ws->get("side.g", n_tokens, dim, DType::F32);
    check(lb_token_side(code(gate.dtype, "gate"), x.f32(), x.stride, tokens, table.data, gate.data, proj.data, weight, g.f32(), n_tokens,
                        static_cast<int>(width), static_cast<int>(dim), eps, s), "token_side");
    launches.fetch_add(1, std::memory_order_relaxed);
}

void latent_store(cudaStream_t s, const Rows& d, const float* gain, const float* freq, const int32_t* positions, const int32_t* slot_mapping,
                  void* cache, DType cache_dtype, int n_tokens, const LatentShape& a, float eps) {
    if (d.dtype != DType::F32 || d.cols != a.rank + a.rot) throw invalid_argument("latent store: the rows must be float32 [tokens, rank + rot]");
    const lb_latent_extras x = latent_extras(a, nullptr);
    check(lb_latent_store_ext(code(cache_dtype, "cache"), d.f32(), d.stride, gain, freq, positions, slot_mapping, cache, n_tokens, a.rank, a.rot, a.rot_dims,
                              eps, &x, s), "latent_store");
}

void rope_heads(cudaStream_t s, const Rows& q, const float* freq, const int32_t* positions, const Rows& wide, int n_tokens, const LatentShape& a) {
    if (wide.cols != static_cast<int64_t>(a.n_head) * (a.rank + a.rot) || q.cols != static_cast<int64_t>(a.n_head) * (a.dim + a.rot))
        throw invalid_argument("rotation of queries: buffers do not fit");
    check(lb_rope_heads_ext(code(q.dtype, "q"), code(wide.dtype, "wide"), q.data, q.stride, freq, positions, wide.data, wide.stride, n_tokens, a.n_head, a.dim,
                            a.rot, a.rot_dims, a.rank, a.interleaved ? 1 : 0, s), "rope_heads");
}

void head_matmul(cudaStream_t s, const Rows& a, int64_t a_head, const Tensor& b, int64_t b_head, int64_t b_k, int64_t b_n, const Rows& c,
                 int64_t c_head, int m, int n, int k, int n_head) {
    if (b.dtype == DType::BF16 && c.dtype == DType::BF16 && lb_head_matmul_mma_supports(a.stride, a_head, b_head, b_k, b_n, c.stride, c_head, n, k)) {
        check(lb_head_matmul_mma(code(a.dtype, "a"), a.data, a.stride, a_head, b.data, b_head, b_k, b_n, c.data, c.stride, c_head, m, n, k, n_head, s), "head_matmul_mma");
        return;
    }
    check(lb_head_matmul(code(a.dtype, "a"), code(b.dtype, "b"), code(c.dtype, "c"), a.data, a.stride, a_head, b.data, b_head, b_k, b_n, c.data, c.stride,
                         c_head, m, n, k, n_head, s), "head_matmul");
}

bool latent_few_supports(const LatentShape& a) { return lb_latent_few_supports(a.dim, a.rot, a.rank, a.vdim, 1) != 0; }

void latent_prepare(cudaStream_t s, const Rows& qd, const Tensor& uk, const float* gain, const float* freq, const int32_t* positions,
                    const int32_t* slot_mapping, void* cache, const Rows& wide, int n_tokens, const LatentShape& a, float eps, const Rows* latent) {
    if (qd.dtype != DType::F32 || uk.dtype != DType::BF16 || wide.dtype != DType::BF16) throw invalid_argument("latent queries: float32 rows, bfloat16 map and wide queries");
    const lb_latent_extras x = latent_extras(a, nullptr, true, latent);
    check(lb_latent_prepare_ext(qd.f32(), qd.stride, uk.data, gain, freq, positions, slot_mapping, cache, wide.data, wide.stride, n_tokens, a.n_head, a.dim,
                                a.rot, a.rot_dims, a.rank, eps, &x, s), "latent_prepare");
}

void latent_finish(cudaStream_t s, const Rows& attended, const float* part_o, const float* part_ml, const Tensor& uv, const Rows& values, int n_tokens,
                   const LatentShape& a, int n_splits, const Rows* gate) {
    if (attended.dtype != DType::F32 || uv.dtype != DType::BF16 || values.dtype != DType::BF16) throw invalid_argument("latent values: float32 latents, bfloat16 map and values");
    const lb_latent_extras x = latent_extras(a, gate);
    check(lb_latent_finish_ext(attended.f32(), attended.stride, part_o, part_ml, uv.data, values.data, values.stride, n_tokens, a.n_head, a.rank, a.vdim, n_splits,
                               &x, s), "latent_finish");
}

bool latent_rows_supports(const LatentShape& a) { return lb_latent_attention_rows_supports(a.n_head, a.rank, a.rot, a.page_size) != 0; }

void latent_attention_rows16(cudaStream_t s, const Rows& wide, const void* cache, const int32_t* q_start, const int32_t* n_past, const int32_t* block_table,
                             int table_width, const Rows& out, int n_tokens, int n_seq, int max_q_len, const LatentShape& a, const Rows* gate) {
    if (wide.dtype != DType::BF16 || out.dtype != DType::BF16) throw invalid_argument("latent attention, 64 rows a block: bfloat16 wide queries and attended latents");
    const lb_latent_extras x = latent_extras(a, gate);
    check(lb_latent_attention_rows16_ext(wide.data, wide.stride, cache, q_start, n_past, block_table, table_width, out.data, out.stride, n_tokens, n_seq, max_q_len,
                                         a.n_head, a.rank, a.rot, a.page_size, a.scale, a.window, &x, s), "latent_attention_rows16");
}

bool latent_mma_supports(const LatentShape& a) { return lb_latent_attention_mma_supports(a.n_head, a.rank, a.rot, a.page_size) != 0; }

int latent_splits(int n_seq, int n_head, int span) {
    // Enough blocks for two waves of the GPU, but no part shorter than two tiles of 32 keys.
    const int blocks = std::max(1, n_seq * ((n_head + 15) / 16)), tiles = span / 32 + 1;
    return std::max(1, std::min({16, tiles / 2, (296 + blocks - 1) / blocks}));
}

void latent_attention_mma(cudaStream_t s, const Rows& wide, const void* cache, const int32_t* q_start, const int32_t* n_past, const int32_t* block_table,
                          int table_width, const Rows& out, float* part_o, float* part_ml, int n_tokens, int n_seq, int max_q_len, const LatentShape& a,
                          int n_splits, bool merge, const Rows* gate) {
    if (wide.dtype != DType::BF16 || out.dtype != DType::F32) throw invalid_argument("latent attention on tensor cores: bfloat16 wide queries, float32 attended latents");
    const lb_latent_extras x = latent_extras(a, gate);
    check(lb_latent_attention_mma_ext(wide.data, wide.stride, cache, q_start, n_past, block_table, table_width, out.f32(), out.stride, part_o, part_ml, n_tokens,
                                      n_seq, max_q_len, a.n_head, a.rank, a.rot, a.page_size, a.scale, a.window, n_splits, merge ? 1 : 0, &x, s),
          "latent_attention_mma");
    if (n_splits > 1 && merge) launches.fetch_add(1, std::memory_order_relaxed);
}

void latent_attention(cudaStream_t s, DType cache_dtype, const Rows& wide, const void* cache, const int32_t* tok_seq, const int32_t* positions,
                      const int32_t* block_table, int table_width, const Rows& out, int n_tokens, const LatentShape& a, const Rows* gate) {
    if (wide.dtype != DType::F32 || out.dtype != DType::F32) throw invalid_argument("latent attention: wide queries and attended latents are float32");
    const lb_latent_extras x = latent_extras(a, gate);
    check(lb_latent_attention_ext(code(cache_dtype, "cache"), wide.f32(), wide.stride, cache, tok_seq, positions, block_table, table_width, out.f32(),
                                  out.stride, n_tokens, a.n_head, a.rank, a.rot, a.page_size, a.scale, a.window, &x, s), "latent_attention");
}

void sample(cudaStream_t s, const float* logits, int64_t row_stride, int n_rows, int vocab, const float* temperature,
            const int32_t* top_k, const float* top_p, const double* uniform, int32_t* out_ids) {
    check(lb_sample(logits, row_stride, n_rows, vocab, temperature, top_k, top_p, uniform, out_ids, nullptr, s), "sample");
}

void status_words_fetch(cudaStream_t s, int* host2) {
    check(lb_gemm_tcgen05_status_async(host2, s), "status_words_fetch");
    check(lb_decode_stack_status_async(host2 + 1, s), "status_words_fetch");
}
void status_words_clear(cudaStream_t s) {
    check(lb_gemm_tcgen05_status_clear(s), "status_words_clear");
    check(lb_decode_stack_status_clear(s), "status_words_clear");
}

}  // namespace liyab::kernels
