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
    throw unsupported("activation '{}' is not supported; supported: gelu_tanh, gelu_erf, none", name);
}

namespace {
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
                      const Rows& out, int m, int act, const Rows* residual, const KvDestination* kv) {
    check(lb_gemm_rows_normed(code(out.dtype, "out"), x.f32(), x.stride, gain, offset, eps, w.data, w.dim(1), bias,
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

bool decode_scalar_supports(const AttentionShape& a) { return lb_decode_attention_supports(a.n_head, a.n_kv_head, a.head_dim, a.page_size) != 0; }
bool decode_mma_supports(const AttentionShape& a) { return lb_decode_attention_mma_supports(a.n_head, a.n_kv_head, a.head_dim, a.page_size) != 0; }
bool prefill_supports(const AttentionShape& a) { return lb_prefill_attention_supports(a.n_head, a.n_kv_head, a.head_dim, a.page_size) != 0; }
bool prefill_tc_supports(const AttentionShape& a) { return lb_prefill_attention_tc_supports(a.n_head, a.n_kv_head, a.head_dim, a.page_size) != 0; }

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
    check(lb_paged_attention_generic(code(dtype, "cache"), q.data, q.stride, cache, tok_seq, positions, block_table, table_width,
                                     out.data, out.stride, n_tokens, a.n_head, a.n_kv_head, a.head_dim, a.page_size, a.scale,
                                     a.window, s), "paged_attention_generic");
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
        check(lb_decode_attention_mma(q.data, q.stride, cache, n_pages, positions, block_table, table_width, out.data, out.stride,
                                      partial, counters, n_seq, a.n_head, a.n_kv_head, a.head_dim, a.page_size, a.scale, a.window,
                                      n_splits, s), "decode_attention_mma");
    else
        check(lb_decode_attention(q.data, q.stride, cache, positions, block_table, table_width, out.data, out.stride, partial,
                                  counters, n_seq, a.n_head, a.n_kv_head, a.head_dim, a.page_size, a.scale, a.window, n_splits, s),
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
                    aligned16(out.data) && blocks <= 4 * static_cast<int64_t>(rt.sm_count);
    if (tc)
        check(lb_prefill_attention_tc(q.data, q.stride, n_tokens, cache, n_pages, q_start, n_past, block_table, table_width,
                                      out.data, out.stride, n_seq, max_q_len, a.n_head, a.n_kv_head, a.head_dim, a.page_size,
                                      a.scale, a.window, rt.stream), "prefill_attention_tc");
    else
        check(lb_prefill_attention(q.data, q.stride, cache, q_start, n_past, block_table, table_width, out.data, out.stride, n_seq,
                                   max_q_len, a.n_head, a.n_kv_head, a.head_dim, a.page_size, a.scale, a.window, rt.stream),
              "prefill_attention");
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
