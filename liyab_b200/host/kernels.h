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

#include "device.h"
#include "spec.h"

namespace liyab::kernels {

// Kernel launches issued through this module (a replayed graph adds its own count).
extern std::atomic<uint64_t> launches;

void check(int status, const char* what);

enum Activation : int { kNone = 0, kGeluTanh = 1, kGeluErf = 2 };
int activation_from_name(const std::string& name);      // UNSUPPORTED when unknown

// Keys and values of a fused projection that go straight to a layer's cache pages.
struct KvDestination {
    void* cache = nullptr;
    const int32_t* slot_mapping = nullptr;
    int q_dim = 0, n_kv_head = 0, head_dim = 0, page_size = 0;
};

void embed_positions(cudaStream_t s, const int32_t* tokens, const int32_t* positions, const Tensor& table,
                     const Tensor* pos_table, const Rows& x, int n_tokens, float scale);
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
// null, eps): up to 16 tokens, K up to 1024, bfloat16 weights.
bool gemm_rows_normed_supports(const Runtime& rt, const Rows& x, const Tensor& w, int m);
void gemm_rows_normed(cudaStream_t s, const Rows& x, const float* gain, const float* offset, float eps, const Tensor& w, const float* bias,
                      const Rows& out, int m, int act, const Rows* residual, const KvDestination* kv);
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
    int window = 0;
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

void sample(cudaStream_t s, const float* logits, int64_t row_stride, int n_rows, int vocab, const float* temperature,
            const int32_t* top_k, const float* top_p, const double* uniform, int32_t* out_ids);

// The two device status words (tcgen05/TMA bounded waits; the fused step's grid barrier): an asynchronous
// copy into `host2` (pinned, two ints) on `s`, and their reset.
void status_words_fetch(cudaStream_t s, int* host2);
void status_words_clear(cudaStream_t s);

}  // namespace liyab::kernels
