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

#define LB_ABI_VERSION 3

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
 * absolute position; window 0 = all earlier keys. */
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
/* The same with scores and weighted values on the tensor cores (head_dim 64 or 128, up to 16 query heads per
 * key/value head, pages of 16 positions or more); same arguments, scratch and split semantics. */
int lb_decode_attention_mma(const void* q, int64_t q_stride, const void* cache, int n_pages, const int32_t* positions,
                            const int32_t* block_table, int table_stride, void* out, int64_t out_stride, float* partial,
                            int* counters, int n_seq, int n_head, int n_kv_head, int head_dim, int page_size, float scale,
                            int window, int n_splits, void* stream);
int lb_decode_attention_mma_supports(int n_head, int n_kv_head, int head_dim, int page_size);
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
/* The same on the tcgen05 tensor cores (head size 64, pages of 16 positions or more): TMA-fed, scores and output
 * accumulated in tensor memory.  n_tokens is the number of rows of q (and out), n_pages the number of pages of the
 * layer's cache (both bound the tensor maps). */
int lb_prefill_attention_tc(const void* q, int64_t q_stride, int n_tokens, const void* cache, int n_pages,
                            const int32_t* q_start, const int32_t* n_past, const int32_t* block_table, int table_stride,
                            void* out, int64_t out_stride, int n_seq, int max_q_len, int n_head, int n_kv_head, int head_dim,
                            int page_size, float scale, int window, void* stream);
int lb_prefill_attention_tc_supports(int n_head, int n_kv_head, int head_dim, int page_size);

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

#ifdef __cplusplus
}
#endif
