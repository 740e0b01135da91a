// Prefill attention for bfloat16: the step's prompt portions (any lengths, cut
// anywhere) against their requests' paged keys and values, with the products on
// the tensor cores and everything else in 32-bit.
//
// One thread block serves 64 consecutive query tokens of one request and one
// head.  It walks the keys the tile can see in tiles of 64 (four pages of 16, or
// fewer larger pages), fetched with cp.async through the block table into shared
// memory through a ring of three tile buffers.  The longest query tiles are
// handed out first.  Scores S = Q K^T and the update O += P V are
// mma.sync m16n8k16 products with 32-bit accumulators; the running maximum, the
// exponentials (exp2 of scores pre-scaled by log2 e) and the sums are 32-bit
// registers, two query rows per thread.  Keys of earlier portions and of this
// portion alike come from the cache, which the step has already written, so a
// token's result does not depend on how its prompt was cut.
//
// The products are mma.sync, which a B200 runs at about 1/16 of its tcgen05 rate
// (measured: this kernel saturates near 150 TFLOP/s with the tensor pipe busy);
// the kernel is bound by that, not by memory or latency.
//
// Reference formulas: scores, causal range, softmax and weighted values
// (src/core/transformer.cpp:2303-2313, 497-510, 2327-2341, 2344-2358).
//
// Sizes: head_dim 16, 32, ... 128 in steps of 16; any number of heads and of
// key/value groups; page_size a power of two (16 or more); an attention window.
#include "api.h"
#include "common.cuh"

#include <math_constants.h>

namespace {

constexpr int kBM = 64;           // query rows per block (16 per warp)
constexpr int kBN = 64;           // keys per tile
constexpr int kThreads = 128;
constexpr int kStages = 3;        // key/value tiles in flight or in use
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16 bytes global -> shared; when `valid` is false the destination is filled with zeros.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// D += A(16x16, row) . B(16x8, col), bfloat16 operands, float accumulators.
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(kThreads)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_stride, const __nv_bfloat16* __restrict__ cache,
                         const int32_t* __restrict__ q_start, const int32_t* __restrict__ n_past,
                         const int32_t* __restrict__ block_table, int table_stride, __nv_bfloat16* __restrict__ out,
                         int64_t out_stride, int n_head, int n_kv_head, int page_shift, float scale, int window) {
    constexpr int LD = HD + 8;                  // padded row of a tile in shared memory (elements)
    constexpr int CH = HD / 8;                  // 16-byte chunks per row
    constexpr int KS = HD / 16;                 // k-steps of Q K^T
    constexpr int NT = kBN / 8;                 // score n-tiles per key tile
    constexpr int OT = HD / 8;                  // output n-tiles
    extern __shared__ __align__(16) uint8_t smem_bytes[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_bytes);            // [kBM][LD]
    lb_wait_for_predecessor();            // queries, keys and values come from the kernel before this one
    lb_dependents_may_launch();
    __nv_bfloat16* k_s = q_s + kBM * LD;                                           // [kStages][kBN][LD]
    __nv_bfloat16* v_s = k_s + kStages * kBN * LD;                                 // [kStages][kBN][LD]

    // The last query tiles of a request see the most keys: they are handed out first, so that the short
    // ones fill the gaps at the end.
    const int seq = blockIdx.z, head = blockIdx.y, tile_q = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int row0 = q_start[seq], q_len = q_start[seq + 1] - row0;
    if (tile_q * kBM >= q_len) return;
    const int past = n_past[seq];
    const int kvh = head / (n_head / n_kv_head);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int page_size = 1 << page_shift;
    const size_t plane = (size_t)n_kv_head * page_size * HD;
    const int32_t* table = block_table + (size_t)seq * table_stride;

    const int rows_here = min(kBM, q_len - tile_q * kBM);
    const int p_min = past + tile_q * kBM, p_max = p_min + rows_here - 1;
    const int kv_lo = (window > 0 ? max(0, p_min - window + 1) : 0) / kBN * kBN;
    const int n_tiles = (p_max - kv_lo) / kBN + 1;

    // Q tile -> shared memory (rows past the portion's end are zeros).
    for (int c = threadIdx.x; c < kBM * CH; c += kThreads) {
        const int r = c / CH, ch = c - r * CH;
        const bool valid = r < rows_here;
        const __nv_bfloat16* src = q + (size_t)(row0 + tile_q * kBM + (valid ? r : 0)) * q_stride + (size_t)head * HD + ch * 8;
        cp_async16(q_s + r * LD + ch * 8, src, valid);
    }
    auto load_kv = [&](int tile, int stage) {
        const int j0 = kv_lo + tile * kBN;
        for (int c = threadIdx.x; c < kBN * CH; c += kThreads) {
            const int r = c / CH, ch = c - r * CH;
            const int j = j0 + r;
            const bool valid = j <= p_max;
            const int page = valid ? table[j >> page_shift] : 0;
            const __nv_bfloat16* src = cache + (size_t)max(page, 0) * 2 * plane +
                                       ((size_t)kvh * page_size + (j & (page_size - 1))) * HD + ch * 8;
            const bool ok = valid && page >= 0;
            cp_async16(k_s + (stage * kBN + r) * LD + ch * 8, src, ok);
            cp_async16(v_s + (stage * kBN + r) * LD + ch * 8, src + plane, ok);
        }
    };
    // kStages - 1 tiles ahead; one group per tile, empty past the last.
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {
        if (i < n_tiles) load_kv(i, i);
        cp_async_commit();
    }

    // Positions of this thread's two rows (rows past the end copy the last valid one; they are not stored).
    const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
    const int pos_lo = past + tile_q * kBM + min(r_lo, rows_here - 1);
    const int pos_hi = past + tile_q * kBM + min(r_hi, rows_here - 1);
    const int first_lo = window > 0 ? pos_lo - window + 1 : 0, first_hi = window > 0 ? pos_hi - window + 1 : 0;

    uint32_t qf[KS][4];
    float o[OT][4];
#pragma unroll
    for (int i = 0; i < OT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_lo = -CUDART_INF_F, m_hi = -CUDART_INF_F, l_lo = 0.0f, l_hi = 0.0f;
    const float sc = scale * kLog2e;

    for (int tile = 0; tile < n_tiles; ++tile) {
        const int stage = tile % kStages;
        cp_async_wait<kStages - 2>();           // this tile's group (and Q's, which went out with the first)
        __syncthreads();                        // ... from every thread; and everyone is done with the tile before
        if (tile + kStages - 1 < n_tiles) load_kv(tile + kStages - 1, (tile + kStages - 1) % kStages);
        cp_async_commit();
        if (tile == 0) {
#pragma unroll
            for (int kk = 0; kk < KS; ++kk) {
                const int mat = lane >> 3, r = lane & 7;
                ldmatrix_x4(qf[kk], smem_addr(q_s + (warp * 16 + (mat & 1) * 8 + r) * LD + kk * 16 + (mat >> 1) * 8));
            }
        }
        const __nv_bfloat16* kt = k_s + stage * kBN * LD;
        const __nv_bfloat16* vt = v_s + stage * kBN * LD;
        // S = Q K^T for this warp's 16 rows and the tile's 64 keys.
        float s[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                uint32_t b[4];
                const int mat = lane >> 3, r = lane & 7;
                ldmatrix_x4(b, smem_addr(kt + ((nt + (mat >> 1)) * 8 + r) * LD + kk * 16 + (mat & 1) * 8));
                mma_bf16(s[nt], qf[kk], b[0], b[1]);
                mma_bf16(s[nt + 1], qf[kk], b[2], b[3]);
            }
        }
        // Scale, mask what the rows cannot see, and update the running softmax.
        const int j0 = kv_lo + tile * kBN;
        const bool need_mask = (j0 + kBN - 1 > p_min) || (window > 0 && j0 < p_max - window + 1);
        float mx_lo = -CUDART_INF_F, mx_hi = -CUDART_INF_F;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[nt][e] * sc;
                if (need_mask) {
                    const int j = j0 + nt * 8 + 2 * t + (e & 1);
                    const bool hi = e >= 2;
                    if (j > (hi ? pos_hi : pos_lo) || j < (hi ? first_hi : first_lo)) v = -CUDART_INF_F;
                }
                s[nt][e] = v;
            }
            mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
            mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float base_lo = mn_lo == -CUDART_INF_F ? 0.0f : mn_lo, base_hi = mn_hi == -CUDART_INF_F ? 0.0f : mn_hi;
        const float corr_lo = exp2f(m_lo - base_lo), corr_hi = exp2f(m_hi - base_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.0f, sum_hi = 0.0f;
        uint32_t pf[NT / 2][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const float p0 = exp2f(s[nt][0] - base_lo), p1 = exp2f(s[nt][1] - base_lo);
            const float p2 = exp2f(s[nt][2] - base_hi), p3 = exp2f(s[nt][3] - base_hi);
            sum_lo += p0 + p1;
            sum_hi += p2 + p3;
            pf[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_lo = l_lo * corr_lo + sum_lo;      // per-thread partial sums; the quad is summed once at the end
        l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
        for (int i = 0; i < OT; ++i) {
            o[i][0] *= corr_lo;
            o[i][1] *= corr_lo;
            o[i][2] *= corr_hi;
            o[i][3] *= corr_hi;
        }
        // O += P V.
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
#pragma unroll
            for (int ot = 0; ot < OT; ot += 2) {
                uint32_t b[4];
                const int mat = lane >> 3, r = lane & 7;
                ldmatrix_x4_trans(b, smem_addr(vt + (kk * 16 + (mat & 1) * 8 + r) * LD + (ot + (mat >> 1)) * 8));
                mma_bf16(o[ot], pf[kk], b[0], b[1]);
                mma_bf16(o[ot + 1], pf[kk], b[2], b[3]);
            }
        }
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
    const size_t out_row = (size_t)(row0 + tile_q * kBM);
#pragma unroll
    for (int ot = 0; ot < OT; ++ot) {
        const int d = ot * 8 + 2 * t;
        if (r_lo < rows_here)
            *reinterpret_cast<uint32_t*>(out + (out_row + r_lo) * out_stride + (size_t)head * HD + d) =
                pack_bf16(o[ot][0] * inv_lo, o[ot][1] * inv_lo);
        if (r_hi < rows_here)
            *reinterpret_cast<uint32_t*>(out + (out_row + r_hi) * out_stride + (size_t)head * HD + d) =
                pack_bf16(o[ot][2] * inv_hi, o[ot][3] * inv_hi);
    }
}

template <int HD>
int launch(const void* q, int64_t q_stride, const void* cache, const int32_t* q_start, const int32_t* n_past,
           const int32_t* block_table, int table_stride, void* out, int64_t out_stride, int n_seq, int max_q_len,
           int n_head, int n_kv_head, int page_shift, float scale, int window, cudaStream_t s) {
    constexpr size_t smem = (size_t)(kBM + 2 * kStages * kBN) * (HD + 8) * sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        LB_CHECK_CUDA(cudaFuncSetAttribute(prefill_attention_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    dim3 grid((max_q_len + kBM - 1) / kBM, n_head, n_seq);
    LB_CHECK_CUDA(lb_launch_overlapped(prefill_attention_kernel<HD>, dim3(grid), dim3(kThreads), smem, s, 
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)cache, q_start, n_past, block_table, table_stride,
        (__nv_bfloat16*)out, out_stride, n_head, n_kv_head, page_shift, scale, window));
    LB_CHECK_LAUNCH();
    return LB_OK;
}

}  // namespace

extern "C" int lb_prefill_attention_supports(int n_head, int n_kv_head, int head_dim, int page_size) {
    return n_kv_head > 0 && n_head % n_kv_head == 0 && head_dim >= 16 && head_dim <= 128 && head_dim % 16 == 0 &&
           page_size >= 8 && (page_size & (page_size - 1)) == 0;
}

extern "C" int lb_prefill_attention(const void* q, int64_t q_stride, const void* cache, const int32_t* q_start,
                                    const int32_t* n_past, const int32_t* block_table, int table_stride, void* out,
                                    int64_t out_stride, int n_seq, int max_q_len, int n_head, int n_kv_head, int head_dim,
                                    int page_size, float scale, int window, void* stream) {
    LB_CHECK_ARG(n_seq >= 0 && max_q_len >= 0, "prefill attention: bad sizes");
    if (!lb_prefill_attention_supports(n_head, n_kv_head, head_dim, page_size))
        return lb_fail(LB_ERR_UNSUPPORTED, "prefill attention: unsupported shape heads %d/%d head_dim %d page_size %d",
                       n_head, n_kv_head, head_dim, page_size);
    LB_CHECK_ARG(q_stride % 8 == 0 && out_stride % 2 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 3) == 0,
                 "prefill attention: q rows must be 16-byte aligned");
    LB_CHECK_ARG(n_seq <= 65535 && n_head <= 65535, "prefill attention: too many requests or heads for one launch");
    if (n_seq == 0 || max_q_len == 0) return LB_OK;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    auto s = static_cast<cudaStream_t>(stream);
#define LB_HD(HD)                                                                                                        \
    case HD:                                                                                                             \
        return launch<HD>(q, q_stride, cache, q_start, n_past, block_table, table_stride, out, out_stride, n_seq, max_q_len, \
                          n_head, n_kv_head, page_shift, scale, window, s)
    switch (head_dim) {
        LB_HD(16);
        LB_HD(32);
        LB_HD(48);
        LB_HD(64);
        LB_HD(80);
        LB_HD(96);
        LB_HD(112);
        LB_HD(128);
    }
#undef LB_HD
    return lb_fail(LB_ERR_INTERNAL, "prefill attention: unreachable");
}
