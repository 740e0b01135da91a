// Decode attention for bfloat16: one query token per request against its paged
// keys and values, bound by the bytes of the cache it has to read.
//
// The keys of a request are split into n_splits equal ranges (a function of the
// token's position and n_splits only), one thread block per (range, key/value
// head, request), so that even a single request keeps the whole GPU streaming its
// cache.  Inside a block HD/8 threads share a key: each loads 16 bytes of the
// key row and of the value row, so a warp reads 512 contiguous bytes per load and
// every byte of the cache is read once, whatever the number of query heads that
// share the key/value head (G of them are served together).  Scores, the running
// maximum, the sum and the weighted values are 32-bit (exp2 of scores pre-scaled
// by log2 e).  Partial results (maximum, sum, unnormalised values) of the ranges
// go to scratch memory; the block that finishes last for a (request, head) merges
// them in range order, so the result does not depend on which block that is.
//
// Reference formulas: scores, softmax, values and the merge of spans by their
// maxima (src/core/transformer.cpp:2303-2313, 2327-2341, 2344-2358, 2367-2385).
#include "api.h"
#include "common.cuh"

#include <math_constants.h>

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kUnroll = 4;
constexpr float kLog2e = 1.4426950408889634f;

// Eight bfloat16 values travel as one 16-byte load (a uint4: the compiler splits a struct of four bfloat162
// into four 4-byte loads, which quadruples the requests).
using Vec8 = uint4;

__device__ __forceinline__ void unpack8(const Vec8& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// Merges the running softmax state (m_b, l_b, acc_b) into (m, l, acc).
template <int N>
__device__ __forceinline__ void merge_state(float& m, float& l, float (&acc)[N], float m_b, float l_b, const float (&acc_b)[N]) {
    const float m_new = fmaxf(m, m_b);
    const float fa = m_new == -CUDART_INF_F ? 0.0f : exp2f(m - m_new);
    const float fb = m_new == -CUDART_INF_F ? 0.0f : exp2f(m_b - m_new);
    l = l * fa + l_b * fb;
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = acc[i] * fa + acc_b[i] * fb;
    m = m_new;
}

template <int HD, int G>
__global__ void __launch_bounds__(kThreads)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_stride, const __nv_bfloat16* __restrict__ cache,
                        const int32_t* __restrict__ positions, const int32_t* __restrict__ block_table, int table_stride,
                        __nv_bfloat16* __restrict__ out, int64_t out_stride, float* __restrict__ partial,
                        int* __restrict__ counters, int n_kv_head, int page_shift, float scale, int window, int n_splits) {
    constexpr int TPK = HD / 8;                 // threads that share a key
    constexpr int KPW = 32 / TPK;               // keys a warp covers with one load
    constexpr int STATE = HD + 2;               // m, l, values
    __shared__ float red[kWarps][G][STATE];
    __shared__ int is_last;
    lb_wait_for_predecessor();
    lb_dependents_may_launch();

    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % TPK, kgroup = lane / TPK;
    const int page_size = 1 << page_shift;
    const int pos = positions[seq];
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_keys = pos + 1 - first;
    const int chunk = (n_keys + n_splits - 1) / n_splits;
    const int begin = first + split * chunk;
    const int end = min(pos + 1, begin + chunk);
    const int32_t* table = block_table + (size_t)seq * table_stride;
    const size_t plane = (size_t)n_kv_head * page_size * HD;

    float qf[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const Vec8 v = __ldg(reinterpret_cast<const Vec8*>(q + (size_t)seq * q_stride + (size_t)(kvh * G + g) * HD + sub * 8));
        unpack8(v, qf[g]);
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[g][i] *= scale * kLog2e;
    }
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -CUDART_INF_F;
        l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
    }

    // The loop bound is the same for every lane of a warp (the shuffles below need all of them).
    for (int jb = begin + warp * KPW; jb < end; jb += kWarps * KPW * kUnroll) {
        const int j0 = jb + kgroup;
        Vec8 kv[kUnroll], vv[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int j = j0 + u * kWarps * KPW;
            if (j < end) {
                const int page = table[j >> page_shift];
                const __nv_bfloat16* row = cache + (size_t)page * 2 * plane +
                                           ((size_t)kvh * page_size + (j & (page_size - 1))) * HD + sub * 8;
                kv[u] = __ldg(reinterpret_cast<const Vec8*>(row));
                vv[u] = __ldg(reinterpret_cast<const Vec8*>(row + plane));
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int j = j0 + u * kWarps * KPW;
            const bool live = j < end;          // uniform within the TPK threads of a key
            float kf[8], vf[8];
            if (live) {
                unpack8(kv[u], kf);
                unpack8(vv[u], vf);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) kf[i] = vf[i] = 0.0f;
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) s = fmaf(qf[g][i], kf[i], s);
#pragma unroll
                for (int o = TPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (live) {
                    const float m_new = fmaxf(m[g], s);
                    const float corr = exp2f(m[g] - m_new);
                    const float p = exp2f(s - m_new);
                    l[g] = l[g] * corr + p;
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(p, vf[i], acc[g][i] * corr);
                    m[g] = m_new;
                }
            }
        }
    }
    // Merge the key groups of a warp, then the warps, in a fixed order.
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int o = TPK; o < 32; o <<= 1) {
            const float m_b = __shfl_xor_sync(0xffffffffu, m[g], o);
            const float l_b = __shfl_xor_sync(0xffffffffu, l[g], o);
            float acc_b[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc_b[i] = __shfl_xor_sync(0xffffffffu, acc[g][i], o);
            // Both partners must end with the same state: order the pair by lane so the sums round alike.
            if ((lane & o) == 0) {
                merge_state<8>(m[g], l[g], acc[g], m_b, l_b, acc_b);
            } else {
                float m_a = m_b, l_a = l_b;
                merge_state<8>(m_a, l_a, acc_b, m[g], l[g], acc[g]);
                m[g] = m_a;
                l[g] = l_a;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[g][i] = acc_b[i];
            }
        }
        if (kgroup == 0) {
            red[warp][g][0] = m[g];
            red[warp][g][1] = l[g];
#pragma unroll
            for (int i = 0; i < 8; ++i) red[warp][g][2 + sub * 8 + i] = acc[g][i];
        }
    }
    __syncthreads();
    // One thread per (head of the group, value channel) folds the warps' states.
    float* my_partial = partial + (((size_t)seq * n_kv_head + kvh) * n_splits + split) * (size_t)(G * STATE);
    for (int idx = threadIdx.x; idx < G * HD; idx += kThreads) {
        const int g = idx / HD, d = idx - g * HD;
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, red[w][g][0]);
        float ll = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float f = mm == -CUDART_INF_F ? 0.0f : exp2f(red[w][g][0] - mm);
            ll += red[w][g][1] * f;
            a += red[w][g][2 + d] * f;
        }
        if (n_splits == 1) {
            out[(size_t)seq * out_stride + (size_t)(kvh * G + g) * HD + d] = __float2bfloat16_rn(a / ll);
        } else {
            my_partial[g * STATE + 2 + d] = a;
            if (d == 0) {
                my_partial[g * STATE] = mm;
                my_partial[g * STATE + 1] = ll;
            }
        }
    }
    if (n_splits == 1) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(&counters[seq * n_kv_head + kvh], 1);
        is_last = done == n_splits - 1;
        if (is_last) counters[seq * n_kv_head + kvh] = 0;      // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* all = partial + ((size_t)seq * n_kv_head + kvh) * n_splits * (size_t)(G * STATE);
    for (int idx = threadIdx.x; idx < G * HD; idx += kThreads) {
        const int g = idx / HD, d = idx - g * HD;
        float mm = -CUDART_INF_F;
        for (int sp = 0; sp < n_splits; ++sp) mm = fmaxf(mm, __ldcg(all + (size_t)sp * G * STATE + g * STATE));
        float ll = 0.0f, a = 0.0f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const float* st = all + (size_t)sp * G * STATE + g * STATE;
            const float f = exp2f(__ldcg(st) - mm);        // an empty range has m = -inf: factor 0
            ll += __ldcg(st + 1) * f;
            a += __ldcg(st + 2 + d) * f;
        }
        out[(size_t)seq * out_stride + (size_t)(kvh * G + g) * HD + d] = __float2bfloat16_rn(a / ll);
    }
}

template <int HD, int G>
int launch(const void* q, int64_t q_stride, const void* cache, const int32_t* positions, const int32_t* block_table,
           int table_stride, void* out, int64_t out_stride, float* partial, int* counters, int n_seq, int n_kv_head,
           int page_shift, float scale, int window, int n_splits, cudaStream_t s) {
    dim3 grid(n_splits, n_kv_head, n_seq);
    LB_CHECK_CUDA(lb_launch_overlapped(decode_attention_kernel<HD, G>, dim3(grid), dim3(kThreads), 0, s, 
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)cache, positions, block_table, table_stride,
        (__nv_bfloat16*)out, out_stride, partial, counters, n_kv_head, page_shift, scale, window, n_splits));
    LB_CHECK_LAUNCH();
    return LB_OK;
}

template <int HD>
int by_group(int group, const void* q, int64_t q_stride, const void* cache, const int32_t* positions,
             const int32_t* block_table, int table_stride, void* out, int64_t out_stride, float* partial, int* counters,
             int n_seq, int n_kv_head, int page_shift, float scale, int window, int n_splits, cudaStream_t s) {
#define LB_GO(G)                                                                                                   \
    return launch<HD, G>(q, q_stride, cache, positions, block_table, table_stride, out, out_stride, partial, counters, \
                         n_seq, n_kv_head, page_shift, scale, window, n_splits, s)
    switch (group) {
        case 1: LB_GO(1);
        case 2: LB_GO(2);
        case 4: LB_GO(4);
        case 8: LB_GO(8);
    }
#undef LB_GO
    return lb_fail(LB_ERR_UNSUPPORTED, "decode attention: %d query heads per key/value head is not supported (1, 2, 4, 8)", group);
}

}  // namespace

// Whether the decode kernel takes this shape (else the caller uses the generic kernel).
extern "C" int lb_decode_attention_supports(int n_head, int n_kv_head, int head_dim, int page_size) {
    if (n_kv_head <= 0 || n_head % n_kv_head != 0) return 0;
    const int g = n_head / n_kv_head;
    const bool hd_ok = head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256;
    const bool g_ok = g == 1 || g == 2 || g == 4 || g == 8;
    return hd_ok && g_ok && page_size > 0 && (page_size & (page_size - 1)) == 0 && !(head_dim == 256 && g == 8);
}

// Floats of scratch for `n_seq` requests split `n_splits` ways, and ints of counters (zeroed once by the caller).
extern "C" int64_t lb_decode_attention_scratch_floats(int n_seq, int n_head, int head_dim, int n_splits) {
    return (int64_t)n_seq * n_head * n_splits * (head_dim + 2);
}

extern "C" int lb_decode_attention(const void* q, int64_t q_stride, const void* cache, const int32_t* positions,
                                   const int32_t* block_table, int table_stride, void* out, int64_t out_stride,
                                   float* partial, int* counters, int n_seq, int n_head, int n_kv_head, int head_dim,
                                   int page_size, float scale, int window, int n_splits, void* stream) {
    LB_CHECK_ARG(n_seq >= 0 && n_splits >= 1, "decode attention: bad sizes n_seq=%d n_splits=%d", n_seq, n_splits);
    if (!lb_decode_attention_supports(n_head, n_kv_head, head_dim, page_size))
        return lb_fail(LB_ERR_UNSUPPORTED, "decode attention: unsupported shape heads %d/%d head_dim %d page_size %d", n_head,
                       n_kv_head, head_dim, page_size);
    LB_CHECK_ARG(n_splits == 1 || (partial != nullptr && counters != nullptr), "decode attention: scratch is missing");
    LB_CHECK_ARG(n_seq <= 65535 && n_kv_head <= 65535, "decode attention: too many requests or heads for one launch");
    if (n_seq == 0) return LB_OK;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    const int group = n_head / n_kv_head;
    auto s = static_cast<cudaStream_t>(stream);
#define LB_HD(HD)                                                                                                     \
    return by_group<HD>(group, q, q_stride, cache, positions, block_table, table_stride, out, out_stride, partial, counters, \
                        n_seq, n_kv_head, page_shift, scale, window, n_splits, s)
    switch (head_dim) {
        case 16: LB_HD(16);
        case 32: LB_HD(32);
        case 64: LB_HD(64);
        case 128: LB_HD(128);
        case 256: LB_HD(256);
    }
#undef LB_HD
    return lb_fail(LB_ERR_INTERNAL, "decode attention: unreachable");
}

// ------------------------------------------------------------------ the entry point that allocates nothing
//
// See no_alloc.h for what it promises.  The scratch lives in the two arrays below.  In host code their
// names stand for the arrays but are not device addresses; the addresses a kernel can use are looked up
// once per device with cudaGetSymbolAddress and kept in g_noalloc.
#include "no_alloc.h"

#include <mutex>

static __device__ __align__(256) float g_noalloc_partial[LB_NOALLOC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_noalloc_counters[LB_NOALLOC_COUNTER_INTS];

namespace {

constexpr int kMaxDevices = 64;

struct NoAllocScratch {
    float* partial = nullptr;
    int* counters = nullptr;
};

NoAllocScratch g_noalloc[kMaxDevices];
std::mutex g_noalloc_mutex;

// The scratch addresses on the current device, looked up at the first call on that device.
int noalloc_scratch(NoAllocScratch* out) {
    int device = -1;
    LB_CHECK_CUDA(cudaGetDevice(&device));
    LB_CHECK_ARG(device >= 0 && device < kMaxDevices, "decode attention (no-alloc): device ordinal %d is not supported", device);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    NoAllocScratch& slot = g_noalloc[device];
    if (slot.partial == nullptr) {
        float* partial = nullptr;
        int* counters = nullptr;
        LB_CHECK_CUDA(cudaGetSymbolAddress((void**)&partial, g_noalloc_partial));
        LB_CHECK_CUDA(cudaGetSymbolAddress((void**)&counters, g_noalloc_counters));
        slot.partial = partial;
        slot.counters = counters;
    }
    *out = slot;
    return LB_OK;
}

}  // namespace

extern "C" int lb_decode_attention_noalloc(const void* q, int64_t q_stride, const void* cache, const int32_t* positions,
                                           const int32_t* block_table, int table_stride, void* out, int64_t out_stride,
                                           int n_seq, int n_head, int n_kv_head, int head_dim, int page_size, float scale,
                                           int window, int n_splits, void* stream) {
    LB_CHECK_ARG(n_seq >= 0 && n_splits >= 1, "decode attention (no-alloc): bad sizes n_seq=%d n_splits=%d", n_seq, n_splits);
    if (!lb_decode_attention_supports(n_head, n_kv_head, head_dim, page_size))
        return lb_fail(LB_ERR_UNSUPPORTED, "decode attention (no-alloc): unsupported shape heads %d/%d head_dim %d page_size %d",
                       n_head, n_kv_head, head_dim, page_size);
    // An unsplit call touches neither array: no limit applies to it and nothing has to be cleared.
    const long long floats = n_splits > 1 ? (long long)n_seq * n_head * n_splits * (head_dim + 2) : 0;
    const long long ints = n_splits > 1 ? (long long)n_seq * n_kv_head : 0;
    LB_CHECK_ARG(floats <= LB_NOALLOC_SCRATCH_FLOATS,
                 "decode attention (no-alloc): %lld floats of scratch needed (n_seq %d x n_head %d x n_splits %d x (head_dim %d + 2)), "
                 "the built-in scratch holds %d; use fewer splits or requests, or lb_decode_attention with your own scratch",
                 floats, n_seq, n_head, n_splits, head_dim, LB_NOALLOC_SCRATCH_FLOATS);
    LB_CHECK_ARG(ints <= LB_NOALLOC_COUNTER_INTS,
                 "decode attention (no-alloc): %lld counters needed (n_seq %d x n_kv_head %d), the built-in scratch holds %d",
                 ints, n_seq, n_kv_head, LB_NOALLOC_COUNTER_INTS);
    if (n_seq == 0) return LB_OK;
    NoAllocScratch scratch;
    const int rc = noalloc_scratch(&scratch);
    if (rc != LB_OK) return rc;
    auto s = static_cast<cudaStream_t>(stream);
    // The array keeps the last call's contents; the counters have to start at zero.
    if (ints > 0) LB_CHECK_CUDA(cudaMemsetAsync(scratch.counters, 0, (size_t)ints * sizeof(int), s));
    return lb_decode_attention(q, q_stride, cache, positions, block_table, table_stride, out, out_stride, scratch.partial,
                               scratch.counters, n_seq, n_head, n_kv_head, head_dim, page_size, scale, window, n_splits,
                               stream);
}
