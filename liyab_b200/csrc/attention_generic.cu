// Causal attention over the paged cache for any mix of prompt portions and
// single decoded tokens, any head size up to 256 and any number of heads and
// key/value groups, with all arithmetic in 32-bit.
//
// This is the 32-bit engine's attention and the fallback of the bfloat16 engine
// for shapes its tensor-core kernels refuse.  One block serves one (token, head).
// The token's visible keys are cut into tiles of 32 from the first visible key;
// tile i goes to warp i mod W (W, the warps of a block, is fixed by the head size),
// every warp keeps a running softmax over its tiles in ascending order, and the
// warps' states are merged in warp order.  So the order of every sum depends on
// the token's position only, never on the batch or on where its pages lie (the
// reference cuts a token's keys into spans by its position alone for the same
// reason and merges the spans in order: src/core/transformer.cpp:2130-2144,
// 2225-2227, 2367-2385).  Scores s_j = (q . k_j) * scale, running maximum,
// p = exp(s - m), o = sum p_j v_j, out = o / sum p (src/core/transformer.cpp:2303-2313,
// 2327-2341, 2344-2358).
#include "api.h"
#include "common.cuh"

#include <math_constants.h>

namespace {

constexpr int kTile = 32;       // keys per step, one per lane
constexpr int kMaxHeadDim = 256;
constexpr long long kFewPairs = 1024;   // up to this many (token, head) pairs take the latency-arranged float32 kernel

// Four consecutive elements as floats with one load (the address is aligned to the four of them).
__device__ __forceinline__ float4 lb_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 lb_load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
}

// Copies the rows of up to 32 keys (lane i knows the row of key i: `base`, negative if there is none) into
// the warp's tile as floats.  Eight loads are issued before any is used, so a lone warp (a decode step of
// one request) still keeps several requests to memory in flight.
template <typename T>
__device__ __forceinline__ void load_tile(const T* __restrict__ cache, long long base, long long offset, float* tile,
                                          int tile_stride, int head_dim, int lane) {
    constexpr int kBatch = 8;
    if (head_dim % 4 == 0) {
        // Four values per load (rows of the cache start on 16-byte, or for 2-byte types 8-byte, boundaries).
        constexpr int kQuadBatch = 4;
        const int quads = head_dim / 4, total4 = kTile * quads;     // a multiple of 32
        for (int idx0 = lane; idx0 < total4; idx0 += 32 * kQuadBatch) {
            float4 r[kQuadBatch];
#pragma unroll
            for (int u = 0; u < kQuadBatch; ++u) {
                const int idx = idx0 + 32 * u;
                r[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (idx < total4) {            // uniform across the warp
                    const int key = idx / quads, d = (idx - key * quads) * 4;
                    const long long b = __shfl_sync(0xffffffffu, base, key);
                    if (b >= 0) r[u] = lb_load4(cache + b + offset + d);
                }
            }
#pragma unroll
            for (int u = 0; u < kQuadBatch; ++u) {
                const int idx = idx0 + 32 * u;
                if (idx < total4) {
                    const int key = idx / quads;
                    float* dst = tile + key * tile_stride + (idx - key * quads) * 4;
                    dst[0] = r[u].x; dst[1] = r[u].y; dst[2] = r[u].z; dst[3] = r[u].w;
                }
            }
        }
        return;
    }
    const int total = kTile * head_dim;        // a multiple of 32: every lane makes the same number of trips
    for (int idx0 = lane; idx0 < total; idx0 += 32 * kBatch) {
        float r[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int idx = idx0 + 32 * u;
            r[u] = 0.0f;
            if (idx < total) {                 // uniform across the warp
                const int key = idx / head_dim, d = idx - key * head_dim;
                const long long b = __shfl_sync(0xffffffffu, base, key);
                if (b >= 0) r[u] = lb_to_float(cache[b + offset + d]);
            }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int idx = idx0 + 32 * u;
            if (idx < total) {
                const int key = idx / head_dim;
                tile[key * tile_stride + (idx - key * head_dim)] = r[u];
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(512)
paged_attention_generic_kernel(const T* __restrict__ q, int64_t q_stride, const T* __restrict__ cache,
                               const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ positions,
                               const int32_t* __restrict__ block_table, int table_stride, T* __restrict__ out,
                               int64_t out_stride, int n_tokens, int n_head, int n_kv_head, int head_dim,
                               int page_size, float scale, int window) {
    extern __shared__ float smem[];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int pair = blockIdx.x;
    const int t = pair / n_head, h = pair - t * n_head;
    const int kvh = h / (n_head / n_kv_head);
    const int pos = positions[t];
    const int32_t* table = block_table + (size_t)tok_seq[t] * table_stride;

    const int tile_stride = head_dim + 1;
    float* q_s = smem + (size_t)warp * (head_dim + kTile * tile_stride + kTile);
    float* tile = q_s + head_dim;
    float* p_s = tile + kTile * tile_stride;

    const T* q_row = q + (size_t)t * q_stride + (size_t)h * head_dim;
    for (int d = lane; d < head_dim; d += 32) q_s[d] = lb_to_float(q_row[d]);

    const size_t plane = (size_t)n_kv_head * page_size * head_dim;
    float m = -CUDART_INF_F, l = 0.0f;
    float acc[kMaxHeadDim / 32];
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.0f;

    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    for (int j0 = first + warp * kTile; j0 <= pos; j0 += n_warps * kTile) {
        const int n_keys = min(kTile, pos + 1 - j0);
        // Each lane resolves its own key's row once; the others fetch it by shuffle.
        long long base = -1;
        if (lane < n_keys) {
            const int j = j0 + lane;
            const int page = table[j / page_size];
            base = (long long)page * 2 * (long long)plane + ((long long)kvh * page_size + (j % page_size)) * head_dim;
        }
        __syncwarp();
        load_tile(cache, base, 0, tile, tile_stride, head_dim, lane);
        __syncwarp();
        float s = -CUDART_INF_F;
        if (lane < n_keys) {
            float dot = 0.0f;
            const float* krow = tile + lane * tile_stride;
            for (int d = 0; d < head_dim; ++d) dot = fmaf(q_s[d], krow[d], dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, lb_warp_max(s));
        const float p = lane < n_keys ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);      // exp(-inf) = 0 on the first tile
        l = l * corr + lb_warp_sum(p);
        m = m_new;
        p_s[lane] = p;
        __syncwarp();
        load_tile(cache, base, (long long)plane, tile, tile_stride, head_dim, lane);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < kMaxHeadDim / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) {
                float o = acc[i] * corr;
                for (int j = 0; j < n_keys; ++j) o = fmaf(p_s[j], tile[j * tile_stride + d], o);
                acc[i] = o;
            }
        }
        __syncwarp();
    }
    // The warps' states (m, l, o) meet in shared memory and are merged in warp order.  A warp without a tile
    // has m = -inf, l = 0, o = 0 and weighs nothing.
    float* merge = smem + (size_t)n_warps * (head_dim + kTile * tile_stride + kTile);
    float* mine = merge + (size_t)warp * (head_dim + 2);
    if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) mine[2 + d] = acc[i];
    }
    __syncthreads();
    T* o_row = out + (size_t)t * out_stride + (size_t)h * head_dim;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float top = -CUDART_INF_F;
        for (int w = 0; w < n_warps; ++w) top = fmaxf(top, merge[(size_t)w * (head_dim + 2)]);
        float total = 0.0f, o = 0.0f;
        for (int w = 0; w < n_warps; ++w) {
            const float* st = merge + (size_t)w * (head_dim + 2);
            const float f = expf(st[0] - top);      // exp(-inf) = 0 for a warp without keys
            total = fmaf(st[1], f, total);
            o = fmaf(st[2 + d], f, o);
        }
        o_row[d] = lb_from_float<T>(o / total);
    }
}

// ---- float32, few (token, head) pairs: the same sums in the same order, arranged around memory latency --------
//
// A decode step of a few requests launches fewer blocks than the GPU has SMs, and each warp's chain of round
// trips to memory sets the pace.  Here keys and values have a buffer each and travel by asynchronous 16-byte copies
// (no registers in between): a tile's values are in flight while its scores are computed, the next tile's keys
// while the values are summed, and the page of the next tile is looked up a tile ahead.  Rows lie head_dim + 4
// floats apart, so a lane reads its key's row as 16-byte pieces without meeting a bank twice.  Every product and
// sum is the one paged_attention_generic_kernel makes, in its order: the two kernels agree bit for bit.

__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Which 16-byte pieces of a 32-key tile a lane copies: piece lane + 32 u, u = 0 .. head_dim / 4 - 1, of the tile's
// [key][piece of the row]; (key, piece) advance by fixed steps, so nothing is divided inside the loop.
struct PieceWalk {
    int key0, c0, dk, dc, quads;
};

// The rows of up to 32 keys (row_s[i]: where key i's row starts, negative if there is none) -> the tile, as copies in flight.
__device__ __forceinline__ void tile_in_flight(const float* __restrict__ cache, const long long* row_s, long long offset,
                                               float* tile, int tile_stride, const PieceWalk& w) {
    int key = w.key0, c = w.c0;
    for (int u = 0; u < w.quads; ++u) {
        const long long b = row_s[key];
        if (b >= 0) cp_async16(tile + key * tile_stride + 4 * c, cache + b + offset + 4 * c);
        key += w.dk;
        c += w.dc;
        if (c >= w.quads) { c -= w.quads; ++key; }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

__global__ void __launch_bounds__(256, 1)
paged_attention_f32_few_kernel(const float* __restrict__ q, int64_t q_stride, const float* __restrict__ cache,
                               const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ positions,
                               const int32_t* __restrict__ block_table, int table_stride, float* __restrict__ out,
                               int64_t out_stride, int n_tokens, int n_head, int n_kv_head, int head_dim,
                               int page_size, float scale, int window) {
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int pair = blockIdx.x;
    const int t = pair / n_head, h = pair - t * n_head;
    const int kvh = h / (n_head / n_kv_head);
    const int pos = positions[t];
    const int32_t* table = block_table + (size_t)tok_seq[t] * table_stride;

    const int tile_stride = head_dim + 4;
    float* q_s = smem + (size_t)warp * (head_dim + 2 * kTile * tile_stride + kTile + 2 * kTile);
    float* k_tile = q_s + head_dim;
    float* v_tile = k_tile + kTile * tile_stride;
    float* p_s = v_tile + kTile * tile_stride;
    long long* row_s = reinterpret_cast<long long*>(p_s + kTile);      // where each key's row of the coming tile starts
    const int quads = head_dim / 4;
    const PieceWalk walk{lane / quads, lane % quads, 32 / quads, 32 % quads, quads};

    const size_t plane = (size_t)n_kv_head * page_size * head_dim;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int step = n_warps * kTile;
    auto row_of = [&](int j0) -> long long {      // this lane's key of the tile that starts at j0
        const int j = j0 + lane;
        if (j0 > pos || j > pos) return -1;
        const int page = __ldg(table + j / page_size);
        return (long long)page * 2 * (long long)plane + ((long long)kvh * page_size + (j % page_size)) * head_dim;
    };
    int j0 = first + warp * kTile;
    row_s[lane] = row_of(j0);            // positions and block table came from the host: looked up before the wait
    lb_wait_for_predecessor();           // queries, and the newest keys and values, come from the kernel before this one
    lb_dependents_may_launch();
    __syncwarp();
    if (j0 <= pos) {
        tile_in_flight(cache, row_s, 0, k_tile, tile_stride, walk);
        tile_in_flight(cache, row_s, (long long)plane, v_tile, tile_stride, walk);
    }
    const float* q_row = q + (size_t)t * q_stride + (size_t)h * head_dim;
    for (int d = lane; d < head_dim; d += 32) q_s[d] = q_row[d];

    float m = -CUDART_INF_F, l = 0.0f;
    float acc[kMaxHeadDim / 32];
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.0f;

    for (; j0 <= pos; j0 += step) {
        const int n_keys = min(kTile, pos + 1 - j0);
        const bool more = j0 + step <= pos;
        const long long next_base = row_of(j0 + step);           // the next tile's page, asked for a tile ahead
        asm volatile("cp.async.wait_group 1;" ::: "memory");     // this tile's keys have landed (its values may not have)
        __syncwarp();
        float s = -CUDART_INF_F;
        if (lane < n_keys) {
            float dot = 0.0f;
            const float4* krow = reinterpret_cast<const float4*>(k_tile + lane * tile_stride);
            const float4* qv = reinterpret_cast<const float4*>(q_s);
            for (int c = 0; c < head_dim / 4; ++c) {
                const float4 kq = krow[c], qq = qv[c];
                dot = fmaf(qq.x, kq.x, dot);
                dot = fmaf(qq.y, kq.y, dot);
                dot = fmaf(qq.z, kq.z, dot);
                dot = fmaf(qq.w, kq.w, dot);
            }
            s = dot * scale;
        }
        const float m_new = fmaxf(m, lb_warp_max(s));
        const float p = lane < n_keys ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);      // exp(-inf) = 0 on the first tile
        l = l * corr + lb_warp_sum(p);
        m = m_new;
        p_s[lane] = p;
        row_s[lane] = next_base;                 // this tile's copies were all issued: the rows of the next one
        __syncwarp();                            // every lane has read the keys: the next tile's go into the buffer
        if (more) tile_in_flight(cache, row_s, 0, k_tile, tile_stride, walk);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");     // this tile's values have landed
        __syncwarp();
        // Each element's sum runs over the keys in ascending order, as in the plain kernel; the elements of a lane
        // advance side by side and share the weight they read.
#pragma unroll
        for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= corr;
#pragma unroll 4
        for (int j = 0; j < n_keys; ++j) {
            const float pj = p_s[j];
            const float* vrow = v_tile + j * tile_stride + lane;
#pragma unroll
            for (int i = 0; i < kMaxHeadDim / 32; ++i)
                if (32 * i < head_dim && lane + 32 * i < head_dim) acc[i] = fmaf(pj, vrow[32 * i], acc[i]);
        }
        __syncwarp();
        if (more) tile_in_flight(cache, row_s, (long long)plane, v_tile, tile_stride, walk);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    float* merge = smem + (size_t)n_warps * (head_dim + 2 * kTile * tile_stride + kTile + 2 * kTile);
    float* mine = merge + (size_t)warp * (head_dim + 2);
    if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) mine[2 + d] = acc[i];
    }
    __syncthreads();
    float* o_row = out + (size_t)t * out_stride + (size_t)h * head_dim;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float top = -CUDART_INF_F;
        for (int w = 0; w < n_warps; ++w) top = fmaxf(top, merge[(size_t)w * (head_dim + 2)]);
        float total = 0.0f, o = 0.0f;
        for (int w = 0; w < n_warps; ++w) {
            const float* st = merge + (size_t)w * (head_dim + 2);
            const float f = expf(st[0] - top);      // exp(-inf) = 0 for a warp without keys
            total = fmaf(st[1], f, total);
            o = fmaf(st[2 + d], f, o);
        }
        o_row[d] = o / total;
    }
}

// Whether a launch takes the kernel above: float32, 16-byte rows, few enough pairs that latency and not throughput
// sets the time, and a block's two tiles per warp fit the shared memory of an SM.
size_t few_smem(int warps, int head_dim) {
    return (size_t)warps * (head_dim + 2 * kTile * (head_dim + 4) + kTile + 2 * kTile + head_dim + 2) * sizeof(float);
}

// Warps per block, by the head size alone: eight while three such blocks fit the shared memory of an SM (up to head size 64), fewer for larger heads.
int warps_for(int head_dim) {
    const size_t per_warp = (size_t)(head_dim + kTile * (head_dim + 1) + kTile + head_dim + 2) * sizeof(float);
    int w = 8;
    while (w > 1 && 3 * w * per_warp > 220 * 1024) w >>= 1;
    return w;
}

template <typename T>
int launch(const void* q, int64_t q_stride, const void* cache, const int32_t* tok_seq, const int32_t* positions,
           const int32_t* block_table, int table_stride, void* out, int64_t out_stride, int n_tokens, int n_head,
           int n_kv_head, int head_dim, int page_size, float scale, int window, cudaStream_t s) {
    const int warps = warps_for(head_dim);
    const size_t smem = (size_t)warps * (head_dim + kTile * (head_dim + 1) + kTile + head_dim + 2) * sizeof(float);
    static size_t configured = 0;   // largest dynamic shared memory asked for so far
    if (smem > configured) {
        LB_CHECK_CUDA(cudaFuncSetAttribute(paged_attention_generic_kernel<T>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    const long long pairs = (long long)n_tokens * n_head;
    LB_CHECK_ARG(pairs <= 2147483647ll, "attention: %lld (token, head) pairs are too many for one launch", pairs);
    if constexpr (sizeof(T) == 4) {
        // Few pairs: the kernel arranged around latency (the same warps per block, so the same sums).
        const size_t few = few_smem(warps, head_dim);
        if (pairs <= kFewPairs && head_dim % 4 == 0 && q_stride % 4 == 0 && few <= 227 * 1024 && ((uintptr_t)cache & 15) == 0) {
            static size_t few_configured = 0;
            if (few > few_configured) {
                LB_CHECK_CUDA(cudaFuncSetAttribute(paged_attention_f32_few_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)few));
                few_configured = few;
            }
            LB_CHECK_CUDA(lb_launch_overlapped(paged_attention_f32_few_kernel, dim3((unsigned)pairs), dim3(warps * 32), few, s, 
                (const float*)q, q_stride, (const float*)cache, tok_seq, positions, block_table, table_stride, (float*)out, out_stride,
                n_tokens, n_head, n_kv_head, head_dim, page_size, scale, window));
            LB_CHECK_LAUNCH();
            return LB_OK;
        }
    }
    LB_CHECK_CUDA(lb_launch_overlapped(paged_attention_generic_kernel<T>, dim3((unsigned)pairs), dim3(warps * 32), smem, s, 
        (const T*)q, q_stride, (const T*)cache, tok_seq, positions, block_table, table_stride, (T*)out, out_stride,
        n_tokens, n_head, n_kv_head, head_dim, page_size, scale, window));
    LB_CHECK_LAUNCH();
    return LB_OK;
}

}  // namespace

extern "C" int lb_paged_attention_generic(int dtype, const void* q, int64_t q_stride, const void* cache,
                                          const int32_t* tok_seq, const int32_t* positions,
                                          const int32_t* block_table, int table_stride, void* out, int64_t out_stride,
                                          int n_tokens, int n_head, int n_kv_head, int head_dim, int page_size,
                                          float scale, int window, void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && n_head > 0 && n_kv_head > 0 && page_size > 0, "attention: bad sizes");
    LB_CHECK_ARG(n_head % n_kv_head == 0, "attention: n_head %d is not a multiple of n_kv_head %d", n_head, n_kv_head);
    LB_CHECK_ARG(head_dim > 0 && head_dim <= kMaxHeadDim, "attention: head_dim %d is outside (0, %d]", head_dim,
                 kMaxHeadDim);
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    if (dtype == LB_F32)
        return launch<float>(q, q_stride, cache, tok_seq, positions, block_table, table_stride, out, out_stride,
                             n_tokens, n_head, n_kv_head, head_dim, page_size, scale, window, s);
    if (dtype == LB_BF16)
        return launch<__nv_bfloat16>(q, q_stride, cache, tok_seq, positions, block_table, table_stride, out,
                                     out_stride, n_tokens, n_head, n_kv_head, head_dim, page_size, scale, window, s);
    return lb_fail(LB_ERR_INVALID_ARGUMENT, "attention: unknown dtype %d", dtype);
}
