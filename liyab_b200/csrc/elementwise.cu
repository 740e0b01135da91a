// Embedding + position add, LayerNorm, and the copy of new keys and values into
// their cache pages.  All three are bound by memory traffic; each row is read
// once and written once.
#include "api.h"
#include "common.cuh"

#include <cstdlib>

#include <cstring>

// ---------------------------------------------------------------- errors

static thread_local char g_last_error[4096] = "";

int lb_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof g_last_error, fmt, ap);
    va_end(ap);
    return code;
}

extern "C" const char* lb_last_error(void) { return g_last_error; }

// The host library's failures land in the same thread-local message.
extern "C" void lb_set_last_error(const char* message) {
    snprintf(g_last_error, sizeof g_last_error, "%s", message != nullptr ? message : "");
}

extern "C" int lb_abi_version(void) { return LB_ABI_VERSION; }

// On unless the environment says LIYAB_B200_LAUNCH_OVERLAP=0 (measurements) or lb_set_launch_overlap(0) was called.
static bool g_launch_overlap = [] {
    const char* env = getenv("LIYAB_B200_LAUNCH_OVERLAP");
    return !(env != nullptr && env[0] == '0');
}();
static int g_overlap_mask = [] {
    const char* env = getenv("LIYAB_B200_OVERLAP_MASK");
    return env != nullptr ? atoi(env) : 15;
}();
bool lb_launch_overlap_enabled(int kind) { return g_launch_overlap && ((g_overlap_mask >> kind) & 1); }
// Whether launches made through lb_launch_overlapped may overlap the kernel before (1, the default) or not (0).
extern "C" int lb_set_launch_overlap(int on) {
    g_launch_overlap = on != 0;
    return LB_OK;
}

// ---------------------------------------------------------------- embedding

// x[t, :] = table[token[t], :] * scale + positions[pos[t], :]  (32-bit sum).
// Reference: embed (src/core/transformer.cpp:5495-5512), add_positions (:2791-2808).
template <typename T>
__global__ void embed_positions_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ pos,
                                       const T* __restrict__ table, const T* __restrict__ pos_table,
                                       float* __restrict__ x, int width, float scale) {
    const int t = blockIdx.x;
    const T* row = table + (size_t)tokens[t] * width;
    const T* prow = pos_table != nullptr ? pos_table + (size_t)pos[t] * width : nullptr;
    float* out = x + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = lb_to_float(row[i]) * scale;
        if (prow != nullptr) v += lb_to_float(prow[i]);
        out[i] = v;
    }
}

extern "C" int lb_embed_positions(int dtype, const int32_t* tokens, const int32_t* positions, const void* table,
                                  const void* pos_table, float* x, int n_tokens, int width, float scale,
                                  void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && width > 0, "embed: bad sizes n_tokens=%d width=%d", n_tokens, width);
    if (n_tokens == 0) return LB_OK;
    const int threads = width >= 1024 ? 256 : 128;
    auto s = static_cast<cudaStream_t>(stream);
    if (dtype == LB_F32) {
        embed_positions_kernel<float><<<n_tokens, threads, 0, s>>>(tokens, positions, (const float*)table,
                                                                  (const float*)pos_table, x, width, scale);
    } else if (dtype == LB_BF16) {
        embed_positions_kernel<__nv_bfloat16><<<n_tokens, threads, 0, s>>>(
            tokens, positions, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pos_table, x, width, scale);
    } else {
        return lb_fail(LB_ERR_INVALID_ARGUMENT, "embed: unknown dtype %d", dtype);
    }
    LB_CHECK_LAUNCH();
    return LB_OK;
}

// ---------------------------------------------------------------- LayerNorm

// y = (x - mean) / sqrt(var + eps) * w + b with the population variance of the
// centred values, both statistics in 32-bit (two passes over the row, so no
// cancellation).  Reference: layernorm (src/core/transformer.cpp:77-106), which
// accumulates in double; the difference is below one 32-bit rounding of y.
// `rows` (optional) gathers: output row r is made from input row rows[r].
template <typename T>
__global__ void layernorm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                 const float* __restrict__ w, const float* __restrict__ b, T* __restrict__ y,
                                 int width, float eps) {
    __shared__ float scratch[33];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int r = blockIdx.x;
    const float* in = x + (size_t)(rows != nullptr ? rows[r] : r) * width;
    T* out = y + (size_t)r * width;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) sum += in[i];
    const float mean = lb_block_sum(sum, scratch) / (float)width;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float d = in[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float var = lb_block_sum(ss, scratch) / (float)width;
    const float inv = 1.0f / sqrtf(var + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = (in[i] - mean) * inv;
        if (w != nullptr) v *= w[i];
        if (b != nullptr) v += b[i];
        out[i] = lb_from_float<T>(v);
    }
}

// The same for rows of up to 4 * 32 * NV values whose width is a multiple of 4: one warp per row, the row held
// in registers (each lane float4s lane, lane + 32, ...), the two sums by warp shuffles; the row is read once
// and no barrier is needed.  The order of additions depends on the width alone.
template <typename T, int NV>
__global__ void __launch_bounds__(128)
layernorm_warp_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ w,
                      const float* __restrict__ b, T* __restrict__ y, int n_rows, int width, float eps) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= n_rows) return;
    const int n4 = width >> 2;
    const float4* in = reinterpret_cast<const float4*>(x + (size_t)(rows != nullptr ? rows[r] : r) * width);
    float4 v[NV];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        v[i] = c < n4 ? in[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = lb_warp_sum(sum) / (float)width;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (lane + 32 * i < n4) {
            const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
            ss += (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
    }
    const float inv = 1.0f / sqrtf(lb_warp_sum(ss) / (float)width + eps);
    T* out = y + (size_t)r * width;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < n4) {
            float4 o = make_float4((v[i].x - mean) * inv, (v[i].y - mean) * inv, (v[i].z - mean) * inv, (v[i].w - mean) * inv);
            if (w != nullptr) {
                const float4 ww = reinterpret_cast<const float4*>(w)[c];
                o.x *= ww.x; o.y *= ww.y; o.z *= ww.z; o.w *= ww.w;
            }
            if (b != nullptr) {
                const float4 bb = reinterpret_cast<const float4*>(b)[c];
                o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
            }
            if constexpr (sizeof(T) == 4) {
                reinterpret_cast<float4*>(out)[c] = o;
            } else {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                reinterpret_cast<uint2*>(out)[c] = pk;
            }
        }
    }
}

// Wider rows (up to 4 * 128 * NV values, a multiple of 4): four warps per row, the row held in registers (each
// thread float4s t, t + 128, ...), the two sums by warp shuffles and then over the four warps in warp order.  A row
// of a few thousand values is then a handful of loads per thread, all in flight together, instead of one warp's long
// chain.  The order of additions depends on the width alone.
template <typename T, int NV>
__global__ void __launch_bounds__(128)
layernorm_row_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ w,
                     const float* __restrict__ b, T* __restrict__ y, int width, float eps) {
    __shared__ float part[2][4];
    const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n4 = width >> 2;
    float4 v[NV], gain[NV], offs[NV];
    // Gains and offsets are weights: they are asked for before the kernel before this one has ended.
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = tid + 128 * i;
        const bool live = c < n4;
        gain[i] = (live && w != nullptr) ? reinterpret_cast<const float4*>(w)[c] : make_float4(1.f, 1.f, 1.f, 1.f);
        offs[i] = (live && b != nullptr) ? reinterpret_cast<const float4*>(b)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const float4* in = reinterpret_cast<const float4*>(x + (size_t)(rows != nullptr ? rows[r] : r) * width);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = tid + 128 * i;
        v[i] = c < n4 ? in[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    sum = lb_warp_sum(sum);
    if (lane == 0) part[0][warp] = sum;
    __syncthreads();
    const float mean = (((part[0][0] + part[0][1]) + part[0][2]) + part[0][3]) / (float)width;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (tid + 128 * i < n4) {
            const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
            ss += (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
    }
    ss = lb_warp_sum(ss);
    if (lane == 0) part[1][warp] = ss;
    __syncthreads();
    const float inv = 1.0f / sqrtf((((part[1][0] + part[1][1]) + part[1][2]) + part[1][3]) / (float)width + eps);
    T* out = y + (size_t)r * width;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = tid + 128 * i;
        if (c < n4) {
            float4 o = make_float4((v[i].x - mean) * inv, (v[i].y - mean) * inv, (v[i].z - mean) * inv, (v[i].w - mean) * inv);
            if (w != nullptr) { o.x *= gain[i].x; o.y *= gain[i].y; o.z *= gain[i].z; o.w *= gain[i].w; }
            if (b != nullptr) { o.x += offs[i].x; o.y += offs[i].y; o.z += offs[i].z; o.w += offs[i].w; }
            if constexpr (sizeof(T) == 4) {
                reinterpret_cast<float4*>(out)[c] = o;
            } else {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                reinterpret_cast<uint2*>(out)[c] = pk;
            }
        }
    }
}

template <typename T>
static void launch_layernorm_row(const float* x, const int32_t* rows, const float* w, const float* b, T* y, int n_rows,
                                 int width, float eps, cudaStream_t s) {
    const int n4 = width / 4;
    if (n4 <= 128 * 2) lb_launch_overlapped_kind(0, layernorm_row_kernel<T, 2>, dim3(n_rows), dim3(128), 0, s, x, rows, w, b, y, width, eps);
    else if (n4 <= 128 * 4) lb_launch_overlapped_kind(0, layernorm_row_kernel<T, 4>, dim3(n_rows), dim3(128), 0, s, x, rows, w, b, y, width, eps);
    else lb_launch_overlapped_kind(0, layernorm_row_kernel<T, 8>, dim3(n_rows), dim3(128), 0, s, x, rows, w, b, y, width, eps);
}

template <typename T>
static void launch_layernorm_warp(const float* x, const int32_t* rows, const float* w, const float* b, T* y, int n_rows,
                                  int width, float eps, cudaStream_t s) {
    const int blocks = (n_rows + 3) / 4, n4 = width / 4;
    if (n4 <= 32 * 2) lb_launch_overlapped_kind(0, layernorm_warp_kernel<T, 2>, dim3(blocks), dim3(128), 0, s, x, rows, w, b, y, n_rows, width, eps);
    else if (n4 <= 32 * 4) lb_launch_overlapped_kind(0, layernorm_warp_kernel<T, 4>, dim3(blocks), dim3(128), 0, s, x, rows, w, b, y, n_rows, width, eps);
    else if (n4 <= 32 * 6) lb_launch_overlapped_kind(0, layernorm_warp_kernel<T, 6>, dim3(blocks), dim3(128), 0, s, x, rows, w, b, y, n_rows, width, eps);
    else if (n4 <= 32 * 8) lb_launch_overlapped_kind(0, layernorm_warp_kernel<T, 8>, dim3(blocks), dim3(128), 0, s, x, rows, w, b, y, n_rows, width, eps);
    else if (n4 <= 32 * 13) lb_launch_overlapped_kind(0, layernorm_warp_kernel<T, 13>, dim3(blocks), dim3(128), 0, s, x, rows, w, b, y, n_rows, width, eps);
    else lb_launch_overlapped_kind(0, layernorm_warp_kernel<T, 16>, dim3(blocks), dim3(128), 0, s, x, rows, w, b, y, n_rows, width, eps);
}

extern "C" int lb_layernorm(int out_dtype, const float* x, const int32_t* rows, const float* weight,
                            const float* bias, void* y, int n_rows, int width, float eps, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && width > 0, "layernorm: bad sizes n_rows=%d width=%d", n_rows, width);
    if (n_rows == 0) return LB_OK;
    const int threads = width >= 2048 ? 256 : 128;   // fixed by the width alone: a row's sums never depend on the batch
    auto s = static_cast<cudaStream_t>(stream);
    // Rows of float4s that fit a warp's registers take the warp-per-row kernel (everything 16-byte aligned).
    const bool warp_rows = width % 4 == 0 && width <= 2048 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 &&
                           (weight == nullptr || ((uintptr_t)weight & 15) == 0) && (bias == nullptr || ((uintptr_t)bias & 15) == 0);
    // By the width alone (never by the number of rows: a row's sums must not depend on the batch): up to 512 values
    // a warp per row, up to 4096 four warps per row.
    const bool block_rows = warp_rows || (width % 4 == 0 && width <= 4096 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 &&
                                          (weight == nullptr || ((uintptr_t)weight & 15) == 0) && (bias == nullptr || ((uintptr_t)bias & 15) == 0));
    if (block_rows && width > 512 && out_dtype == LB_F32) {
        launch_layernorm_row<float>(x, rows, weight, bias, (float*)y, n_rows, width, eps, s);
    } else if (block_rows && width > 512 && out_dtype == LB_BF16) {
        launch_layernorm_row<__nv_bfloat16>(x, rows, weight, bias, (__nv_bfloat16*)y, n_rows, width, eps, s);
    } else if (warp_rows && out_dtype == LB_F32) {
        launch_layernorm_warp<float>(x, rows, weight, bias, (float*)y, n_rows, width, eps, s);
    } else if (warp_rows && out_dtype == LB_BF16) {
        launch_layernorm_warp<__nv_bfloat16>(x, rows, weight, bias, (__nv_bfloat16*)y, n_rows, width, eps, s);
    } else if (out_dtype == LB_F32) {
        lb_launch_overlapped_kind(0, layernorm_kernel<float>, dim3(n_rows), dim3(threads), 0, s, x, rows, weight, bias, (float*)y, width, eps);
    } else if (out_dtype == LB_BF16) {
        lb_launch_overlapped_kind(0, layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, s, x, rows, weight, bias, (__nv_bfloat16*)y, width, eps);
    } else {
        return lb_fail(LB_ERR_INVALID_ARGUMENT, "layernorm: unknown dtype %d", out_dtype);
    }
    LB_CHECK_LAUNCH();
    return LB_OK;
}

// ---------------------------------------------------------------- cache append

// Copies each new token's key and value rows into its page.  A layer's cache is
// [page][K|V][kv_head][slot][head_dim]; slot_mapping[t] = page * page_size + slot
// (negative: the token's keys are not kept, e.g. a layer that reads another's cache).
// Reference: store_kv (src/core/transformer.cpp:2875-2890, src/core/kv_cache.cpp:322-332).
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k, const T* __restrict__ v, int64_t row_stride,
                                 const int32_t* __restrict__ slot_mapping, T* __restrict__ cache, int n_kv_head,
                                 int head_dim, int page_size) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int t = blockIdx.x;
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    const int page = slot / page_size, off = slot - page * page_size;
    const int row = n_kv_head * head_dim;
    const size_t plane = (size_t)n_kv_head * page_size * head_dim;
    T* kdst = cache + (size_t)page * 2 * plane;
    T* vdst = kdst + plane;
    const T* ksrc = k + (size_t)t * row_stride;
    const T* vsrc = v + (size_t)t * row_stride;
    for (int i = threadIdx.x; i < row; i += blockDim.x) {
        const int h = i / head_dim, d = i - h * head_dim;
        const size_t at = ((size_t)h * page_size + off) * head_dim + d;
        kdst[at] = ksrc[i];
        vdst[at] = vsrc[i];
    }
}

// The same in 16-byte pieces (head_dim * sizeof(T) a multiple of 16, everything 16-byte aligned): thread c of a
// token's block moves piece c of the key row or of the value row; four tokens per block.
template <typename T>
__global__ void __launch_bounds__(256)
kv_append_vec_kernel(const T* __restrict__ k, const T* __restrict__ v, int64_t row_stride,
                     const int32_t* __restrict__ slot_mapping, T* __restrict__ cache, int n_tokens, int n_kv_head,
                     int head_dim, int page_size) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    constexpr int kPer = 16 / (int)sizeof(T);                    // elements per piece
    const int pieces_head = head_dim / kPer, pieces_row = n_kv_head * pieces_head;
    const int per_token = 2 * pieces_row;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int t = (int)(idx / per_token);
    if (t >= n_tokens) return;
    int c = (int)(idx - (long)t * per_token);
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    const bool is_v = c >= pieces_row;
    if (is_v) c -= pieces_row;
    const int h = c / pieces_head, d = (c - h * pieces_head) * kPer;
    const int page = slot / page_size, off = slot - page * page_size;
    const size_t plane = (size_t)n_kv_head * page_size * head_dim;
    const T* src = (is_v ? v : k) + (size_t)t * row_stride + (size_t)h * head_dim + d;
    T* dst = cache + (size_t)page * 2 * plane + (is_v ? plane : 0) + ((size_t)h * page_size + off) * head_dim + d;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
}

extern "C" int lb_kv_append(int dtype, const void* k, const void* v, int64_t row_stride, const int32_t* slot_mapping,
                            void* cache, int n_tokens, int n_kv_head, int head_dim, int page_size, void* stream) {
    LB_CHECK_ARG(n_tokens >= 0 && n_kv_head > 0 && head_dim > 0 && page_size > 0, "kv_append: bad sizes");
    if (n_tokens == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    const int threads = 128;
    const int elem = dtype == LB_F32 ? 4 : 2;
    const bool vec = (dtype == LB_F32 || dtype == LB_BF16) && (head_dim * elem) % 16 == 0 && (row_stride * elem) % 16 == 0 &&
                     ((uintptr_t)k & 15) == 0 && ((uintptr_t)v & 15) == 0 && ((uintptr_t)cache & 15) == 0;
    if (vec) {
        const long pieces = (long)n_tokens * 2 * n_kv_head * (head_dim * elem / 16);
        const int blocks = (int)((pieces + 255) / 256);
        if (dtype == LB_F32)
            LB_CHECK_CUDA(lb_launch_overlapped(kv_append_vec_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)k, (const float*)v, row_stride, slot_mapping,
                                                              (float*)cache, n_tokens, n_kv_head, head_dim, page_size));
        else
            LB_CHECK_CUDA(lb_launch_overlapped(kv_append_vec_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, row_stride,
                                                                      slot_mapping, (__nv_bfloat16*)cache, n_tokens, n_kv_head,
                                                                      head_dim, page_size));
    } else if (dtype == LB_F32) {
        LB_CHECK_CUDA(lb_launch_overlapped(kv_append_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)k, (const float*)v, row_stride, slot_mapping,
                                                            (float*)cache, n_kv_head, head_dim, page_size));
    } else if (dtype == LB_BF16) {
        LB_CHECK_CUDA(lb_launch_overlapped(kv_append_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                                    row_stride, slot_mapping, (__nv_bfloat16*)cache,
                                                                    n_kv_head, head_dim, page_size));
    } else {
        return lb_fail(LB_ERR_INVALID_ARGUMENT, "kv_append: unknown dtype %d", dtype);
    }
    LB_CHECK_LAUNCH();
    return LB_OK;
}

// ---------------------------------------------------------------- tokens that are still on the device

// dst[i] = src[map[i]] where map[i] >= 0 (else dst[i] stays): the tokens a step sampled go straight into the next
// step's token array, without a round trip through the host.
__global__ void gather_tokens_kernel(int32_t* __restrict__ dst, const int32_t* __restrict__ src,
                                     const int32_t* __restrict__ map, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && map[i] >= 0) dst[i] = src[map[i]];
}

extern "C" int lb_gather_tokens(int32_t* dst, const int32_t* src, const int32_t* map, int n, void* stream) {
    LB_CHECK_ARG(n >= 0, "gather_tokens: bad size %d", n);
    if (n == 0) return LB_OK;
    gather_tokens_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(dst, src, map, n);
    LB_CHECK_LAUNCH();
    return LB_OK;
}

// ---------------------------------------------------------------- logit scale and soft cap

// The head's finishing touches where a model has them (the reference's finish_logits and
// apply_final_softcap: src/core/transformer.cpp:2613-2620): x * scale, then cap * tanh(x / cap).
__global__ void scale_softcap_kernel(float* __restrict__ x, int64_t n, float scale, float cap) {
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = x[i] * scale;
        if (cap > 0.0f) v = cap * tanhf(v / cap);
        x[i] = v;
    }
}

extern "C" int lb_scale_softcap(float* logits, int64_t count, float scale, float soft_cap, void* stream) {
    LB_CHECK_ARG(logits != nullptr && count >= 0, "scale_softcap: bad arguments");
    if (count == 0) return LB_OK;
    const int blocks = (int)((count + 255) / 256 < 1184 ? (count + 255) / 256 : 1184);
    LB_CHECK_CUDA(lb_launch_overlapped(scale_softcap_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), logits, count, scale, soft_cap));
    LB_CHECK_LAUNCH();
    return LB_OK;
}
