// Shared helpers of the kernel library: status codes, the thread-local error
// message, element types and warp/block reductions.
//
// Every exported function returns a status in the reference's numbering
// (include/liyab/liyab_c_api.h:41-53) and leaves a message for lb_last_error(),
// the way the reference's C API guards every call and keeps a thread-local last
// error (src/c_api/liyab_c_api.cpp:34-58).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

enum lb_status : int {
    LB_OK = 0,
    LB_ERR_INVALID_ARGUMENT = 1,
    LB_ERR_UNSUPPORTED = 4,
    LB_ERR_BACKEND = 8,
    LB_ERR_INTERNAL = 10,
};

// Element types of tensors passed through the C interface.
enum lb_dtype : int {
    LB_F32 = 0,
    LB_BF16 = 1,
};

// Activations fused into a matrix product's epilogue.
enum lb_activation : int {
    LB_ACT_NONE = 0,
    LB_ACT_GELU_TANH = 1,
    LB_ACT_GELU_ERF = 2,
};

int lb_fail(int code, const char* fmt, ...);

#define LB_CHECK_ARG(cond, ...)                                      \
    do {                                                             \
        if (!(cond)) return lb_fail(LB_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define LB_CHECK_CUDA(expr)                                                                          \
    do {                                                                                             \
        cudaError_t err__ = (expr);                                                                  \
        if (err__ != cudaSuccess)                                                                    \
            return lb_fail(LB_ERR_BACKEND, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), \
                           __FILE__, __LINE__);                                                      \
    } while (0)

#define LB_CHECK_LAUNCH() LB_CHECK_CUDA(cudaGetLastError())

// ---- launches that overlap the end of the kernel before ----
//
// A kernel launched through lb_launch_overlapped may be started while the kernel before it on the stream is still
// running (programmatic dependent launch): its blocks set up, ask for what does not depend on the kernel before
// (weights, block tables) and only then wait for it with lb_wait_for_predecessor(), which returns once that kernel
// has completed and its writes are visible.  Every thread of such a kernel passes lb_wait_for_predecessor() before
// it reads what an earlier kernel wrote or writes what an earlier kernel may still read.  The kernel before
// lets its successor start by lb_dependents_may_launch() (from all its blocks; without it the successor starts when
// it ends); a thread calls it only after its own lb_wait_for_predecessor(): let go before that, a step's later
// kernels ran ahead of data they needed (measured: wrong logits), whatever the reading of the instruction says.  In a kernel launched the ordinary way both are no-ops, and an ordinary launch after an overlapped one
// waits for the whole of it, as always.  lb_set_launch_overlap(0) makes every launch ordinary (measurements).
__device__ __forceinline__ void lb_dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void lb_wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool lb_launch_overlap_enabled(int kind = 0);

// cluster_x > 1: the grid's blocks form clusters of cluster_x blocks along x (gridDim.x a multiple of it).
template <typename... Params, typename... Args>
inline cudaError_t lb_launch_overlapped_cluster(int kind, int cluster_x, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                                cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = lb_launch_overlap_enabled(kind) ? 1 : 0;
    config.attrs = attribute;
    config.numAttrs = 1;
    if (cluster_x > 1) {
        attribute[1].id = cudaLaunchAttributeClusterDimension;
        attribute[1].val.clusterDim.x = (unsigned)cluster_x;
        attribute[1].val.clusterDim.y = 1;
        attribute[1].val.clusterDim.z = 1;
        config.numAttrs = 2;
    }
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

template <typename... Params, typename... Args>
inline cudaError_t lb_launch_overlapped_kind(int kind, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                        Args... args) {
    return lb_launch_overlapped_cluster(kind, 1, kernel, grid, block, smem, stream, args...);
}

__device__ __forceinline__ float lb_to_float(float v) { return v; }
__device__ __forceinline__ float lb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T lb_from_float(float v);
template <>
__device__ __forceinline__ float lb_from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 lb_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float lb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float lb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of additions is fixed by the block size alone.
__device__ __forceinline__ float lb_block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    v = lb_warp_sum(v);
    __syncthreads();  // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.0f;
        t = lb_warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// GELU, tanh form: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
// (reference: src/core/transformer.cpp:125-130).
__device__ __forceinline__ float lb_gelu_tanh(float x) {
    const float k = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}

// GELU, exact form: 0.5 x (1 + erf(x / sqrt 2)) (reference: src/core/transformer.cpp:139-142).
__device__ __forceinline__ float lb_gelu_erf(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}

__device__ __forceinline__ float lb_activate(float x, int act) {
    if (act == LB_ACT_GELU_TANH) return lb_gelu_tanh(x);
    if (act == LB_ACT_GELU_ERF) return lb_gelu_erf(x);
    return x;
}

template <typename... Params, typename... Args>
inline cudaError_t lb_launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    return lb_launch_overlapped_kind(0, kernel, grid, block, smem, stream, args...);
}
