// out[M, N] = epilogue(A[M, K] . W[N, K]^T) on the ordinary 32-bit units.
//
// This is the true 32-bit matrix product of the engine (no tensor cores, no
// reduced-precision mode), and the fallback for 16-bit operands whose sizes the
// tensor-core kernel refuses.  Each output element is one chain of fused
// multiply-adds over k = 0 .. K-1 in ascending order, whatever the tile shape
// and whatever else is in the batch, so a row's result never depends on how many
// other rows share the launch (the reference promises the same of its matmul:
// include/liyab/backend.h:40-42).
//
// Epilogue, in the reference's order (src/core/transformer.cpp:111-118, 4903-4912,
// 5526-5532): + bias[n], activation, + residual[m, n].
#include "api.h"
#include "common.cuh"

namespace {

template <typename TI, typename TO, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_ffma_kernel(const TI* __restrict__ A, int64_t lda, const TI* __restrict__ W, int64_t ldw,
                 const float* __restrict__ bias, const float* residual, int64_t ldr, TO* out, int64_t ldo, int M,
                 int N, int K, int act) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    // A thread's pieces of the next tiles wait in registers while the current ones are multiplied: the loads of
    // step i + 1 travel under the arithmetic of step i.
    constexpr int LA = BM * BK / THREADS, LW = BN * BK / THREADS;
    static_assert(LA * THREADS == BM * BK && LW * THREADS == BN * BK, "the tiles divide among the threads");
    float ra[LA], rw[LW];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < LA; ++i) {
            const int idx = tid + i * THREADS, r = idx / BK, k = idx % BK;
            const int gm = m0 + r, gk = k0 + k;
            ra[i] = (gm < M && gk < K) ? lb_to_float(A[(size_t)gm * lda + gk]) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < LW; ++i) {
            const int idx = tid + i * THREADS, r = idx / BK, k = idx % BK;
            const int gn = n0 + r, gk = k0 + k;
            rw[i] = (gn < N && gk < K) ? lb_to_float(W[(size_t)gn * ldw + gk]) : 0.0f;
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < LA; ++i) {
            const int idx = tid + i * THREADS;
            As[idx % BK][idx / BK] = ra[i];
        }
#pragma unroll
        for (int i = 0; i < LW; ++i) {
            const int idx = tid + i * THREADS;
            Ws[idx % BK][idx / BK] = rw[i];
        }
        __syncthreads();
        if (k0 + BK < K) fetch(k0 + BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias != nullptr) v += bias[gn];
            v = lb_activate(v, act);
            if (residual != nullptr) v += residual[(size_t)gm * ldr + gn];
            out[(size_t)gm * ldo + gn] = lb_from_float<TO>(v);
        }
    }
}

template <typename TI, typename TO>
int launch(const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, const float* residual,
           int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act, cudaStream_t s) {
    if (M <= 16) {
        // Few tokens: one output per thread, 16 features per block (so that a narrow matrix still gives every SM a
        // block) and 64 columns of K per step.
        dim3 grid((N + 15) / 16, (M + 15) / 16);
        gemm_ffma_kernel<TI, TO, 16, 16, 64, 1, 1><<<grid, 256, 0, s>>>((const TI*)A, lda, (const TI*)W, ldw, bias,
                                                                      residual, ldr, (TO*)out, ldo, M, N, K, act);
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        gemm_ffma_kernel<TI, TO, 64, 64, 16, 4, 4><<<grid, 256, 0, s>>>((const TI*)A, lda, (const TI*)W, ldw, bias,
                                                                      residual, ldr, (TO*)out, ldo, M, N, K, act);
    }
    LB_CHECK_LAUNCH();
    return LB_OK;
}

}  // namespace

extern "C" int lb_gemm_ffma(int in_dtype, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw,
                            const float* bias, const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N,
                            int K, int act, void* stream) {
    LB_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    LB_CHECK_ARG(lda >= K && ldw >= K && ldo >= N, "gemm: a row stride is shorter than the row");
    LB_CHECK_ARG((M + 63) / 64 <= 65535, "gemm: M=%d is too large for one launch", M);
    if (M == 0) return LB_OK;
    auto s = static_cast<cudaStream_t>(stream);
    if (in_dtype == LB_F32 && out_dtype == LB_F32)
        return launch<float, float>(A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, s);
    if (in_dtype == LB_BF16 && out_dtype == LB_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, s);
    if (in_dtype == LB_BF16 && out_dtype == LB_F32)
        return launch<__nv_bfloat16, float>(A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, s);
    return lb_fail(LB_ERR_INVALID_ARGUMENT, "gemm: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
}
