// out[M, N] = epilogue(A[M, K] . W[N, K]^T) on the ordinary 32-bit units.
//
// This is the true 32-bit matrix product of the engine (no tensor cores, no
// reduced-precision mode), and the fallback for 16-bit operands whose sizes the
// tensor-core kernel refuses.  The order in which an output element's products
// are summed is a function of K alone, whatever the kernel, the tile shape and
// whatever else is in the batch, so a row's result never depends on how many
// other rows share the launch (the reference promises the same of its matmul:
// include/liyab/backend.h:40-42):
//
//   K is cut into chunks of 64 (the last may be shorter); a chunk's products are one
//   chain of fused multiply-adds in ascending k starting from zero; G = ceil(chunks /
//   32) consecutive chunks form a group whose chunk sums are added in ascending
//   order; the (at most 32) group sums are added in ascending order.
//
// Two kernels follow that order.  The tiled one (any number of tokens) lets every
// thread carry its outputs through all of K and folds the running chain into the
// group and total sums at the boundaries.  The one for up to 16 tokens (decoding)
// is bound by reading the weights once: a block owns eight features and all of K,
// each of its 32 (warp, slot) pairs owns one group of chunks for those features,
// a thread fetches its 64 weights of a chunk as 16-byte pieces that are all in
// flight together and multiplies them with the tokens' activations from the warp's
// buffer in shared memory; the group sums meet in shared memory and are added in
// order.
//
// Epilogue, in the reference's order (src/core/transformer.cpp:111-118, 4903-4912,
// 5526-5532): + bias[n], activation, + residual[m, n].
#include "api.h"
#include "common.cuh"

namespace {

constexpr int kChunk = 64;           // products per chain
constexpr int kGroups = 32;          // at most this many group sums per output

__host__ __device__ inline int chunks_per_group(int K) {
    const int chunks = (K + kChunk - 1) / kChunk;
    return (chunks + kGroups - 1) / kGroups;
}

template <typename TI, typename TO, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_ffma_kernel(const TI* __restrict__ A, int64_t lda, const TI* __restrict__ W, int64_t ldw,
                 const float* __restrict__ bias, const float* residual, int64_t ldr, TO* out, int64_t ldo, int M,
                 int N, int K, int act) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 1];
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    // acc: the running chain of the current chunk of 64; grp: the current group's chunk sums; tot: the group sums.
    float acc[TM][TN], grp[TM][TN], tot[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = grp[i][j] = tot[i][j] = 0.0f;
    static_assert(kChunk % BK == 0, "a chunk is a whole number of k-tiles");
    const int group_len = chunks_per_group(K) * kChunk;

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
        const int k_end = k0 + BK;              // the chunk, the group or K itself may end with this tile
        const bool last = k_end >= K;
        if (k_end % kChunk == 0 || last) {
            const bool first_chunk = (k_end - 1) / kChunk * kChunk % group_len == 0;
            const bool group_ends = k_end % group_len == 0 || last;
            const bool first_group = (k_end - 1) / group_len == 0;
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    grp[i][j] = first_chunk ? acc[i][j] : grp[i][j] + acc[i][j];
                    acc[i][j] = 0.0f;
                    if (group_ends) tot[i][j] = first_group ? grp[i][j] : tot[i][j] + grp[i][j];
                }
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
            float v = tot[i][j];
            if (bias != nullptr) v += bias[gn];
            v = lb_activate(v, act);
            if (residual != nullptr) v += residual[(size_t)gm * ldr + gn];
            out[(size_t)gm * ldo + gn] = lb_from_float<TO>(v);
        }
    }
}

// ---- up to 16 tokens: the weights are read once, everything else is arranged around that -----------------

constexpr int kSkinnyFeatures = 8;       // features per block
constexpr int kSkinnyTokens = 16;        // the most tokens; the kernel is also built for 8 (half the products and buffers)
// Floats between the buffers of a warp's four slots: banks 8 apart.
__host__ __device__ constexpr int skinny_pitch(int tokens) { return tokens * kChunk + 8; }

__device__ __forceinline__ void cp_async16_zfill(void* dst, const void* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

// 64 weights of one feature as floats: sixteen (float) or eight (bfloat16) 16-byte loads, all issued before use.
template <typename TI>
struct WeightChunk;
template <>
struct WeightChunk<float> {
    float4 v[16];
    __device__ __forceinline__ void load(const float* row, int k0, int K, bool live) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
            v[i] = (live && k0 + 4 * i < K) ? __ldg(reinterpret_cast<const float4*>(row + k0 + 4 * i)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __device__ __forceinline__ float4 quad(int i) const { return v[i]; }
};
template <>
struct WeightChunk<__nv_bfloat16> {
    uint4 v[8];
    __device__ __forceinline__ void load(const __nv_bfloat16* row, int k0, int K, bool live) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            v[i] = (live && k0 + 8 * i < K) ? __ldg(reinterpret_cast<const uint4*>(row + k0 + 8 * i)) : make_uint4(0, 0, 0, 0);
    }
    __device__ __forceinline__ float4 quad(int i) const {
        const uint4 u = v[i >> 1];
        const uint32_t lo = (i & 1) ? u.z : u.x, hi = (i & 1) ? u.w : u.y;
        return make_float4(__uint_as_float(lo << 16), __uint_as_float(lo & 0xffff0000u), __uint_as_float(hi << 16),
                           __uint_as_float(hi & 0xffff0000u));
    }
};

// K, lda and ldw are multiples of the 16-byte vector (4 floats, 8 bfloat16) and the bases 16-byte aligned.
// The block has as many warps as the reduction length has groups of chunks to give them (four groups a warp).
template <typename TI, typename TO, int TOKENS>
__global__ void __launch_bounds__(256)
gemm_ffma_skinny_kernel(const TI* __restrict__ A, int64_t lda, const TI* __restrict__ W, int64_t ldw,
                        const float* __restrict__ bias, const float* residual, int64_t ldr, TO* out, int64_t ldo, int M,
                        int N, int K, int act) {
    constexpr int VEC = 16 / (int)sizeof(TI);                   // elements per 16-byte piece
    constexpr int kPitch = skinny_pitch(TOKENS);
    extern __shared__ __align__(16) float skinny_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int fi = lane & 7, slot = lane >> 3;                   // feature within the block, chunk slot within the warp
    const int f = blockIdx.x * kSkinnyFeatures + fi;
    const int group = warp * 4 + slot;                           // this thread's group of chunks
    const int n_chunks = (K + kChunk - 1) / kChunk, G = chunks_per_group(K);
    const int c_begin = min(n_chunks, group * G), c_end = min(n_chunks, c_begin + G);
    // The warp's buffers: [slot][token][64] floats of activations (as stored: float or bfloat16 widened on use).
    float* my_buf = skinny_smem + (size_t)warp * 4 * kPitch;
    const TI* w_row = W + (size_t)min(f, N - 1) * ldw;
    float grp[TOKENS];
#pragma unroll
    for (int r = 0; r < TOKENS; ++r) grp[r] = 0.0f;
    for (int ci = 0; ci < G; ++ci) {                             // the same trip count for the whole warp
        const int c = c_begin + ci;
        const bool live = c < c_end;
        const int k0 = c * kChunk;
        WeightChunk<TI> w;
        w.load(w_row, k0, K, live && f < N);
        if (ci == 0) {
            // The first chunk's weights are under way; the activations come from the kernel before this one.
            lb_wait_for_predecessor();
            lb_dependents_may_launch();
        }
        // The warp's four slots bring their chunks of the tokens' activations: slot s2's chunk, token r, piece q.
        __syncwarp();
        for (int idx = lane; idx < 4 * TOKENS * (kChunk / VEC); idx += 32) {
            const int s2 = idx / (TOKENS * (kChunk / VEC)), rem = idx - s2 * (TOKENS * (kChunk / VEC));
            const int r = rem / (kChunk / VEC), q = rem - r * (kChunk / VEC);
            const int c2 = min(n_chunks, (warp * 4 + s2) * G) + ci;
            const int kk = c2 * kChunk + q * VEC;
            const bool valid = c2 < min(n_chunks, min(n_chunks, (warp * 4 + s2) * G) + G) && r < M && kk < K;
            TI* dst = reinterpret_cast<TI*>(my_buf + (size_t)s2 * kPitch) + r * kChunk + q * VEC;
            cp_async16_zfill(dst, A + (size_t)(valid ? r : 0) * lda + (valid ? kk : 0), valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        const TI* a_s = reinterpret_cast<const TI*>(my_buf + (size_t)slot * kPitch);
        float acc[TOKENS];
#pragma unroll
        for (int r = 0; r < TOKENS; ++r) acc[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < kChunk / 4; ++i) {
            const float4 wq = w.quad(i);
#pragma unroll
            for (int r = 0; r < TOKENS; ++r) {
                float4 aq;
                if constexpr (sizeof(TI) == 4) {
                    aq = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a_s) + r * kChunk + 4 * i);
                } else {
                    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a_s) + r * kChunk + 4 * i);
                    aq = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                                     __uint_as_float(u.y & 0xffff0000u));
                }
                acc[r] = fmaf(aq.x, wq.x, acc[r]);
                acc[r] = fmaf(aq.y, wq.y, acc[r]);
                acc[r] = fmaf(aq.z, wq.z, acc[r]);
                acc[r] = fmaf(aq.w, wq.w, acc[r]);
            }
        }
        if (live) {
#pragma unroll
            for (int r = 0; r < TOKENS; ++r) grp[r] = ci == 0 ? acc[r] : grp[r] + acc[r];
        }
    }
    // The group sums of the block meet in shared memory (over the activation buffers) and are added in ascending order.
    __syncthreads();
    float* red = skinny_smem;                                    // [group][token][feature]
#pragma unroll
    for (int r = 0; r < TOKENS; ++r) red[(group * TOKENS + r) * kSkinnyFeatures + fi] = grp[r];
    __syncthreads();
    for (int idx = threadIdx.x; idx < TOKENS * kSkinnyFeatures; idx += blockDim.x) {
        const int r = idx / kSkinnyFeatures, ff = idx % kSkinnyFeatures;
        const int gn = blockIdx.x * kSkinnyFeatures + ff;
        if (r < M && gn < N) {
            const int n_groups = (n_chunks + G - 1) / G;
            float v = red[(0 * TOKENS + r) * kSkinnyFeatures + ff];
            for (int g2 = 1; g2 < n_groups; ++g2) v += red[(g2 * TOKENS + r) * kSkinnyFeatures + ff];
            if (bias != nullptr) v += bias[gn];
            v = lb_activate(v, act);
            if (residual != nullptr) v += residual[(size_t)r * ldr + gn];
            out[(size_t)r * ldo + gn] = lb_from_float<TO>(v);
        }
    }
}

template <typename TI, typename TO>
int launch(const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, const float* residual,
           int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act, cudaStream_t s) {
    constexpr int VEC = 16 / (int)sizeof(TI);
    const bool vectors = K % VEC == 0 && lda % VEC == 0 && ldw % VEC == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0;
    if (M <= kSkinnyTokens && vectors) {
        // Few tokens: bound by reading the weights once (see the head of the file).  A warp serves four groups of
        // chunks, so a short reduction length makes small blocks, of which several share an SM.
        const int n_chunks = (K + kChunk - 1) / kChunk, per_group = chunks_per_group(K);
        const int n_groups = (n_chunks + per_group - 1) / per_group, warps = (n_groups + 3) / 4;
        const dim3 grid((N + kSkinnyFeatures - 1) / kSkinnyFeatures);
        if (M <= 8) {
            const size_t smem = (size_t)warps * 4 * skinny_pitch(8) * sizeof(float);
            static bool configured = false;
            if (!configured) {
                LB_CHECK_CUDA(cudaFuncSetAttribute(gemm_ffma_skinny_kernel<TI, TO, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)(8 * 4 * skinny_pitch(8) * sizeof(float))));
                configured = true;
            }
            LB_CHECK_CUDA(lb_launch_overlapped(gemm_ffma_skinny_kernel<TI, TO, 8>, dim3(grid), dim3(warps * 32), smem, s, (const TI*)A, lda, (const TI*)W, ldw, bias, residual, ldr,
                                                                             (TO*)out, ldo, M, N, K, act));
        } else {
            const size_t smem = (size_t)warps * 4 * skinny_pitch(16) * sizeof(float);
            static bool configured = false;
            if (!configured) {
                LB_CHECK_CUDA(cudaFuncSetAttribute(gemm_ffma_skinny_kernel<TI, TO, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)(8 * 4 * skinny_pitch(16) * sizeof(float))));
                configured = true;
            }
            LB_CHECK_CUDA(lb_launch_overlapped(gemm_ffma_skinny_kernel<TI, TO, 16>, dim3(grid), dim3(warps * 32), smem, s, (const TI*)A, lda, (const TI*)W, ldw, bias, residual, ldr,
                                                                              (TO*)out, ldo, M, N, K, act));
        }
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        LB_CHECK_CUDA(lb_launch_overlapped(gemm_ffma_kernel<TI, TO, 64, 64, 16, 4, 4>, dim3(grid), dim3(256), 0, s, (const TI*)A, lda, (const TI*)W, ldw, bias,
                                                                      residual, ldr, (TO*)out, ldo, M, N, K, act));
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
