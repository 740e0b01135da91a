// out[M, N] = epilogue(A[M, K] . W[N, K]^T) for 1 to 64 tokens (bfloat16
// operands): the products of a decode step, too small to fill a tcgen05 tile row,
// whose reduction is short enough (the host takes it for K up to 1024, and for up
// to 16 tokens up to 4096 where one pass covers a block's features).
//
// At these sizes a product reads a few MB of weights and does next to no
// arithmetic; what it costs is latency.  The tcgen05 kernel needs K split over
// blocks and a second kernel to add the partial sums (two launches, 8-9 us per
// product).  Here one launch does it: every block takes a slice of the output
// features and the whole reduction length, as the matrix phases of the fused
// decode step do: the activations of all tokens come into shared memory by
// cp.async in chunks of 256 columns (two buffers: the next chunk travels while the
// current one is used), each warp takes 32 columns of every chunk, requests all
// its weights of the pass (up to four groups of eight features) at the start with
// 16-byte loads that go straight into mma.sync m16n8k16 fragments (tokens are the
// rows: one to four tiles of 16), and the eight warps' partial tiles are summed in
// warp order through shared memory.  For up to 16 tokens all columns of the
// activations are staged at once (or made in the kernel by a LayerNorm of the
// float32 rows), and a thread asks for the bias and residual of the elements it
// will finish before its products.  The launch may overlap the kernel before:
// weights are asked for before the wait for it, activations after.
// Every weight byte is read once; a row's result does not depend on the other
// rows.  Accumulators, bias, activation and residual sum are 32-bit, in the
// reference's order (src/core/transformer.cpp:111-118, 4903-4912, 5526-5532).
#include "api.h"
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kChunk = 256;           // columns of the activations per chunk: one k-block of 32 per warp
constexpr int kChunkLd = kChunk + 32; // row stride in a buffer: 64 bytes mod 128, conflict-free 16-byte reads
constexpr int kMaxRows = 64;
constexpr int kWRegs = 16;            // 16-byte weight pieces a thread holds: groups per pass x chunks

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Optional second destination of a fused query/key/value projection: features from q_dim on are keys, then values,
// and go (as bfloat16) to the token's slot of its cache page as well (layout [page][K|V][kv_head][slot][head_dim];
// slot_mapping[token] = page * page_size + slot, negative: not kept).  cache == nullptr: none.
struct KvScatter {
    __nv_bfloat16* cache;
    const int32_t* slot_mapping;
    int q_dim, n_kv_head, head_dim, page_size;
};

// Activations made in the kernel from the float32 residual rows by a LayerNorm (two-pass 32-bit statistics,
// (x - mean) / sqrt(var + eps) * gain + offset, as the separate kernel computes them): for up to 16 tokens and a
// reduction length of up to 1024 a block normalises the rows itself, one warp per row with the row in registers (one
// round trip), and keeps them in shared memory for all its passes.  That saves the LayerNorm's launch.  x == nullptr: off.
struct RowNorm {
    const float* x;
    int64_t ldx;
    const float* gain;
    const float* offset;
    float eps;
};

__device__ void layernorm_rows_to_smem(const RowNorm& n, int M, int K, __nv_bfloat16* act, int ld, int k_pad) {
    constexpr int kVecs = 8;                       // float4 per lane: rows of up to 1024 values
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_vec = K / 4;
    float4 gain[kVecs], offs[kVecs];
#pragma unroll
    for (int j = 0; j < kVecs; ++j) {              // weights: asked for before the kernel before this one has ended
        const int i = lane + 32 * j;
        gain[j] = (i < n_vec && n.gain != nullptr) ? __ldg(reinterpret_cast<const float4*>(n.gain) + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        offs[j] = (i < n_vec && n.offset != nullptr) ? __ldg(reinterpret_cast<const float4*>(n.offset) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    for (int r = warp; r < 16; r += kWarps) {
        __nv_bfloat16* dst = act + r * ld;
        if (r >= M) {                              // rows past the step's tokens: zeros
            for (int i = lane * 8; i < k_pad; i += 256) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0, 0, 0, 0);
            continue;
        }
        const float* row = n.x + (size_t)r * n.ldx;
        float4 v[kVecs];
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int i = lane + 32 * j;
            v[j] = i < n_vec ? __ldcg(reinterpret_cast<const float4*>(row) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        const float mean = lb_warp_sum(sum) / (float)K;
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            if (lane + 32 * j < n_vec) {
                const float d0 = v[j].x - mean, d1 = v[j].y - mean, d2 = v[j].z - mean, d3 = v[j].w - mean;
                ss = fmaf(d0, d0, ss);
                ss = fmaf(d1, d1, ss);
                ss = fmaf(d2, d2, ss);
                ss = fmaf(d3, d3, ss);
            }
        }
        const float inv = 1.0f / sqrtf(lb_warp_sum(ss) / (float)K + n.eps);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int i = lane + 32 * j;
            if (i < n_vec) {
                const float4 g = gain[j], o = offs[j];
                const __nv_bfloat162 lo = __floats2bfloat162_rn((v[j].x - mean) * inv * g.x + o.x, (v[j].y - mean) * inv * g.y + o.y);
                const __nv_bfloat162 hi = __floats2bfloat162_rn((v[j].z - mean) * inv * g.z + o.z, (v[j].w - mean) * inv * g.w + o.w);
                uint2 packed;
                packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst + 4 * i) = packed;
            }
        }
        for (int i = K + lane; i < k_pad; i += 32) dst[i] = __float2bfloat16_rn(0.0f);
    }
}

// MT: tiles of 16 tokens (1 to 4).  NG: feature groups (of 8 features) per pass: 4, 2 or 1, for a reduction length
// of up to 1024, 2048 or 4096 (NG x chunks = the 16 weight pieces a thread holds: all of a pass's weights are
// requested at its start, one DRAM round trip, and used as the chunks of activations come in).
// STAGE: how the activations reach shared memory.  0: chunk by chunk through two buffers (any number of tokens).
// 1 (up to 16 tokens): all columns at once, one round trip, kept for all of the block's passes.  2 (up to 16 tokens,
// K up to 1024): the same, made here from the float32 rows by a LayerNorm.
template <int MT, int NG, typename TO, int STAGE = 0>
__global__ void __launch_bounds__(kThreads, 1)
gemm_rows_kernel(const __nv_bfloat16* __restrict__ A, int64_t lda, const __nv_bfloat16* __restrict__ W, int64_t ldw,
                 const float* __restrict__ bias, const float* residual, int64_t ldr, TO* out, int64_t ldo, int M, int N, int K,
                 int act, KvScatter kv, RowNorm norm) {
    static_assert(STAGE == 0 || MT == 1, "all columns at once for up to 16 tokens only");
    static_assert(STAGE != 2 || NG == 4, "rows are normalised in the kernel for K up to 1024");
    constexpr bool FULL = STAGE != 0;
    constexpr int kRows = MT * 16, MC = kWRegs / NG;
    extern __shared__ __align__(16) uint8_t smem_bytes[];
    // The activations: two buffers of one chunk each, [2][kRows][kChunkLd]; or (FULL) all columns at once, [16][ld_full].
    __nv_bfloat16* act_s = reinterpret_cast<__nv_bfloat16*>(smem_bytes);
    const int ld_full = (K + kChunk - 1) / kChunk * kChunk + 32;        // 64 bytes mod 128 as well
    const size_t act_bytes = FULL ? (size_t)16 * ld_full * sizeof(__nv_bfloat16) : (size_t)2 * kRows * kChunkLd * sizeof(__nv_bfloat16);
    float* red_s = reinterpret_cast<float*>(smem_bytes + act_bytes);   // [kWarps][NG][MT][128]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n_groups = (N + 7) / 8;
    const int per_cta = (n_groups + (int)gridDim.x - 1) / (int)gridDim.x;
    const int g_begin = min(n_groups, (int)blockIdx.x * per_cta), g_end = min(n_groups, g_begin + per_cta);
    const int n_chunks = (K + kChunk - 1) / kChunk;            // at most MC (the host checks)

    // Chunk c of the activations -> buffer c & 1 (rows past M and columns past K as zeros).
    auto stage = [&](int c) {
        __nv_bfloat16* dst = act_s + (size_t)(c & 1) * kRows * kChunkLd;
        const int k0 = c * kChunk;
        constexpr int kPieces = kChunk / 8;
        for (int idx = threadIdx.x; idx < kRows * kPieces; idx += kThreads) {
            const int r = idx / kPieces, p = idx - r * kPieces;
            const bool valid = r < M && k0 + p * 8 < K;
            cp_async16(dst + r * kChunkLd + p * 8, A + (valid ? (size_t)r * lda + k0 + p * 8 : 0), valid);
        }
    };

    for (int gp = g_begin; gp < g_end; gp += NG) {
        const int ng = min(NG, g_end - gp);
        // This warp's k-block of every chunk (columns c * 256 + warp * 32 ...), for every group of the pass.
        uint4 w[kWRegs];
#pragma unroll
        for (int c = 0; c < MC; ++c)
#pragma unroll
            for (int gi = 0; gi < NG; ++gi) {
                const int f = (gp + gi) * 8 + g, k = c * kChunk + warp * 32 + t * 8;
                w[c * NG + gi] = (c < n_chunks && gi < ng && f < N && k < K) ? __ldg(reinterpret_cast<const uint4*>(W + (size_t)f * ldw + k))
                                                                           : make_uint4(0, 0, 0, 0);
            }
        float acc[NG][MT][4];
#pragma unroll
        for (int i = 0; i < NG; ++i)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[i][m][0] = acc[i][m][1] = acc[i][m][2] = acc[i][m][3] = 0.0f;
        if (gp == g_begin) {
            // The first pass's weights are under way; the activations come from the kernel before this one.
            if constexpr (STAGE == 2) {
                layernorm_rows_to_smem(norm, M, K, act_s, ld_full, n_chunks * kChunk);
                __syncthreads();
            } else if constexpr (STAGE == 1) {
                lb_wait_for_predecessor();
                lb_dependents_may_launch();
                const int pieces = n_chunks * kChunk / 8;
                for (int idx = threadIdx.x; idx < 16 * pieces; idx += kThreads) {
                    const int r = idx / pieces, p = idx - r * pieces;
                    const bool valid = r < M && p * 8 < K;
                    cp_async16(act_s + r * ld_full + p * 8, A + (valid ? (size_t)r * lda + p * 8 : 0), valid);
                }
                cp_async_commit();
                cp_async_wait<0>();
                __syncthreads();
            } else {
                lb_wait_for_predecessor();
                lb_dependents_may_launch();
            }
        }
        if constexpr (!FULL) {
            stage(0);
            cp_async_commit();
        }
        // A thread finishes at most kEarly elements of a pass (element idx = threadIdx.x + 256 e); their bias and residual
        // are asked for now and arrive under the products instead of after them.
        constexpr int kEarly = (NG * kRows * 8 + kThreads - 1) / kThreads;
        float2 early[kEarly];
#pragma unroll
        for (int e = 0; e < kEarly; ++e) {
            early[e] = make_float2(0.f, 0.f);
            const int idx = threadIdx.x + e * kThreads;
            const int gi = idx / (kRows * 8), rest = idx - gi * kRows * 8, r = rest >> 3, f = (gp + gi) * 8 + (rest & 7);
            if (gi < ng && r < M && f < N)
                early[e] = make_float2(bias != nullptr ? __ldg(bias + f) : 0.0f, residual != nullptr ? __ldcg(residual + (size_t)r * ldr + f) : 0.0f);
        }
#pragma unroll
        for (int c = 0; c < MC; ++c) {
            if (c < n_chunks) {                                 // the same for every thread
                if constexpr (!FULL) {
                    if (c + 1 < n_chunks) stage(c + 1);
                    cp_async_commit();
                    cp_async_wait<1>();
                    __syncthreads();
                }
                const int kLd = FULL ? ld_full : kChunkLd;
                const __nv_bfloat16* buf = (FULL ? act_s + c * kChunk : act_s + (size_t)(c & 1) * kRows * kChunkLd) + warp * 32 + t * 8;
                if (c * kChunk + warp * 32 < K) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const uint4 lo = *reinterpret_cast<const uint4*>(buf + (m * 16 + g) * kLd);
                        const uint4 hi = *reinterpret_cast<const uint4*>(buf + (m * 16 + g + 8) * kLd);
#pragma unroll
                        for (int gi = 0; gi < NG; ++gi) {
                            if (gi < ng) {
                                mma_bf16(acc[gi][m], lo.x, hi.x, lo.y, hi.y, w[c * NG + gi].x, w[c * NG + gi].y);
                                mma_bf16(acc[gi][m], lo.z, hi.z, lo.w, hi.w, w[c * NG + gi].z, w[c * NG + gi].w);
                            }
                        }
                    }
                }
                if constexpr (!FULL) __syncthreads();        // the buffer is free: the chunk after next goes into it
            }
        }
        // Partial tiles of the eight warps -> shared memory -> summed in warp order -> epilogue.
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
            if (gi < ng) {
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float* tile = red_s + ((size_t)(warp * NG + gi) * MT + m) * 128;
                    tile[g * 8 + 2 * t] = acc[gi][m][0];
                    tile[g * 8 + 2 * t + 1] = acc[gi][m][1];
                    tile[(g + 8) * 8 + 2 * t] = acc[gi][m][2];
                    tile[(g + 8) * 8 + 2 * t + 1] = acc[gi][m][3];
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int e = 0; e < kEarly; ++e) {
            const int idx = threadIdx.x + e * kThreads;
            const int gi = idx / (kRows * 8), rest = idx - gi * kRows * 8, r = rest >> 3, cfeat = rest & 7;
            const int f = (gp + gi) * 8 + cfeat;
            if (gi < ng && r < M && f < N) {
                const int m = r >> 4, rr = r & 15;
                float v = 0.0f;
#pragma unroll
                for (int wp = 0; wp < kWarps; ++wp) v += red_s[((size_t)(wp * NG + gi) * MT + m) * 128 + rr * 8 + cfeat];
                float y = lb_activate(v + early[e].x, act);
                if (residual != nullptr) y += early[e].y;
                out[(size_t)r * ldo + f] = lb_from_float<TO>(y);
                if (kv.cache != nullptr && f >= kv.q_dim) {
                    // A key or value feature of a fused projection: also into the token's slot of its cache page.
                    const int kvf = f - kv.q_dim, kv_dim = kv.n_kv_head * kv.head_dim;
                    const int which = kvf >= kv_dim ? 1 : 0, within = kvf - which * kv_dim;
                    const int head = within / kv.head_dim, dd = within - head * kv.head_dim;
                    const int slot = __ldg(kv.slot_mapping + r);
                    if (slot >= 0) {
                        const int page = slot / kv.page_size, off = slot - page * kv.page_size;
                        const size_t plane = (size_t)kv.n_kv_head * kv.page_size * kv.head_dim;
                        kv.cache[(size_t)page * 2 * plane + (size_t)which * plane + ((size_t)head * kv.page_size + off) * kv.head_dim + dd] =
                            __float2bfloat16_rn(y);
                    }
                }
            }
        }
        __syncthreads();
    }
}

template <int MT, int NG, typename TO, int STAGE = 0>
int launch(const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, const float* residual, int64_t ldr,
           void* out, int64_t ldo, int M, int N, int K, int act, KvScatter kv, int n_sm, cudaStream_t s, RowNorm norm = RowNorm{}) {
    const size_t ld_full = (size_t)(K + kChunk - 1) / kChunk * kChunk + 32;
    const size_t act_bytes = STAGE != 0 ? 16 * ld_full * sizeof(__nv_bfloat16) : (size_t)2 * MT * 16 * kChunkLd * sizeof(__nv_bfloat16);
    const size_t smem = act_bytes + (size_t)kWarps * NG * MT * 128 * sizeof(float);
    static size_t configured = 0;
    if (smem > configured) {
        LB_CHECK_CUDA(cudaFuncSetAttribute(gemm_rows_kernel<MT, NG, TO, STAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    const int n_groups = (N + 7) / 8;
    const int grid = n_groups < n_sm ? n_groups : n_sm;
    LB_CHECK_CUDA(lb_launch_overlapped(gemm_rows_kernel<MT, NG, TO, STAGE>, dim3(grid), dim3(kThreads), smem, s, (const __nv_bfloat16*)A, lda,
                                       (const __nv_bfloat16*)W, ldw, bias, residual, ldr, (TO*)out, ldo, M, N, K, act, kv, norm));
    return LB_OK;
}

template <int MT, typename TO, int STAGE = 0>
int launch_by_k(const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, const float* residual, int64_t ldr,
                void* out, int64_t ldo, int M, int N, int K, int act, KvScatter kv, int n_sm, cudaStream_t s) {
    if (K <= 4 * kChunk) return launch<MT, 4, TO, STAGE>(A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, kv, n_sm, s);
    if (K <= 8 * kChunk) return launch<MT, 2, TO, STAGE>(A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, kv, n_sm, s);
    return launch<MT, 1, TO, STAGE>(A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, kv, n_sm, s);
}

}  // namespace

// Whether the kernel takes the product: 1 to 64 tokens, a reduction length of up to 4096, K and the row strides of
// A and W multiples of 8, 16-byte aligned bases, and at most four passes over the feature groups of a block (the
// head's vocabulary is left to the tcgen05 kernel, whose tiles suit it).
extern "C" int lb_gemm_rows_supports(const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N, int K) {
    if (M <= 0 || M > kMaxRows || N <= 0 || K <= 0) return 0;
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)A & 15) != 0 || ((uintptr_t)W & 15) != 0) return 0;
    if (K > kWRegs * kChunk) return 0;
    const int ng = K <= 4 * kChunk ? 4 : K <= 8 * kChunk ? 2 : 1;
    return (N + 7) / 8 <= 148 * 4 * ng;
}

// The same product for up to 16 tokens and a reduction length of up to 1024 with the activations made in the kernel:
// LayerNorm (two-pass 32-bit statistics, eps, gain and offset or null) of the float32 rows x, normalised by every
// block for itself.  lb_gemm_rows_normed_supports says whether the kernel takes the operands.
extern "C" int lb_gemm_rows_normed_supports(const void* x, int64_t ldx, const void* W, int64_t ldw, int M, int N, int K) {
    if (M <= 0 || M > 16 || N <= 0 || K <= 0 || K > 4 * kChunk) return 0;
    if (K % 8 != 0 || ldx % 4 != 0 || ldw % 8 != 0 || ((uintptr_t)x & 15) != 0 || ((uintptr_t)W & 15) != 0) return 0;
    return (N + 7) / 8 <= 148 * 4 * 4;
}

extern "C" int lb_gemm_rows_normed(int out_dtype, const float* x, int64_t ldx, const float* gain, const float* offset, float eps,
                                   const void* W, int64_t ldw, const float* bias, const float* residual, int64_t ldr, void* out,
                                   int64_t ldo, int M, int N, int K, int act, void* kv_cache, const int32_t* slot_mapping, int q_dim,
                                   int n_kv_head, int head_dim, int page_size, void* stream) {
    LB_CHECK_ARG(out_dtype == LB_BF16 || out_dtype == LB_F32, "gemm_rows_normed: unknown output dtype %d", out_dtype);
    if (!lb_gemm_rows_normed_supports(x, ldx, W, ldw, M, N, K) || ((uintptr_t)gain & 15) != 0 || ((uintptr_t)offset & 15) != 0)
        return lb_fail(LB_ERR_UNSUPPORTED, "gemm_rows_normed: takes 1 to 16 tokens, K up to 1024 and a multiple of 8, 16-byte aligned bases "
                       "(M=%d N=%d K=%d ldx=%lld ldw=%lld)", M, N, K, (long long)ldx, (long long)ldw);
    LB_CHECK_ARG(ldx >= K && ldw >= K && ldo >= N, "gemm_rows_normed: a row stride is shorter than the row");
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        LB_CHECK_CUDA(cudaGetDevice(&dev));
        LB_CHECK_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
    }
    KvScatter kv{static_cast<__nv_bfloat16*>(kv_cache), slot_mapping, q_dim, n_kv_head, head_dim, page_size};
    if (kv_cache != nullptr)
        LB_CHECK_ARG(slot_mapping != nullptr && q_dim >= 0 && n_kv_head > 0 && head_dim > 0 && page_size > 0 &&
                         q_dim + 2 * n_kv_head * head_dim == N,
                     "gemm_rows_normed: the cache destination needs N = q_dim + 2 * n_kv_head * head_dim (N=%d q_dim=%d heads %d x %d)", N,
                     q_dim, n_kv_head, head_dim);
    const RowNorm norm{x, ldx, gain, offset, eps};
    auto s = static_cast<cudaStream_t>(stream);
    if (out_dtype == LB_F32)
        return launch<1, 4, float, 2>(nullptr, 0, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, kv, n_sm, s, norm);
    return launch<1, 4, __nv_bfloat16, 2>(nullptr, 0, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, kv, n_sm, s, norm);
}

extern "C" int lb_gemm_rows(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias,
                            const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act,
                            void* kv_cache, const int32_t* slot_mapping, int q_dim, int n_kv_head, int head_dim, int page_size,
                            void* stream) {
    LB_CHECK_ARG(out_dtype == LB_BF16 || out_dtype == LB_F32, "gemm_rows: unknown output dtype %d", out_dtype);
    if (!lb_gemm_rows_supports(A, lda, W, ldw, M, N, K))
        return lb_fail(LB_ERR_UNSUPPORTED, "gemm_rows: takes 1 to 64 tokens, K and row strides multiples of 8 and 16-byte aligned "
                       "bases (M=%d N=%d K=%d lda=%lld ldw=%lld)", M, N, K, (long long)lda, (long long)ldw);
    LB_CHECK_ARG(lda >= K && ldw >= K && ldo >= N, "gemm_rows: a row stride is shorter than the row");
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        LB_CHECK_CUDA(cudaGetDevice(&dev));
        LB_CHECK_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
    }
    KvScatter kv{static_cast<__nv_bfloat16*>(kv_cache), slot_mapping, q_dim, n_kv_head, head_dim, page_size};
    if (kv_cache != nullptr)
        LB_CHECK_ARG(slot_mapping != nullptr && q_dim >= 0 && n_kv_head > 0 && head_dim > 0 && page_size > 0 &&
                         q_dim + 2 * n_kv_head * head_dim == N,
                     "gemm_rows: the cache destination needs N = q_dim + 2 * n_kv_head * head_dim (N=%d q_dim=%d heads %d x %d)", N,
                     q_dim, n_kv_head, head_dim);
    auto s = static_cast<cudaStream_t>(stream);
    const int mt = (M + 15) / 16;
#define LB_GO(MT)                                                                                                          \
    return out_dtype == LB_F32 ? launch_by_k<MT, float>(A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, kv, n_sm, s)   \
                               : launch_by_k<MT, __nv_bfloat16>(A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, kv, n_sm, s)
    if (mt <= 1)           // up to 16 tokens: all columns of the activations at once
        return out_dtype == LB_F32 ? launch_by_k<1, float, 1>(A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, kv, n_sm, s)
                                   : launch_by_k<1, __nv_bfloat16, 1>(A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, kv, n_sm, s);
    if (mt == 2) LB_GO(2);
    if (mt == 3) LB_GO(3);
    LB_GO(4);
#undef LB_GO
}
