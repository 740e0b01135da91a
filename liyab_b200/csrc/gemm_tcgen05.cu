// out[M, N] = epilogue(A[M, K] . W[N, K]^T) for bfloat16 operands on the fifth
// generation tensor cores: operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), products issued by one thread with
// tcgen05.mma into an accumulator in tensor memory, read back with tcgen05.ld
// for the epilogue (bias, activation, residual sum, in the reference's order:
// src/core/transformer.cpp:111-118, 4903-4912, 5526-5532).
//
// The product is computed transposed: the weight tile [128 output features x 64]
// is the instruction's M operand and the activation tile [BN tokens x 64] its N
// operand, so a decode step with a handful of tokens still fills the 128 rows of
// the instruction with weights, and every weight byte crosses HBM once.  In
// tensor memory lane i holds feature n0 + i and column j holds token m0 + j; the
// 32 threads of an epilogue warp therefore write 32 consecutive features of one
// token with each store.
//
// One CTA computes one [128 x BN] tile.  Warp 0 issues the TMA loads, warp 1
// allocates tensor memory and issues the MMAs, warps 2..5 run the epilogue.  A
// ring of shared-memory stages is handed back and forth through mbarriers
// (full: TMA bytes landed; empty: tcgen05.commit after the MMAs that read the
// stage).  Every wait is bounded: after about two seconds without progress the
// kernel records where it gave up in a device status word, skips the rest, waits
// for its own copies, frees its tensor memory and returns.
//
// Sizes: any M and N (TMA fills out-of-range rows with zeros, stores are
// masked); K a multiple of 8 and both row strides multiples of 8 elements
// (16-byte TMA rule); everything else is refused by the host function.
#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"

#include <map>
#include <mutex>
#include <tuple>

namespace {

using namespace lb_tc;

constexpr int kThreads = 192;

__device__ int g_status = 0;         // 0 ok; else (site << 8) | detail of the first bounded wait that ran out
static int g_withhold_next = 0;      // host side: the next launch leaves its accumulator-ready barrier unsignalled (tests)

// ------------------------------------------------------------------ the kernel

// `lane operand`: the matrix whose rows become the 128 lanes of the accumulator (the instruction's M);
// `column operand`: the matrix whose BN rows become its columns (the instruction's N).
template <int BN, int STAGES>
struct SharedStorage {
    alignas(1024) __nv_bfloat16 lane_tile[STAGES][kLaneTile * kBlockK];   // 16 KB each
    alignas(1024) __nv_bfloat16 col_tile[STAGES][BN * kBlockK];
    alignas(8) uint64_t full[STAGES];
    alignas(8) uint64_t empty[STAGES];
    alignas(8) uint64_t acc_ready;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void store_row16(float* dst, const float (&x)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
}

__device__ __forceinline__ void store_row16(__nv_bfloat16* dst, const float (&x)[16]) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 v;
        v.x = pack2(x[8 * i], x[8 * i + 1]);
        v.y = pack2(x[8 * i + 2], x[8 * i + 3]);
        v.z = pack2(x[8 * i + 4], x[8 * i + 5]);
        v.w = pack2(x[8 * i + 6], x[8 * i + 7]);
        reinterpret_cast<uint4*>(dst)[i] = v;
    }
}

// TOKENS_ON_LANES = false (few tokens): the weights are the lane operand, lane i = feature n0 + i, column
// j = token m0 + j.  TOKENS_ON_LANES = true (many tokens): the activations are the lane operand, lane i =
// token m0 + i, column j = feature n0 + j, so a thread owns a run of one token's features and stores vectors.
template <int BN, int STAGES, bool TOKENS_ON_LANES, typename TO>
__global__ void __launch_bounds__(kThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_lane, const __grid_constant__ CUtensorMap map_col,
                    const float* __restrict__ bias, const float* residual, int64_t ldr, TO* out, int64_t ldo, int M,
                    int N, int K, int act, int vec_ok, float* partial, int* counters, int n_splits, int withhold_ready) {
    extern __shared__ uint8_t smem_raw[];
    using Storage = SharedStorage<BN, STAGES>;
    Storage& s = *reinterpret_cast<Storage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;
    constexpr uint32_t kStageBytes = (kLaneTile + BN) * kBlockK * sizeof(__nv_bfloat16);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * (TOKENS_ON_LANES ? BN : kLaneTile);     // first output feature of the tile
    const int m0 = blockIdx.y * (TOKENS_ON_LANES ? kLaneTile : BN);     // first token of the tile
    const int lane_row0 = TOKENS_ON_LANES ? m0 : n0, col_row0 = TOKENS_ON_LANES ? n0 : m0;
    // With n_splits > 1 (few tokens, weights on the lanes) block z of a tile takes a range of the k-blocks.
    const int all_kb = (K + kBlockK - 1) / kBlockK;
    const int per_split = (all_kb + n_splits - 1) / n_splits;
    const int kb_first = (int)blockIdx.z * per_split;
    const int n_kb = min(all_kb, kb_first + per_split) - kb_first;
    volatile int* abort_flag = &s.abort_flag;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_lane);
        prefetch_tensormap(&map_col);
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        mbar_init(&s.acc_ready, 1);
        s.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(&s.tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            // The weights of the first ring of stages are asked for before the kernel before this one has ended
            // (they do not depend on it); the activations of those stages follow once it has.
            const int ahead = n_kb < STAGES ? n_kb : STAGES;
            for (int kb = 0; kb < ahead; ++kb) {
                mbar_expect_tx(&s.full[kb], kStageBytes);
                if (TOKENS_ON_LANES) tma_load_2d(s.col_tile[kb], &map_col, &s.full[kb], (kb_first + kb) * kBlockK, col_row0);
                else tma_load_2d(s.lane_tile[kb], &map_lane, &s.full[kb], (kb_first + kb) * kBlockK, lane_row0);
            }
            lb_wait_for_predecessor();
            lb_dependents_may_launch();
            for (int kb = 0; kb < ahead; ++kb) {
                if (TOKENS_ON_LANES) tma_load_2d(s.lane_tile[kb], &map_lane, &s.full[kb], (kb_first + kb) * kBlockK, lane_row0);
                else tma_load_2d(s.col_tile[kb], &map_col, &s.full[kb], (kb_first + kb) * kBlockK, col_row0);
            }
            int issued = ahead;
            for (int kb = ahead; kb < n_kb; ++kb) {
                const int st = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(&s.empty[st], ph ^ 1, abort_flag)) {
                    atomicCAS(&g_status, 0, (1 << 8) | st);
                    s.abort_flag = 1;
                    break;
                }
                mbar_expect_tx(&s.full[st], kStageBytes);
                tma_load_2d(s.lane_tile[st], &map_lane, &s.full[st], (kb_first + kb) * kBlockK, lane_row0);
                tma_load_2d(s.col_tile[st], &map_col, &s.full[st], (kb_first + kb) * kBlockK, col_row0);
                issued = kb + 1;
            }
            if (s.abort_flag != 0 && issued > 0) {
                // Leave no copy in flight: the last stage issued signals its full barrier when its bytes landed.
                const int kb = issued - 1;
                mbar_wait(&s.full[kb % STAGES], (kb / STAGES) & 1, nullptr);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(kLaneTile, BN);
            bool ok = true;
            for (int kb = 0; kb < n_kb && ok; ++kb) {
                const int st = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(&s.full[st], ph, abort_flag)) {
                    atomicCAS(&g_status, 0, (2 << 8) | st);
                    s.abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t l_addr = smem_u32(s.lane_tile[st]), c_addr = smem_u32(s.col_tile[st]);
#pragma unroll
                for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                    const uint32_t off = k * kUmmaK * sizeof(__nv_bfloat16);
                    umma_bf16(tmem_base, umma_desc(l_addr + off), umma_desc(c_addr + off), idesc, (kb | k) != 0 ? 1u : 0u);
                }
                umma_commit(&s.empty[st]);      // the stage is free once these MMAs have read it
            }
            // The accumulator is complete once every MMA retired.  (`withhold_ready`: a test's launch, whose
            // epilogue then meets a barrier that nothing signals and has to give up at its limit.)
            if (ok && withhold_ready == 0) umma_commit(&s.acc_ready);
        }
    } else {
        // Epilogue: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31.
        const int quarter = warp & 3;
        const uint32_t tmem_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
        lb_wait_for_predecessor();           // before the residual is read and anything is written
        lb_dependents_may_launch();
        if (!mbar_wait(&s.acc_ready, 0, abort_flag)) {
            if (lane == 0) atomicCAS(&g_status, 0, (3 << 8) | quarter);
            s.abort_flag = 1;
        } else if (TOKENS_ON_LANES) {
            tc_fence_after();
            const int t = m0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                const int f0 = n0 + c;
                if (f0 >= N) break;              // uniform across the block
                uint32_t v[16];
                tmem_ld16(tmem_row + (uint32_t)c, v);
                tmem_ld_wait();
                if (t >= M) continue;
                float x[16];
                if (vec_ok && f0 + 16 <= N) {
                    float r[16];
                    if (residual != nullptr) {
                        const float4* rp = reinterpret_cast<const float4*>(residual + (size_t)t * ldr + f0);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float4 q = rp[i];
                            r[4 * i] = q.x; r[4 * i + 1] = q.y; r[4 * i + 2] = q.z; r[4 * i + 3] = q.w;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float y = __uint_as_float(v[j]);
                        if (bias != nullptr) y += __ldg(bias + f0 + j);
                        y = lb_activate(y, act);
                        if (residual != nullptr) y += r[j];
                        x[j] = y;
                    }
                    store_row16(out + (size_t)t * ldo + f0, x);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int f = f0 + j;
                        if (f < N) {
                            float y = __uint_as_float(v[j]);
                            if (bias != nullptr) y += bias[f];
                            y = lb_activate(y, act);
                            if (residual != nullptr) y += residual[(size_t)t * ldr + f];
                            out[(size_t)t * ldo + f] = lb_from_float<TO>(y);
                        }
                    }
                }
            }
        } else if (n_splits == 1) {
            tc_fence_after();
            const int f = n0 + quarter * 32 + lane;
            const float b = (bias != nullptr && f < N) ? bias[f] : 0.0f;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (m0 + c >= M) break;          // uniform across the block
                uint32_t v[16];
                tmem_ld16(tmem_row + (uint32_t)c, v);
                tmem_ld_wait();
                if (f < N) {
                    // All of the chunk's residual values are requested before the first store: the output may
                    // be the residual buffer itself, and a load queued behind a store would wait for it.
                    float r[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = m0 + c + j;
                        r[j] = (residual != nullptr && t < M) ? residual[(size_t)t * ldr + f] : 0.0f;
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = m0 + c + j;
                        if (t < M) out[(size_t)t * ldo + f] = lb_from_float<TO>(lb_activate(__uint_as_float(v[j]) + b, act) + r[j]);
                    }
                }
            }
        } else {
            // Split K: this block's partial sums go to scratch [split][token][feature]; a second, element-wise
            // kernel adds the splits in order and finishes the elements.
            tc_fence_after();
            const int f = n0 + quarter * 32 + lane;
            float* mine = partial + ((size_t)blockIdx.z * M) * N;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (m0 + c >= M) break;
                uint32_t v[16];
                tmem_ld16(tmem_row + (uint32_t)c, v);
                tmem_ld_wait();
                if (f < N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = m0 + c + j;
                        if (t < M) mine[(size_t)t * N + f] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    __syncwarp();            // the elected lanes rejoin their warps before the block-wide barrier
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Where a split product is a fused projection of queries, keys and values, its second half also puts the keys and
// values (the features from q_dim on) into the tokens' cache slots, as lb_kv_append would.
struct FinishKv {
    __nv_bfloat16* cache = nullptr;
    const int32_t* slot_mapping = nullptr;
    int q_dim = 0, n_kv_head = 0, head_dim = 0, page_size = 0;
};

// out[t, f] = act(sum over splits, in order, of partial[split][t][f] + bias[f]) + residual[t, f].
template <typename TO>
__global__ void splitk_finish_kernel(const float* __restrict__ partial, const float* __restrict__ bias, const float* residual,
                                     int64_t ldr, TO* out, int64_t ldo, int M, int N, int n_splits, int act, const FinishKv kv) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const bool mine = idx < M * N;
    const int t = mine ? idx / N : 0, f = mine ? idx - t * N : 0;
    // The bias is a weight, and the residual was complete before the product whose sums this kernel finishes began
    // its own work (that product waited for the kernel before it): both are asked for before this kernel waits for
    // the product.  (Through L2: what an SM's first-level cache may still hold of the residual is older.)
    const float b = (mine && bias != nullptr) ? __ldg(bias + f) : 0.0f;
    const float r = (mine && residual != nullptr) ? __ldcg(residual + (size_t)t * ldr + f) : 0.0f;
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    if (!mine) return;
    float v[16];
#pragma unroll
    for (int sp = 0; sp < 16; ++sp) v[sp] = sp < n_splits ? partial[((size_t)sp * M + t) * N + f] : 0.0f;
    float acc = 0.0f;
#pragma unroll
    for (int sp = 0; sp < 16; ++sp) acc += v[sp];
    float y = lb_activate(acc + b, act);
    if (residual != nullptr) y += r;
    out[(size_t)t * ldo + f] = lb_from_float<TO>(y);
    if (kv.cache != nullptr && f >= kv.q_dim) {
        const int slot = kv.slot_mapping[t];
        if (slot >= 0) {
            const int kv_dim = kv.n_kv_head * kv.head_dim, kvf = f - kv.q_dim, which = kvf >= kv_dim ? 1 : 0;
            const int within = kvf - which * kv_dim, head = within / kv.head_dim, dd = within - head * kv.head_dim;
            const int page = slot / kv.page_size, off = slot - page * kv.page_size;
            const size_t plane = (size_t)kv.n_kv_head * kv.page_size * kv.head_dim;
            kv.cache[(size_t)page * 2 * plane + (size_t)which * plane + ((size_t)head * kv.page_size + off) * kv.head_dim + dd] =
                __float2bfloat16_rn(y);
        }
    }
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// A [rows, cols] matrix with `ld` elements between rows, moved in boxes of [box_rows, 128 bytes].
int make_map(CUtensorMap* map, const void* base, int elem_bytes, int rows, int cols, int64_t ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return lb_fail(LB_ERR_BACKEND, "gemm_tcgen05: cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * (cuuint64_t)elem_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                          const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return lb_fail(LB_ERR_BACKEND, "gemm_tcgen05: cuTensorMapEncodeTiled failed with %d (rows %d cols %d ld %lld box rows %d)",
                       (int)r, rows, cols, (long long)ld, box_rows);
    return LB_OK;
}

// Tensor maps are cached by what they describe: encoding costs microseconds on the host, a decode step has dozens.
struct MapKey {
    const void* base;
    int elem_bytes, rows, cols, box_rows;
    int64_t ld;
    bool operator<(const MapKey& o) const {
        return std::tie(base, elem_bytes, rows, cols, box_rows, ld) < std::tie(o.base, o.elem_bytes, o.rows, o.cols, o.box_rows, o.ld);
    }
};

int cached_map(CUtensorMap* out, const void* base, int rows, int cols, int64_t ld, int box_rows) {
    return lb_tensor_map_2d(out, base, 2, rows, cols, ld, box_rows);
}

template <int BN, int STAGES, bool TOKENS_ON_LANES, typename TO>
int launch(const CUtensorMap& map_lane, const CUtensorMap& map_col, const float* bias, const float* residual, int64_t ldr,
           void* out, int64_t ldo, int M, int N, int K, int act, int vec_ok, float* partial, int* counters, int n_splits,
           cudaStream_t stream) {
    constexpr size_t smem = sizeof(SharedStorage<BN, STAGES>) + 1024;
    static bool configured = false;
    if (!configured) {
        LB_CHECK_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, TOKENS_ON_LANES, TO>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    dim3 grid(TOKENS_ON_LANES ? (N + BN - 1) / BN : (N + kLaneTile - 1) / kLaneTile,
              TOKENS_ON_LANES ? (M + kLaneTile - 1) / kLaneTile : (M + BN - 1) / BN, n_splits);
    LB_CHECK_CUDA(lb_launch_overlapped_kind(1, gemm_tcgen05_kernel<BN, STAGES, TOKENS_ON_LANES, TO>, grid, dim3(kThreads), smem, stream, map_lane,
                                       map_col, bias, residual, ldr, (TO*)out, ldo, M, N, K, act, vec_ok, partial, counters, n_splits,
                                       g_withhold_next));
    g_withhold_next = 0;
    return LB_OK;
}

}  // namespace

int lb_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, int rows, int cols, int64_t ld, int box_rows) {
    static std::map<MapKey, CUtensorMap> cache;
    static std::mutex mu;
    const MapKey key{base, elem_bytes, rows, cols, box_rows, ld};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
        CUtensorMap m;
        const int rc = make_map(&m, base, elem_bytes, rows, cols, ld, box_rows);
        if (rc != LB_OK) return rc;
        if (cache.size() > 4096) cache.clear();
        it = cache.emplace(key, m).first;
    }
    *out = it->second;
    return LB_OK;
}

int lb_tc_status_word(int** out) {
    static int* addr = nullptr;
    if (addr == nullptr) LB_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_status));
    *out = addr;
    return LB_OK;
}

// The tile along the tokens for M tokens: 16, 32 or 64 tokens as accumulator columns (weights on the
// lanes) up to 64 tokens; beyond that 128 tokens on the lanes (reported as 128, or 256 when the product is
// large enough to fill the GPU several times with 128 x 256 tiles).
extern "C" int lb_gemm_tcgen05_token_tile(int M, int N) {
    if (M <= 16) return 16;
    if (M <= 32) return 32;
    if (M <= 64) return 64;
    const long long big_tiles = (long long)((M + 127) / 128) * ((N + 255) / 256);
    return big_tiles >= 4 * 148 ? 256 : 128;
}

static int gemm_tcgen05_run(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias,
                            const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act,
                            int token_tile, float* partial, int* counters, int n_splits, const FinishKv& kv, void* stream) {
    LB_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm_tcgen05: bad sizes M=%d N=%d K=%d", M, N, K);
    if (n_splits < 1) n_splits = 1;
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)A & 15) != 0 || ((uintptr_t)W & 15) != 0)
        return lb_fail(LB_ERR_UNSUPPORTED,
                       "gemm_tcgen05: TMA needs K and both row strides to be multiples of 8 elements and 16-byte aligned "
                       "bases (K=%d lda=%lld ldw=%lld)", K, (long long)lda, (long long)ldw);
    LB_CHECK_ARG(lda >= K && ldw >= K && ldo >= N, "gemm_tcgen05: a row stride is shorter than the row");
    LB_CHECK_ARG(out_dtype == LB_BF16 || out_dtype == LB_F32, "gemm_tcgen05: unknown output dtype %d", out_dtype);
    if (M == 0) return LB_OK;
    const int tile = token_tile > 0 ? token_tile : lb_gemm_tcgen05_token_tile(M, N);
    LB_CHECK_ARG(tile == 16 || tile == 32 || tile == 64 || tile == 128 || tile == 256, "gemm_tcgen05: token tile %d", tile);
    const bool tokens_on_lanes = tile >= 128;
    LB_CHECK_ARG(kv.cache == nullptr || n_splits > 1, "gemm_tcgen05: the cache is filled from the second half of a split product only");
    if (n_splits > 1) {
        const int all_kb = (K + kBlockK - 1) / kBlockK;
        LB_CHECK_ARG(!tokens_on_lanes && partial != nullptr && n_splits <= 16,
                     "gemm_tcgen05: K is split (at most 16 ways) only with at most 64 tokens, and needs scratch");
        n_splits = n_splits > all_kb ? all_kb : n_splits;
        const int per = (all_kb + n_splits - 1) / n_splits;
        n_splits = (all_kb + per - 1) / per;                  // no block without a k-block
    }
    const int token_box = tokens_on_lanes ? kLaneTile : tile;
    const int feature_box = tokens_on_lanes ? tile : kLaneTile;       // tile 128/256 names the feature columns there
    LB_CHECK_ARG((M + token_box - 1) / token_box <= 65535, "gemm_tcgen05: M=%d is too large for one launch", M);
    CUtensorMap map_w, map_a;
    int rc = cached_map(&map_w, W, N, K, ldw, feature_box);
    if (rc != LB_OK) return rc;
    rc = cached_map(&map_a, A, M, K, lda, token_box);
    if (rc != LB_OK) return rc;
    auto s = static_cast<cudaStream_t>(stream);
    // Vector stores need 16-byte aligned rows of the output (and of the residual and bias when given).
    const int elem = out_dtype == LB_F32 ? 4 : 2;
    const int vec_ok = ((uintptr_t)out & 15) == 0 && (ldo * elem) % 16 == 0 &&
                       (residual == nullptr || (((uintptr_t)residual & 15) == 0 && (ldr * 4) % 16 == 0));
#define LB_GO(BN, STAGES, TOL, TO)                                                                                \
    {                                                                                                             \
        rc = launch<BN, STAGES, TOL, TO>(TOL ? map_a : map_w, TOL ? map_w : map_a, bias, residual, ldr, out, ldo, M, N, K, \
                                         act, vec_ok, partial, counters, n_splits, s);                            \
        if (rc != LB_OK || n_splits == 1) return rc;                                                              \
        LB_CHECK_CUDA(lb_launch_overlapped_kind(2, splitk_finish_kernel<TO>, dim3((M * N + 255) / 256), dim3(256), 0, s, partial, bias, residual, \
                                           ldr, (TO*)out, ldo, M, N, n_splits, act, kv));                          \
        return LB_OK;                                                                                             \
    }
    if (out_dtype == LB_BF16) {
        switch (tile) {
            case 16: LB_GO(16, 4, false, __nv_bfloat16);
            case 32: LB_GO(32, 4, false, __nv_bfloat16);
            case 64: LB_GO(64, 4, false, __nv_bfloat16);
            case 128: LB_GO(128, 3, true, __nv_bfloat16);
            default: LB_GO(256, 4, true, __nv_bfloat16);
        }
    }
    switch (tile) {
        case 16: LB_GO(16, 4, false, float);
        case 32: LB_GO(32, 4, false, float);
        case 64: LB_GO(64, 4, false, float);
        case 128: LB_GO(128, 3, true, float);
        default: LB_GO(256, 4, true, float);
    }
#undef LB_GO
}

extern "C" int lb_gemm_tcgen05(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias,
                               const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act,
                               int token_tile, float* partial, int* counters, int n_splits, void* stream) {
    return gemm_tcgen05_run(out_dtype, A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, token_tile, partial, counters,
                            n_splits, FinishKv{}, stream);
}

// How many ways lb_gemm_tcgen05 would really split K when asked for n_splits (no block is left without a k-block).
extern "C" int lb_gemm_tcgen05_splits(int M, int K, int n_splits) {
    if (M > 64 || n_splits <= 1) return 1;
    const int all_kb = (K + kBlockK - 1) / kBlockK;
    n_splits = n_splits > 16 ? 16 : n_splits;
    n_splits = n_splits > all_kb ? all_kb : n_splits;
    const int per = (all_kb + n_splits - 1) / n_splits;
    return (all_kb + per - 1) / per;
}

extern "C" int lb_gemm_tcgen05_kv(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias,
                                  void* out, int64_t ldo, int M, int N, int K, float* partial, int n_splits, void* kv_cache,
                                  const int32_t* slot_mapping, int q_dim, int n_kv_head, int head_dim, int page_size, void* stream) {
    LB_CHECK_ARG(kv_cache != nullptr && slot_mapping != nullptr && n_kv_head > 0 && head_dim > 0 && page_size > 0 && q_dim >= 0 &&
                     q_dim + 2 * n_kv_head * head_dim == N,
                 "gemm_tcgen05_kv: %d features are not [q %d | k | v] of %d heads of %d", N, q_dim, n_kv_head, head_dim);
    if (lb_gemm_tcgen05_splits(M, K, n_splits) <= 1)
        return lb_fail(LB_ERR_UNSUPPORTED, "gemm_tcgen05_kv: needs a split of K (at most 64 tokens, more than one k-block)");
    FinishKv kv;
    kv.cache = static_cast<__nv_bfloat16*>(kv_cache);
    kv.slot_mapping = slot_mapping;
    kv.q_dim = q_dim;
    kv.n_kv_head = n_kv_head;
    kv.head_dim = head_dim;
    kv.page_size = page_size;
    return gemm_tcgen05_run(out_dtype, A, lda, W, ldw, bias, nullptr, 0, out, ldo, M, N, K, 0, 0, partial, nullptr, n_splits, kv, stream);
}

// Reads and clears the status word of the bounded waits (0: every wait so far completed).  Synchronises the device.
extern "C" int lb_gemm_tcgen05_status(int* status) {
    int zero = 0;
    LB_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_status, sizeof(int)));
    LB_CHECK_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
    return LB_OK;
}

// The same word without a device synchronisation: copies it into `host` (pinned memory) on `stream`;
// lb_gemm_tcgen05_status_clear zeroes it on `stream`.
extern "C" int lb_gemm_tcgen05_status_async(int* host, void* stream) {
    int* word = nullptr;
    const int rc = lb_tc_status_word(&word);
    if (rc != LB_OK) return rc;
    LB_CHECK_CUDA(cudaMemcpyAsync(host, word, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    return LB_OK;
}

extern "C" int lb_gemm_tcgen05_status_clear(void* stream) {
    int* word = nullptr;
    const int rc = lb_tc_status_word(&word);
    if (rc != LB_OK) return rc;
    LB_CHECK_CUDA(cudaMemsetAsync(word, 0, sizeof(int), static_cast<cudaStream_t>(stream)));
    return LB_OK;
}

// The next launch of the one-tile kernel never signals its accumulator-ready barrier: its epilogue warps wait
// to their limit (about two seconds), report it in the status word and go on to the block's end, where the
// tensor memory is given back.  A test of the give-up path that faults nothing.
extern "C" int lb_gemm_tcgen05_withhold_next(int on) {
    g_withhold_next = on != 0 ? 1 : 0;
    return LB_OK;
}

// Writes the word (tests of the host's handling of a reported wait; synchronises).
extern "C" int lb_gemm_tcgen05_status_set(int value) {
    LB_CHECK_CUDA(cudaMemcpyToSymbol(g_status, &value, sizeof(int)));
    return LB_OK;
}
