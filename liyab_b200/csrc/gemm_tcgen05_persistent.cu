// out[M, N] = epilogue(A[M, K] . W[N, K]^T) for many tokens (prefill): a persistent
// tcgen05 kernel with the epilogue of one tile under the main loop of the next.
//
// One block per SM walks tiles of [128 tokens x BN features] (BN chosen by the
// host, 32..256).  Tokens are the lanes of the accumulator, features its columns.
//   warp 0      TMA producer: A and W k-blocks into a ring of shared-memory stages,
//               and the tile's residual [128 x BN] float32 into the staging buffer.
//   warp 1      allocates tensor memory (two accumulators) and issues tcgen05.mma.
//   warps 2..9  epilogue, in two groups of four that take alternate 128-byte-wide
//               strips of the tile: tcgen05.ld of their 32 lanes, bias, activation,
//               residual (read from the staging buffer, where TMA put it), result
//               written back to the same place, then one TMA store per strip.
// The two single-thread roles run once per k-block while the tensor pipe waits for
// them, so their loops are kept to a few dozen instructions (32-bit shared-memory
// addresses, running stage index, descriptor words advanced by addition).
// The staging buffer is laid out as TMA's 128-byte swizzle wants it ([strip][128
// rows][128 bytes], 16-byte chunk c of row r at chunk c ^ (r & 7)), which also
// keeps a warp's stores to it (one row per thread) free of bank conflicts.  Global
// memory is therefore only touched by TMA: every load and store is a full,
// coalesced tile, clipped by the hardware at the matrix's edge, and the residual
// arrives while the products run.
//
// Handshakes (all mbarriers; every wait is bounded and a wait that runs out makes
// the whole block stop, drain its copies, free tensor memory and return, leaving a
// code in the device status word):
//   full[s] / empty[s]        stage s holds a k-block / has been read by the MMAs
//   acc_full[b] / acc_empty[b] accumulator b is complete / has been read out
//   res_full / staging_free   the residual landed / the last tile's stores have
//                             read the staging buffer
//
// Epilogue order as the reference's (src/core/transformer.cpp:111-118, 4903-4912,
// 5526-5532): bias, activation, then the residual sum, all in 32-bit.
#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace lb_tc;

constexpr int kEpilogueWarps = 8;
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kThreads = 64 + kEpilogueThreads;
constexpr int kMaxStages = 8;
constexpr int kStripBytes = 128 * 128;        // [128 rows][128 bytes]
constexpr int kATileBytes = kLaneTile * kBlockK * (int)sizeof(__nv_bfloat16);
constexpr size_t kSmemLimit = 227 * 1024;

struct Control {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t res_full;
    uint64_t staging_free;
    uint64_t peer_sent;         // (pairs) the other block's half of this block's strips lies in the staging buffer
    uint64_t may_send;          // (pairs) the other block has read what this block sent for the tile before
    uint32_t tmem_base;
    int abort_flag;
};

// Optional time stamps (nanoseconds of the global timer), eight per block, for finding out where a launch's time
// goes: 0 entry, 1 set-up done, 2 first k-block landed, 3 first tile's products issued, 4 first accumulator
// complete, 5 first tile staged, 6 last store complete, 7 last load issued.  Off (null) unless a buffer is set.
__device__ __forceinline__ void stamp(unsigned long long* timing, int slot) {
    if (timing != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        timing[(size_t)blockIdx.x * 8 + slot] = t;
    }
}

unsigned long long* g_timing = nullptr;

__device__ __forceinline__ void give_up(Control* c, int* status, int site, int detail) {
    atomicCAS(status, 0, (site << 8) | (detail & 0xff));
    c->abort_flag = 1;
}

// The loops of the two single-thread roles run once per k-block while the tensor pipe waits for them: they work on
// 32-bit shared-memory addresses and a running stage index, with no division and no 64-bit pointer arithmetic.
__device__ __forceinline__ bool try_wait_u32(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool wait_u32(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (try_wait_u32(bar, parity)) return true;
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
        if (try_wait_u32(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (try_wait_u32(bar, parity)) return true;
        if (abort_flag != nullptr && *abort_flag != 0) return false;
        if (clock64() - t0 > kWaitLimitCycles) return false;
    }
}

// Handshakes between the two blocks of a pair (a cluster): the address of a barrier or of a piece of the staging
// buffer in the other block, an arrival there that publishes this thread's (and, after a warp barrier, its warp's)
// writes to the cluster, a wait that sees what the other block published, and a float32 addition into the other
// block's shared memory.
__device__ __forceinline__ uint32_t peer_address(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ void arrive_at_peer(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ bool try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
        if (try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (try_wait_cluster(bar, parity)) return true;
        if (abort_flag != nullptr && *abort_flag != 0) return false;
        if (clock64() - t0 > kWaitLimitCycles) return false;
    }
}
__device__ __forceinline__ void store_at_peer(uint32_t remote, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ void expect_tx_u32(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tma_load_u32(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void commit_u32(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// tcgen05.mma with both shared-memory descriptors given as (low word, common high word).
__device__ __forceinline__ void umma_lo(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ float4 lds4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts4(uint32_t addr, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void sts4(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// The activation inside the epilogue.  Results that are rounded to bfloat16 take tanh as 1 - 2 / (1 + exp(2u)) with
// the fast exponential and division (relative error about 1e-6, far below bfloat16's rounding), a few
// instructions instead of dozens; float32 results take the library functions.
template <int ACT, bool FAST>
__device__ __forceinline__ float activate(float x) {
    if constexpr (ACT == LB_ACT_GELU_TANH) {
        if constexpr (FAST) {
            const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
            const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));
            return 0.5f * x * (1.0f + t);
        } else {
            return lb_gelu_tanh(x);
        }
    } else if constexpr (ACT == LB_ACT_GELU_ERF) {
        return lb_gelu_erf(x);
    } else {
        return x;
    }
}

// Where the features from q_dim on go instead of `out` when the product is a fused query/key/value projection:
// the pages of the cache ([page][K|V][kv_head][slot][head_dim]), row (token) i at slot_mapping[i] (negative: nowhere).
// A 64-feature strip lies inside one head (head_dim and q_dim are multiples of 64): 128 contiguous bytes per token.
struct KvTarget {
    __nv_bfloat16* cache;
    const int32_t* slot_mapping;
    int q_dim, n_kv_head, head_dim, page_shift;
};

// PAIR: two blocks (a cluster) share every tile, each with half of the k-blocks and its own accumulator, and each
// finishes half of the tile's strips (block r the strips r, r + 2, ...): it sends its sums of the other block's strips
// into that block's staging buffer through distributed shared memory (the slot of the neighbouring strip, which that
// block does not use), and adds what it receives for its own strips, with bias and residual, before it stores them.
// A product with few tiles and a long reduction (the down projection) gets twice the blocks without handing partial
// tiles through global memory.  Float32 output without activation, an even number of strips.
template <typename TO, int ACT, bool HAS_RES, bool KV, bool PAIR = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                       const __grid_constant__ CUtensorMap map_res, const __grid_constant__ CUtensorMap map_out,
                       const float* __restrict__ bias, int M, int N, int K, int BN, int n_stages, int* status,
                       unsigned long long* timing, const KvTarget kv) {
    if (threadIdx.x == 0) stamp(timing, 0);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t stage_bytes = (uint32_t)(kLaneTile + BN) * kBlockK * sizeof(__nv_bfloat16);
    constexpr int kStripCols = 128 / (int)sizeof(TO);                 // features per strip: 32 (float32) or 64 (bfloat16)
    const int n_strips = BN / kStripCols;
    uint8_t* staging = base + (size_t)n_stages * stage_bytes;        // a multiple of 1024 from a 1024-aligned base
    float* bias_s = reinterpret_cast<float*>(staging + (size_t)n_strips * kStripBytes);
    Control* c = reinterpret_cast<Control*>(bias_s + 256);
    volatile int* abort_flag = &c->abort_flag;
    const uint32_t stages_u32 = smem_u32(base), staging_u32 = smem_u32(staging), bias_u32 = smem_u32(bias_s);
    const uint32_t full_u32 = smem_u32(&c->full[0]), empty_u32 = smem_u32(&c->empty[0]);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + kLaneTile - 1) / kLaneTile, n_tiles = (N + BN - 1) / BN;
    const int total = m_tiles * n_tiles;
    uint32_t rank = 0;
    if constexpr (PAIR) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int cta = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, n_cta = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int all_kb = (K + kBlockK - 1) / kBlockK;
    const int kb_lo = PAIR && rank != 0 ? (all_kb + 1) / 2 : 0;           // this block's k-blocks: kb_lo .. kb_lo + n_kb - 1
    const int n_kb = PAIR ? (rank == 0 ? (all_kb + 1) / 2 : all_kb - (all_kb + 1) / 2) : all_kb;
    const bool res_here = HAS_RES;
    const int res_first = PAIR ? (int)rank : 0, res_step = PAIR ? 2 : 1;          // the strips whose residual this block needs
    const uint32_t acc_stride = BN > 128 ? 256u : 128u;               // columns between the two accumulators
    const uint32_t tmem_cols = 2 * acc_stride;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_out);
        if (HAS_RES) prefetch_tensormap(&map_res);
        for (int i = 0; i < n_stages; ++i) {
            mbar_init(&c->full[i], 1);
            mbar_init(&c->empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&c->acc_full[i], 1);
            mbar_init(&c->acc_empty[i], kEpilogueThreads / 32);     // one arrival per epilogue warp
        }
        mbar_init(&c->res_full, 1);
        mbar_init(&c->staging_free, 2);
        mbar_init(&c->peer_sent, kEpilogueWarps);
        mbar_init(&c->may_send, kEpilogueWarps);
        c->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(&c->tmem_base, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = c->tmem_base;
    if (threadIdx.x == 0) stamp(timing, 1);
    if constexpr (PAIR) {
        // Both blocks' barriers exist before one arrives at the other's.
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }

    if (warp == 0) {
        if (lane == 0) {
            uint32_t st = 0, empty_parity = 1;                      // a fresh barrier passes a wait for parity 1
            int issued = 0, last_stage = 0;
            uint32_t last_parity = 0;
            bool res_in_flight = false;
            uint32_t res_parity = 0;
            int it = 0;
            bool ok = true;
            // The residual goes out once the ring is full for the first time in a tile (or after the tile's
            // last k-block): by then the loads that the MMAs wait for first are under way.
            const int res_at = (n_kb < n_stages ? n_kb : n_stages) - 1;
            // The first tile's first ring of stages: the weights are asked for before the kernel before this one has
            // ended (they do not depend on it); activations and residual follow once it has.
            const int ahead = res_at + 1;
            int kb_start = 0;
            if (cta < total) {
                const int tile = cta;
                const int m0 = (tile % m_tiles) * kLaneTile, n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < ahead; ++kb) {
                    expect_tx_u32(full_u32 + 8 * kb, stage_bytes);
                    tma_load_u32(stages_u32 + kb * stage_bytes + kATileBytes, &map_w, full_u32 + 8 * kb, (kb_lo + kb) * kBlockK, n0);
                }
                lb_wait_for_predecessor();
                lb_dependents_may_launch();
                for (int kb = 0; kb < ahead; ++kb)
                    tma_load_u32(stages_u32 + kb * stage_bytes, &map_a, full_u32 + 8 * kb, (kb_lo + kb) * kBlockK, m0);
                issued = ahead;
                last_stage = ahead - 1;
                last_parity = 0;
                st = (uint32_t)ahead;
                if (st == (uint32_t)n_stages) {
                    st = 0;
                    empty_parity ^= 1;
                }
                if (res_here) {                    // the staging buffer is free before the first tile
                    mbar_expect_tx(&c->res_full, (uint32_t)((n_strips - res_first + res_step - 1) / res_step) * kStripBytes);
                    for (int sp = res_first; sp < n_strips; sp += res_step)
                        tma_load_2d(staging + (size_t)sp * kStripBytes, &map_res, &c->res_full, n0 + sp * kStripCols, m0);
                    res_in_flight = true;
                    res_parity = 0;
                }
                kb_start = ahead;
            }
            for (int tile = cta; tile < total && ok; tile += n_cta, ++it) {
                const int m0 = (tile % m_tiles) * kLaneTile, n0 = (tile / m_tiles) * BN;
                for (int kb = kb_start; kb < n_kb; ++kb) {
                    if (!wait_u32(empty_u32 + 8 * st, empty_parity, abort_flag)) {
                        give_up(c, status, 1, st);
                        ok = false;
                        break;
                    }
                    const uint32_t dst = stages_u32 + st * stage_bytes, bar = full_u32 + 8 * st;
                    expect_tx_u32(bar, stage_bytes);
                    tma_load_u32(dst, &map_a, bar, (kb_lo + kb) * kBlockK, m0);
                    tma_load_u32(dst + kATileBytes, &map_w, bar, (kb_lo + kb) * kBlockK, n0);
                    ++issued;
                    last_stage = st;
                    last_parity = empty_parity ^ 1;
                    if (++st == (uint32_t)n_stages) {
                        st = 0;
                        empty_parity ^= 1;
                    }
                    if (res_here && kb == res_at) {
                        if (!mbar_wait(&c->staging_free, (it & 1) ^ 1, abort_flag)) {
                            give_up(c, status, 4, 0);
                            ok = false;
                            break;
                        }
                        mbar_expect_tx(&c->res_full, (uint32_t)((n_strips - res_first + res_step - 1) / res_step) * kStripBytes);
                        for (int sp = res_first; sp < n_strips; sp += res_step)
                            tma_load_2d(staging + (size_t)sp * kStripBytes, &map_res, &c->res_full, n0 + sp * kStripCols, m0);
                        res_in_flight = true;
                        res_parity = it & 1;
                    }
                }
                kb_start = 0;
            }
            stamp(timing, 7);
            if (*abort_flag != 0) {
                // Leave no copy in flight: the barriers of the last loads issued complete when their bytes landed.
                if (issued > 0) mbar_wait(&c->full[last_stage], last_parity, nullptr);
                if (res_in_flight) mbar_wait(&c->res_full, res_parity, nullptr);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(kLaneTile, BN);
            // Descriptor words: the high one is the same for every tile (stride between 8-row groups 1024 bytes,
            // version 1, 128-byte swizzle); the low one holds the start address >> 4 and moves with stage and k.
            const uint32_t desc_hi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
            const uint32_t lo0 = ((stages_u32 & 0x3FFFFu) >> 4) | (1u << 16);
            const uint32_t lo_stage = stage_bytes >> 4, lo_w = kATileBytes >> 4;
            uint32_t st = 0, full_parity = 0;
            int it = 0;
            bool ok = true;
            for (int tile = cta; tile < total && ok; tile += n_cta, ++it) {
                const int buf = it & 1;
                if (!mbar_wait(&c->acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag)) {
                    give_up(c, status, 5, buf);
                    break;
                }
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)buf * acc_stride;
                for (int kb = 0; kb < n_kb; ++kb) {
                    if (!wait_u32(full_u32 + 8 * st, full_parity, abort_flag)) {
                        give_up(c, status, 2, st);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (it == 0 && kb == 0) stamp(timing, 2);
                    const uint32_t a_lo = lo0 + st * lo_stage, w_lo = a_lo + lo_w;
                    umma_lo(d, a_lo, w_lo, desc_hi, idesc, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (uint32_t k = 1; k < kBlockK / kUmmaK; ++k)
                        umma_lo(d, a_lo + 2 * k, w_lo + 2 * k, desc_hi, idesc, 1u);      // 16 elements = 32 bytes further
                    commit_u32(empty_u32 + 8 * st);
                    if (++st == (uint32_t)n_stages) {
                        st = 0;
                        full_parity ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(&c->acc_full[buf]);
                if (it == 0) stamp(timing, 3);
            }
        }
    } else {
        // Eight warps in two groups of four: group g stages the strips g, g + 2, ...; within a group warp w owns
        // tensor-memory lanes 32 * (w % 4) .. + 31, one token per thread.
        const int ew = warp - 2;
        const int group = ew >> 2, quarter = warp & 3;
        const int row = quarter * 32 + lane;                           // this thread's token within the tile
        const int et = threadIdx.x - 64;                               // 0..255 among the epilogue threads
        const bool elected = (et & 127) == 0;                          // one per group: issues and tracks its stores
        const uint32_t swz = (uint32_t)(row & 7);
        const uint32_t row_u32 = staging_u32 + (uint32_t)row * 128u;
        lb_wait_for_predecessor();           // before anything this block stores, and before a cache page is written
        lb_dependents_may_launch();
        int it = 0;
        for (int tile = cta; tile < total; tile += n_cta, ++it) {
            const int m0 = (tile % m_tiles) * kLaneTile, n0 = (tile / m_tiles) * BN;
            const int buf = it & 1;
            // The bias of this tile's features.  (The last tile's readers are past their last barrier.)
            for (int i = et; i < BN; i += kEpilogueThreads) bias_s[i] = (bias != nullptr && n0 + i < N) ? bias[n0 + i] : 0.0f;
            bool ok = mbar_wait(&c->acc_full[buf], (it >> 1) & 1, abort_flag);
            if (ok && res_here) ok = mbar_wait(&c->res_full, it & 1, abort_flag);
            if (!ok) give_up(c, status, 3, quarter);
            named_barrier(1, kEpilogueThreads);
            if (*abort_flag != 0) break;                               // the same answer for all epilogue threads
            tc_fence_after();
            if (et == 0 && it == 0) stamp(timing, 4);
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * acc_stride;
            int slot = -1;                                             // where this thread's token lies in the cache
            if constexpr (KV) slot = m0 + row < M ? __ldg(kv.slot_mapping + m0 + row) : -1;
            if constexpr (PAIR) {
                const uint32_t peer = rank ^ 1u;
                const int half = n_strips / 2;
                // This block's sums of the other block's strips go to that block's staging buffer (the slot beside the
                // strip's own), once that block has read what was sent for the tile before.  (The host launches one
                // pair per tile today, so a pair's second tile and its wait are not exercised by any test.)
                if (it > 0 && !wait_cluster(smem_u32(&c->may_send), (uint32_t)((it - 1) & 1), abort_flag)) give_up(c, status, 6, quarter);
                if (*abort_flag == 0) {
                    const uint32_t peer_row = peer_address(row_u32, peer);
                    for (int j = group; j < half; j += 2) {
                        const int sp = (int)peer + 2 * j;
                        uint32_t v[32];
                        tmem_ld32(t_row + (uint32_t)(sp * 32), v);
                        tmem_ld_wait();
                        const uint32_t slot = peer_row + (uint32_t)(sp ^ 1) * kStripBytes;
#pragma unroll
                        for (int ch = 0; ch < 8; ++ch)
                            store_at_peer(slot + (((uint32_t)ch ^ swz) << 4), v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]);
                    }
                }
                __syncwarp();
                if (lane == 0) arrive_at_peer(peer_address(smem_u32(&c->peer_sent), peer));
                // This block's own strips: its sums, the other block's (received beside them), bias and residual.
                if (!wait_cluster(smem_u32(&c->peer_sent), (uint32_t)(it & 1), abort_flag)) give_up(c, status, 7, quarter);
                for (int j = group; j < half; j += 2) {
                    const int sp = (int)rank + 2 * j;
                    const uint32_t strip = row_u32 + (uint32_t)sp * kStripBytes, inbox = row_u32 + (uint32_t)(sp ^ 1) * kStripBytes;
                    const uint32_t b = bias_u32 + (uint32_t)(sp * kStripCols) * 4u;
                    uint32_t v[32];
                    tmem_ld32(t_row + (uint32_t)(sp * 32), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        const uint32_t off = ((uint32_t)ch ^ swz) << 4;
                        const float4 bb = lds4(b + 16 * ch), other = lds4(inbox + off);
                        float4 y;
                        y.x = (__uint_as_float(v[4 * ch]) + other.x) + bb.x;
                        y.y = (__uint_as_float(v[4 * ch + 1]) + other.y) + bb.y;
                        y.z = (__uint_as_float(v[4 * ch + 2]) + other.z) + bb.z;
                        y.w = (__uint_as_float(v[4 * ch + 3]) + other.w) + bb.w;
                        if constexpr (HAS_RES) {
                            const float4 r = lds4(strip + off);
                            y.x += r.x; y.y += r.y; y.z += r.z; y.w += r.w;
                        }
                        sts4(strip + off, y);
                    }
                    fence_async_shared();
                    named_barrier(2 + group, 128);
                    if (elected) {
                        if (n0 + sp * kStripCols < N) tma_store_2d(&map_out, staging + (size_t)sp * kStripBytes, n0 + sp * kStripCols, m0);
                        bulk_commit();
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&c->acc_empty[buf]);
                    arrive_at_peer(peer_address(smem_u32(&c->may_send), peer));      // what it sent has been read
                }
                if (elected) {
                    bulk_wait_read();
                    mbar_arrive(&c->staging_free);
                }
                if (tile + n_cta < total) named_barrier(1, kEpilogueThreads);
                continue;
            }
            for (int sp = group; sp < n_strips; sp += 2) {
                const uint32_t strip = row_u32 + (uint32_t)sp * kStripBytes;
                const uint32_t b = bias_u32 + (uint32_t)(sp * kStripCols) * 4u;
                // A strip of keys or values goes straight from the registers to its page, a strip of queries to `out`.
                bool to_cache = false;
                uint4* cache_row = nullptr;
                if constexpr (KV) {
                    const int col0 = n0 + sp * kStripCols;
                    to_cache = col0 >= kv.q_dim;
                    if (to_cache && slot >= 0 && col0 < N) {
                        const int kvd = kv.n_kv_head * kv.head_dim, rel = col0 - kv.q_dim;
                        const int which = rel >= kvd ? 1 : 0, within = rel - which * kvd;
                        const int head = within / kv.head_dim, dd = within - head * kv.head_dim;
                        const int page = slot >> kv.page_shift, off = slot & ((1 << kv.page_shift) - 1);
                        const size_t at = ((((size_t)page * 2 + which) * kv.n_kv_head + head) << kv.page_shift) + off;
                        cache_row = reinterpret_cast<uint4*>(kv.cache + at * kv.head_dim + dd);
                    }
                }
                if constexpr (sizeof(TO) == 4) {
                    uint32_t v[32];
                    tmem_ld32(t_row + (uint32_t)(sp * 32), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        const uint32_t at = strip + (((uint32_t)ch ^ swz) << 4);
                        const float4 bb = lds4(b + 16 * ch);
                        float4 y;
                        y.x = activate<ACT, false>(__uint_as_float(v[4 * ch]) + bb.x);
                        y.y = activate<ACT, false>(__uint_as_float(v[4 * ch + 1]) + bb.y);
                        y.z = activate<ACT, false>(__uint_as_float(v[4 * ch + 2]) + bb.z);
                        y.w = activate<ACT, false>(__uint_as_float(v[4 * ch + 3]) + bb.w);
                        if constexpr (HAS_RES) {
                            const float4 r = lds4(at);
                            y.x += r.x; y.y += r.y; y.z += r.z; y.w += r.w;
                        }
                        sts4(at, y);
                    }
                } else {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t v[32];
                        tmem_ld32(t_row + (uint32_t)(sp * 64 + half * 32), v);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int ch = half * 4 + q;
                            const float4 b0 = lds4(b + 128 * half + 32 * q), b1 = lds4(b + 128 * half + 32 * q + 16);
                            uint4 y;
                            y.x = pack2(activate<ACT, true>(__uint_as_float(v[8 * q]) + b0.x), activate<ACT, true>(__uint_as_float(v[8 * q + 1]) + b0.y));
                            y.y = pack2(activate<ACT, true>(__uint_as_float(v[8 * q + 2]) + b0.z), activate<ACT, true>(__uint_as_float(v[8 * q + 3]) + b0.w));
                            y.z = pack2(activate<ACT, true>(__uint_as_float(v[8 * q + 4]) + b1.x), activate<ACT, true>(__uint_as_float(v[8 * q + 5]) + b1.y));
                            y.w = pack2(activate<ACT, true>(__uint_as_float(v[8 * q + 6]) + b1.z), activate<ACT, true>(__uint_as_float(v[8 * q + 7]) + b1.w));
                            if (KV && to_cache) {
                                if (cache_row != nullptr) cache_row[ch] = y;
                            } else {
                                sts4(strip + (((uint32_t)ch ^ swz) << 4), y);
                            }
                        }
                    }
                }
                // The strip is complete once the group's four warps have written their rows: off it goes.
                fence_async_shared();
                named_barrier(2 + group, 128);
                if (elected) {
                    if (!to_cache && n0 + sp * kStripCols < N)
                        tma_store_2d(&map_out, staging + (size_t)sp * kStripBytes, n0 + sp * kStripCols, m0);
                    bulk_commit();
                }
            }
            // The accumulator has been read: the MMAs of the tile after next may overwrite it.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&c->acc_empty[buf]);
            if (et == 0 && it == 0) stamp(timing, 5);
            if (elected) {
                bulk_wait_read();                   // this group's stores have read the staging buffer
                mbar_arrive(&c->staging_free);
            }
            // Nobody writes the staging buffer or the bias again before both groups are done with this tile's.
            if (tile + n_cta < total) named_barrier(1, kEpilogueThreads);
        }
        if (elected) {
            bulk_wait_all();
            if (et == 0) stamp(timing, 6);
        }
    }
    __syncwarp();            // the elected lanes rejoin their warps before the block-wide barrier
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
    if constexpr (PAIR) {
        // Neither block leaves while the other may still reach into its shared memory (also after a wait ran out).
        asm volatile("barrier.cluster.arrive.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    }
}

size_t smem_bytes(int BN, int n_stages, int elem) {
    return 1024 + (size_t)n_stages * (kLaneTile + BN) * kBlockK * 2 + (size_t)kLaneTile * BN * elem + 256 * sizeof(float) +
           sizeof(Control);
}

int stages_for(int BN, int elem) {
    int n = 0;
    while (n < kMaxStages && smem_bytes(BN, n + 1, elem) <= kSmemLimit) ++n;
    return n;
}

// The feature tile whose rounds over the SMs cost least, and that cost in nanoseconds (0: none fits).  `pairs`: every
// tile is shared by two blocks with half of the k-blocks each (one round only: tiles x 2 blocks must fit the SMs).
int best_tile(int elem, int M, int N, int K, int n_sm, bool pairs, long* cost_out) {
    const int step = elem == 4 ? 32 : 64;
    const long m_tiles = (M + kLaneTile - 1) / kLaneTile;
    const long n_kb = (K + kBlockK - 1) / kBlockK;
    int best = 0;
    long best_cost = 0;
    for (int bn = 256; bn >= step; bn -= step) {
        if (stages_for(bn, elem) < 3) continue;
        if (bn > step && bn - step >= N) continue;                      // wider than the matrix by a whole strip
        const long tiles = m_tiles * ((N + bn - 1) / bn);
        long cost;
        if (pairs) {
            // Half the k-blocks, and about 2.5 us for the exchange: the first block's stores wait for the second's sums.
            if (tiles * 2 > n_sm || n_kb < 8 || (bn / step) % 2 != 0) continue;
            cost = (n_kb + 1) / 2 * (bn > 192 ? 420 : 300) + 1000 + 1000 * bn / 256 + 2500;
        } else {
            const long rounds = (tiles + n_sm - 1) / n_sm;
            cost = rounds * (n_kb * (bn > 192 ? 420 : 300) + 1000 + 1000 * bn / 256);
        }
        if (best == 0 || cost < best_cost) {
            best = bn;
            best_cost = cost;
        }
    }
    if (cost_out != nullptr) *cost_out = best_cost;
    return best;
}

}  // namespace

// Whether the persistent kernel takes the product, and with which feature tile.  It needs more than 64 tokens, TMA's
// 16-byte rule on every row stride and base, a residual only with float32 output; then it picks the tile width
// whose rounds over the SMs cost least.
extern "C" int lb_gemm_persistent_tile(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw,
                                       const float* residual, int64_t ldr, const void* out, int64_t ldo, int M, int N, int K) {
    const int elem = out_dtype == LB_F32 ? 4 : 2;
    if (M <= 64 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)A & 15) != 0 || ((uintptr_t)W & 15) != 0) return 0;
    if (((uintptr_t)out & 15) != 0 || (ldo * elem) % 16 != 0) return 0;
    if (residual != nullptr && (out_dtype != LB_F32 || ((uintptr_t)residual & 15) != 0 || (ldr * 4) % 16 != 0)) return 0;
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            n_sm = 148;
    }
    // Cost of a choice, in nanoseconds: rounds over the SMs x (k-blocks x time per k-block + epilogue).  Measured on
    // B200: a tcgen05.mma of 128 rows takes about as long for 32 columns as for 192 (the tensor core walks the rows),
    // so a k-block costs about 300 ns up to 192 columns and 420 ns at 256; the epilogue of a tile costs about a
    // microsecond plus one per 256 columns.  Ties go to the wider tile (fewer blocks fetch the same activations).
    return best_tile(elem, M, N, K, n_sm, false, nullptr);
}

// Whether lb_gemm_persistent can send the features from q_dim on to the pages of a cache instead of `out`.
extern "C" int lb_gemm_persistent_kv_supports(int out_dtype, int N, int act, int has_residual, int q_dim, int n_kv_head,
                                              int head_dim, int page_size) {
    return out_dtype == LB_BF16 && act == LB_ACT_NONE && !has_residual && q_dim > 0 && q_dim % 64 == 0 && head_dim > 0 &&
           head_dim % 64 == 0 && n_kv_head > 0 && N == q_dim + 2 * n_kv_head * head_dim && page_size > 0 &&
           (page_size & (page_size - 1)) == 0;
}

// Profiling aid: eight time stamps per block go to `buffer` (device memory, 8 * 148 64-bit words) on every launch
// from now on; null switches them off again.
extern "C" int lb_gemm_persistent_timing(unsigned long long* buffer) {
    g_timing = buffer;
    return LB_OK;
}

// LIYAB_B200_GEMM_PAIRS=0 in the environment keeps every tile with one block (measurements).
static bool pairs_enabled() {
    static const bool on = [] { const char* e = getenv("LIYAB_B200_GEMM_PAIRS"); return e == nullptr || e[0] != '0'; }();
    return on;
}

static int launch_persistent(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, const float* residual,
                             int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act, int bn, bool pair, const KvTarget& kv,
                             int n_sm, void* stream);

extern "C" int lb_gemm_persistent(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias,
                                  const float* residual, int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act,
                                  int feature_tile, void* kv_cache, const int32_t* slot_mapping, int q_dim, int n_kv_head,
                                  int head_dim, int page_size, void* stream) {
    LB_CHECK_ARG(M > 0 && N > 0 && K > 0, "gemm_persistent: bad sizes M=%d N=%d K=%d", M, N, K);
    KvTarget kv{static_cast<__nv_bfloat16*>(kv_cache), slot_mapping, q_dim, n_kv_head, head_dim, 0};
    if (kv_cache != nullptr) {
        if (!lb_gemm_persistent_kv_supports(out_dtype, N, act, residual != nullptr, q_dim, n_kv_head, head_dim, page_size))
            return lb_fail(LB_ERR_UNSUPPORTED,
                           "gemm_persistent: keys and values go to the cache only from a bfloat16 product without activation "
                           "or residual, with q_dim and head_dim multiples of 64 and a power-of-two page (N=%d q_dim=%d "
                           "kv_heads=%d head_dim=%d page_size=%d)", N, q_dim, n_kv_head, head_dim, page_size);
        LB_CHECK_ARG(slot_mapping != nullptr, "gemm_persistent: the slot mapping is missing");
        while ((1 << kv.page_shift) < page_size) ++kv.page_shift;
    }
    LB_CHECK_ARG(out_dtype == LB_BF16 || out_dtype == LB_F32, "gemm_persistent: unknown output dtype %d", out_dtype);
    LB_CHECK_ARG(lda >= K && ldw >= K && ldo >= N, "gemm_persistent: a row stride is shorter than the row");
    const int elem = out_dtype == LB_F32 ? 4 : 2;
    const int bn = feature_tile > 0 ? feature_tile : lb_gemm_persistent_tile(out_dtype, A, lda, W, ldw, residual, ldr, out, ldo, M, N, K);
    if (bn <= 0 || lb_gemm_persistent_tile(out_dtype, A, lda, W, ldw, residual, ldr, out, ldo, M, N, K) == 0)
        return lb_fail(LB_ERR_UNSUPPORTED,
                       "gemm_persistent: needs more than 64 tokens, K and all row strides on 16-byte boundaries, and float32 "
                       "output where a residual is given (M=%d K=%d lda=%lld ldw=%lld ldo=%lld ldr=%lld)",
                       M, K, (long long)lda, (long long)ldw, (long long)ldo, (long long)ldr);
    const int step = elem == 4 ? 32 : 64;
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        LB_CHECK_CUDA(cudaGetDevice(&dev));
        LB_CHECK_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
    }
    // Few tiles and a long reduction (float32 out, no activation): two blocks a tile, where the estimate says it pays.
    bool pair = false;
    int bn_used = bn;
    if (feature_tile <= 0 && elem == 4 && act == LB_ACT_NONE && kv_cache == nullptr && pairs_enabled()) {
        long single = 0, paired = 0;
        best_tile(elem, M, N, K, n_sm, false, &single);
        const int bn_pair = best_tile(elem, M, N, K, n_sm, true, &paired);
        if (bn_pair > 0 && paired < single) {
            pair = true;
            bn_used = bn_pair;
        }
    }
    LB_CHECK_ARG(bn % step == 0 && bn >= step && bn <= 256, "gemm_persistent: feature tile %d (a multiple of %d up to 256)", bn, step);
    return launch_persistent(out_dtype, A, lda, W, ldw, bias, residual, ldr, out, ldo, M, N, K, act, bn_used, pair, kv, n_sm, stream);
}

static int launch_persistent(int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, const float* bias, const float* residual,
                             int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int act, int bn, bool pair, const KvTarget& kv,
                             int n_sm, void* stream) {
    const int elem = out_dtype == LB_F32 ? 4 : 2;
    const void* kv_cache = kv.cache;
    const int n_stages = stages_for(bn, elem);
    LB_CHECK_ARG(n_stages >= 2, "gemm_persistent: feature tile %d leaves no room for two stages", bn);
    CUtensorMap map_a, map_w, map_res, map_out;
    int rc = lb_tensor_map_2d(&map_a, A, 2, M, K, lda, kLaneTile);
    if (rc == LB_OK) rc = lb_tensor_map_2d(&map_w, W, 2, N, K, ldw, bn);
    if (rc == LB_OK) rc = lb_tensor_map_2d(&map_out, out, elem, M, N, ldo, kLaneTile);
    if (rc == LB_OK) rc = residual != nullptr ? lb_tensor_map_2d(&map_res, residual, 4, M, N, ldr, kLaneTile) : LB_OK;
    if (rc != LB_OK) return rc;
    if (residual == nullptr) map_res = map_out;
    int* status = nullptr;
    rc = lb_tc_status_word(&status);
    if (rc != LB_OK) return rc;
    const long tiles = (long)((M + kLaneTile - 1) / kLaneTile) * ((N + bn - 1) / bn);
    const int grid = pair ? (int)(2 * tiles) : (int)(tiles < n_sm ? tiles : n_sm);
    // More than half of an SM's shared memory always, so that two blocks (each holding up to all of tensor memory)
    // never share an SM.
    size_t smem = smem_bytes(bn, n_stages, elem);
    if (smem < 120 * 1024) smem = 120 * 1024;
    auto s = static_cast<cudaStream_t>(stream);
#define LB_GO_KV(TO, ACT, RES, KV)                                                                                       \
    {                                                                                                                    \
        static bool configured = false;                                                                                  \
        if (!configured) {                                                                                               \
            LB_CHECK_CUDA(cudaFuncSetAttribute(gemm_persistent_kernel<TO, ACT, RES, KV>,                                 \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit));           \
            configured = true;                                                                                           \
        }                                                                                                                \
        LB_CHECK_CUDA(lb_launch_overlapped(gemm_persistent_kernel<TO, ACT, RES, KV>, dim3(grid), dim3(kThreads), smem, s, map_a, map_w, \
                                           map_res, map_out, bias, M, N, K, bn, n_stages, status, g_timing, kv));         \
    }
#define LB_GO(TO, ACT, RES) LB_GO_KV(TO, ACT, RES, false)
#define LB_GO_ACT(TO, RES)                                                  \
    switch (act) {                                                          \
        case LB_ACT_NONE: LB_GO(TO, LB_ACT_NONE, RES); break;               \
        case LB_ACT_GELU_TANH: LB_GO(TO, LB_ACT_GELU_TANH, RES); break;     \
        case LB_ACT_GELU_ERF: LB_GO(TO, LB_ACT_GELU_ERF, RES); break;       \
        default: return lb_fail(LB_ERR_INVALID_ARGUMENT, "gemm_persistent: unknown activation %d", act); \
    }
    if (pair) {
#define LB_GO_PAIR(RES)                                                                                                  \
    {                                                                                                                    \
        static bool configured = false;                                                                                  \
        if (!configured) {                                                                                               \
            LB_CHECK_CUDA(cudaFuncSetAttribute(gemm_persistent_kernel<float, LB_ACT_NONE, RES, false, true>,            \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit));           \
            configured = true;                                                                                           \
        }                                                                                                                \
        LB_CHECK_CUDA(lb_launch_overlapped_cluster(0, 2, gemm_persistent_kernel<float, LB_ACT_NONE, RES, false, true>, dim3(grid),        \
                                                   dim3(kThreads), smem, s, map_a, map_w, map_res, map_out, bias, M, N, K, bn, n_stages, \
                                                   status, g_timing, kv));                                               \
    }
        if (residual != nullptr) LB_GO_PAIR(true) else LB_GO_PAIR(false)
#undef LB_GO_PAIR
    } else if (elem == 4) {
        if (residual != nullptr) LB_GO_ACT(float, true) else LB_GO_ACT(float, false)
    } else if (kv_cache != nullptr) {
        LB_GO_KV(__nv_bfloat16, LB_ACT_NONE, false, true)
    } else {
        LB_GO_ACT(__nv_bfloat16, false)
    }
#undef LB_GO_ACT
#undef LB_GO
#undef LB_GO_KV
    LB_CHECK_LAUNCH();
    return LB_OK;
}
