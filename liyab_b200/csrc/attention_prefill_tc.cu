// Prefill attention for bfloat16 on the fifth-generation tensor cores (head size
// 64): the step's prompt portions (any lengths, cut anywhere) against their
// requests' paged keys and values.
//
// One block serves 128 consecutive query tokens of one request and one head and
// walks the keys the tile can see in tiles of 128 (eight runs of 16 keys, each
// inside one page):
//   warp 0      TMA producer.  The query tile comes from the activations through
//               one tensor map, key and value tiles from the cache through another
//               ([all rows of all pages][64]): lanes 0..7 fetch the eight 16-key
//               boxes of a key tile, lanes 8..15 those of the value tile, into a
//               ring of three stages.  A box past the last visible key is asked for
//               at an out-of-range row and arrives as zeros.
//   warp 1      issues tcgen05.mma: S = Q K^T (128 x 128, accumulator columns
//               0..127 of tensor memory) and O += P V (128 x 64, columns 128..191),
//               the scores of tile j+1 before the update of tile j.  V is used as it
//               lies in the cache ([key][dim], the "MN-major" operand form).
//   warps 2..17 softmax, four threads per query row (tensor-memory lane = row; warps
//               2..5 take the first 32 keys of a tile, warps 6..9 the next 32, and so
//               on; the parts' maxima meet in shared memory once per tile):
//               tcgen05.ld of the scores (two accumulators: the tensor core
//               computes the next tile's scores meanwhile), scale, causal/window
//               mask, running maximum, exp2, the probabilities as bfloat16 into one
//               of two buffers in shared memory in the swizzled K-major layout that
//               the second product reads, and the rescaling of O (tcgen05.ld /
//               tcgen05.st) when a maximum moved.
// Softmax, sums and both accumulators are 32-bit.  Every wait is bounded; a wait
// that runs out records a code in the device status word and the block drains
// its copies, frees tensor memory and returns.
//
// Reference formulas: scores, causal range, softmax and weighted values
// (src/core/transformer.cpp:2303-2313, 497-510, 2327-2341, 2344-2358).
#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"

#include <math_constants.h>

namespace {

using namespace lb_tc;

constexpr int kHD = 64;
constexpr int kBM = 128;              // query rows per block
constexpr int kBN = 128;              // keys per tile
constexpr int kStages = 3;
constexpr int kThreads = 576;
constexpr int kParts = 4;                   // threads per query row, each with 32 of a tile's 128 keys
constexpr int kSoftmaxThreads = 128 * kParts;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kTileBytes = 128 * 128;          // [128 rows][128 bytes]: Q, a K tile, a V tile, half of P
constexpr uint32_t kTmemCols = 512;    // scores twice (columns 0..127 and 128..255), output (256..319)
constexpr uint32_t kOCol = 256;

struct Control {
    uint64_t q_full;
    uint64_t kv_full[kStages];
    uint64_t kv_empty[kStages];
    uint64_t s_full[2];
    uint64_t s_free[2];
    uint64_t p_full[2];
    uint64_t p_free[2];
    uint64_t o_done;
    uint32_t tmem_base;
    int abort_flag;
    float row_max[2][kParts][kBM];        // [tile parity][key part][row]: the parts' maxima of a tile
    float row_sum[kParts][kBM];           // [key part][row]: the parts' sums at the end
};

__device__ __forceinline__ void give_up(Control* c, int* status, int site) {
    atomicCAS(status, 0, (0xA << 12) | site);
    c->abort_flag = 1;
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
          "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
// 2^x for x <= 0 or so: the hardware approximation alone (results below the normal range become zero).
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Descriptor of the value tile as the second operand in its MN-major form: rows of 64 dims (128 bytes, swizzled by
// TMA), eight keys to a 1024-byte group; both offset fields name that group stride.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(1024 >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor as umma_idesc, with the second operand MN-major (bit 16).
__host__ __device__ constexpr uint32_t umma_idesc_b_mn(int m, int n) { return umma_idesc(m, n) | (1u << 16); }

__global__ void __launch_bounds__(kThreads)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const int32_t* __restrict__ q_start, const int32_t* __restrict__ n_past,
                            const int32_t* __restrict__ block_table, int table_stride, __nv_bfloat16* __restrict__ out,
                            int64_t out_stride, int n_head, int n_kv_head, int page_shift, int kv_rows, float scale, int window,
                            int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    lb_wait_for_predecessor();            // queries, keys and values come from the kernel before this one
    lb_dependents_may_launch();
    uint8_t* q_s = base;                                   // 16 KB
    uint8_t* k_s = q_s + kTileBytes;                       // [kStages] 16 KB
    uint8_t* v_s = k_s + kStages * kTileBytes;             // [kStages] 16 KB
    uint8_t* p_s = v_s + kStages * kTileBytes;             // [2 buffers][2 key halves] 16 KB
    Control* c = reinterpret_cast<Control*>(p_s + 4 * kTileBytes);
    volatile int* abort_flag = &c->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The last query tiles of a request see the most keys: blocks are numbered so that all of those start first.
    const int head = blockIdx.x % n_head, seq = blockIdx.x / n_head, tile_q = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int row0 = q_start[seq], q_len = q_start[seq + 1] - row0;
    if (tile_q * kBM >= q_len) return;
    const int past = n_past[seq];
    const int kvh = head / (n_head / n_kv_head);
    const int page_size = 1 << page_shift;
    const int rows_here = min(kBM, q_len - tile_q * kBM);
    const int p_min = past + tile_q * kBM, p_max = p_min + rows_here - 1;
    const int kv_lo = (window > 0 ? max(0, p_min - window + 1) : 0) / kBN * kBN;
    const int n_tiles = (p_max - kv_lo) / kBN + 1;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_kv);
        mbar_init(&c->q_full, 1);
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&c->kv_full[i], 1);
            mbar_init(&c->kv_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&c->s_full[i], 1);
            mbar_init(&c->s_free[i], kSoftmaxThreads / 32);      // one arrival per softmax warp
            mbar_init(&c->p_full[i], kSoftmaxThreads / 32);
            mbar_init(&c->p_free[i], 1);
        }
        mbar_init(&c->o_done, 1);
        c->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(&c->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = c->tmem_base;

    if (warp == 0) {
        // ---- producer: Q once, then the key and value tiles through the ring.
        if (lane == 0) {
            mbar_expect_tx(&c->q_full, kTileBytes);
            tma_load_2d(q_s, &map_q, &c->q_full, head * kHD, row0 + tile_q * kBM);
        }
        const int32_t* table = block_table + (size_t)seq * table_stride;
        int issued = 0;
        for (int tile = 0; tile < n_tiles; ++tile) {
            const int st = tile % kStages;
            const uint32_t ph = (tile / kStages) & 1;
            bool ok = true;
            if (lane == 0) ok = mbar_wait(&c->kv_empty[st], ph ^ 1, abort_flag);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) {
                if (lane == 0) give_up(c, status, 1);
                break;
            }
            if (lane == 0) mbar_expect_tx(&c->kv_full[st], 2 * kTileBytes);
            __syncwarp();
            if (lane < 16) {
                const int sub = lane & 7, kv = lane >> 3;              // lanes 0..7: keys, 8..15: values
                const int j0 = kv_lo + tile * kBN + sub * 16;
                int row = kv_rows;                                      // out of range: the box arrives as zeros
                if (j0 <= p_max) {
                    const int page = table[j0 >> page_shift];
                    if (page >= 0) row = ((page * 2 + kv) * n_kv_head + kvh) * page_size + (j0 & (page_size - 1));
                }
                uint8_t* dst = (kv == 0 ? k_s : v_s) + (size_t)st * kTileBytes + sub * 2048;
                tma_load_2d(dst, &map_kv, &c->kv_full[st], 0, row);
            }
            issued = tile + 1;
        }
        if (*abort_flag != 0 && lane == 0) {
            // Leave no copy in flight: the barriers of the last loads issued complete when their bytes landed.
            mbar_wait(&c->q_full, 0, nullptr);
            if (issued > 0) mbar_wait(&c->kv_full[(issued - 1) % kStages], ((issued - 1) / kStages) & 1, nullptr);
        }
    } else if (warp == 1) {
        // ---- products: scores of tile j + 1 before the update of tile j.
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(kBM, kBN);
            constexpr uint32_t idesc_o = umma_idesc_b_mn(kBM, kHD);
            const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
            // Descriptors are made once per operand tile and moved by addition (the start address sits in the low bits
            // in units of 16 bytes, and no tile crosses the field's range): this thread's instructions between two
            // products are what the softmax threads wait for.
            const uint64_t dq = umma_desc(q_addr);
            bool ok = mbar_wait(&c->q_full, 0, abort_flag);
            if (!ok) give_up(c, status, 2);
            auto scores = [&](int tile) -> bool {
                const int st = tile % kStages;
                if (!mbar_wait(&c->kv_full[st], (tile / kStages) & 1, abort_flag)) { give_up(c, status, 3); return false; }
                const int sb = tile & 1;
                if (!mbar_wait(&c->s_free[sb], ((tile >> 1) & 1) ^ 1, abort_flag)) { give_up(c, status, 4); return false; }
                tc_fence_after();
                const uint64_t dk = umma_desc(smem_u32(k_s + (size_t)st * kTileBytes));
#pragma unroll
                for (int kk = 0; kk < kHD / kUmmaK; ++kk)
                    umma_bf16(tmem_base + sb * kBN, dq + (uint64_t)(kk * 2), dk + (uint64_t)(kk * 2), idesc_s, kk != 0 ? 1u : 0u);
                umma_commit(&c->s_full[sb]);
                return true;
            };
            if (ok) ok = scores(0);
            for (int tile = 0; tile < n_tiles && ok; ++tile) {
                // Two accumulators for scores: the next tile's are computed while the softmax threads work on this one's.
                if (tile + 1 < n_tiles) ok = scores(tile + 1);
                if (!ok) break;
                const int pb = tile & 1;
                if (!mbar_wait(&c->p_full[pb], (tile >> 1) & 1, abort_flag)) { give_up(c, status, 5); break; }
                tc_fence_after();
                const int st = tile % kStages;
                const uint64_t dp = umma_desc(p_addr + pb * 2 * kTileBytes);
                const uint64_t dv = umma_desc_mn(smem_u32(v_s + (size_t)st * kTileBytes));
#pragma unroll
                for (int ks = 0; ks < kBN / kUmmaK; ++ks) {
                    // P: key half ks / 4 (its own 16 KB tile), 32 bytes per 16 keys within it; V: 16 keys = 2048 bytes.
                    const uint64_t da = dp + (uint64_t)(((ks >> 2) * kTileBytes + (ks & 3) * 32) >> 4);
                    const uint64_t db = dv + (uint64_t)((ks * 2048) >> 4);
                    umma_bf16(tmem_base + kOCol, da, db, idesc_o, (tile | ks) != 0 ? 1u : 0u);
                }
                umma_commit(&c->kv_empty[st]);      // keys and values of the stage have been read
                umma_commit(&c->p_free[pb]);        // and this buffer of probabilities
                umma_commit(&c->o_done);            // O holds tile `tile`
            }
        }
    } else {
        // ---- softmax: four threads per query row (warps 2..5 take the first 32 keys of every tile, warps 6..9 the
        // next 32, and so on; all see tensor-memory lanes 32 * (warp % 4) .. + 31).  Four warps per scheduler: with
        // two, every instruction's latency showed (0.45 instructions a clock).
        const int quarter = warp & 3, part = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;                              // row of the tile = lane of tensor memory
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int pos = past + tile_q * kBM + min(r, rows_here - 1);    // rows past the end copy the last one; not stored
        const int first = window > 0 ? pos - window + 1 : 0;
        const float sc = scale * kLog2e;
        const uint32_t swz = (uint32_t)(r & 7);
        uint8_t* p_row = p_s + (size_t)r * 128;
        float m = -CUDART_INF_F, l = 0.0f;                              // l: this thread's part of the row's sum
        bool ok = true;
        for (int tile = 0; tile < n_tiles; ++tile) {
            const int sb = tile & 1, pb = tile & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(&c->s_full[sb], (tile >> 1) & 1, abort_flag));      // one answer for the warp
            if (!ok) give_up(c, status, 6);
            tc_fence_after();
            const int j0 = kv_lo + tile * kBN + part * 32;             // this thread's first key of the tile
            const bool need_mask = (j0 + 31 > p_min) || (window > 0 && j0 < p_max - window + 1);
            const uint32_t s_row = t_row + (uint32_t)(sb * kBN + part * 32);
            // First pass: the maximum of this part of the row; the parts meet in shared memory.
            float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F, mx2 = -CUDART_INF_F, mx3 = -CUDART_INF_F;
            uint32_t v[32];
            if (ok) {
                tmem_ld32(s_row, v);
                tmem_ld_wait();
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (j0 + i > pos || j0 + i < first) v[i] = __float_as_uint(-CUDART_INF_F);
                }
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    mx0 = fmaxf(mx0, __uint_as_float(v[i]));
                    mx1 = fmaxf(mx1, __uint_as_float(v[i + 1]));
                    mx2 = fmaxf(mx2, __uint_as_float(v[i + 2]));
                    mx3 = fmaxf(mx3, __uint_as_float(v[i + 3]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0u;
            }
            c->row_max[tile & 1][part][r] = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            named_barrier(1, kSoftmaxThreads);              // reached by all softmax threads, also after a wait ran out
            if (*abort_flag != 0) break;
            float mx = c->row_max[tile & 1][0][r];
#pragma unroll
            for (int q = 1; q < kParts; ++q) mx = fmaxf(mx, c->row_max[tile & 1][q][r]);
            const float m_new = fmaxf(m, mx * sc);
            const float base_m = m_new == -CUDART_INF_F ? 0.0f : m_new;
            const float corr = exp2f(m - base_m);
            // This buffer of probabilities was last read by the update of the tile before last.
            if (tile >= 2) {
                ok = __all_sync(0xffffffffu, mbar_wait(&c->p_free[pb], ((tile >> 1) - 1) & 1, abort_flag));
                if (!ok) { give_up(c, status, 7); break; }
            }
            // Second pass, on the scores still in registers (masked ones are -inf: weight 0): probabilities -> shared
            // memory (bfloat16, swizzled), and their sum.  One multiply-add and one MUFU per score: the SM's
            // exponential unit (16 results a clock) and its issue slots, not the tensor core, set this kernel's pace.
            float sum0 = 0.0f, sum1 = 0.0f;
            uint8_t* half_row = p_row + (size_t)(pb * 2 + (part >> 1)) * kTileBytes;
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
                float p[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) p[i] = ex2_approx(fmaf(__uint_as_float(v[q8 * 8 + i]), sc, -base_m));
                sum0 += (p[0] + p[1]) + (p[2] + p[3]);
                sum1 += (p[4] + p[5]) + (p[6] + p[7]);
                uint4 pk;
                pk.x = pack2(p[0], p[1]);
                pk.y = pack2(p[2], p[3]);
                pk.z = pack2(p[4], p[5]);
                pk.w = pack2(p[6], p[7]);
                const uint32_t chunk = (uint32_t)((part & 1) * 4 + q8);                // 16-byte chunk within the 64-key half
                *reinterpret_cast<uint4*>(half_row + ((chunk ^ swz) << 4)) = pk;
            }
            // The scores have been read: the tile after next may overwrite them.
            // (One lane arrives for its warp: hundreds of arrivals on one barrier word would queue up behind one another.)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&c->s_free[sb]);
            l = l * corr + (sum0 + sum1);
            m = m_new;
            // O *= corr where some row of the warp moved its maximum (never for the first tile: O is overwritten);
            // the update of the tile before must be complete for that.  Each part rescales 16 of the 64 columns.
            if (tile > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait(&c->o_done, (tile - 1) & 1, abort_flag));
                if (!ok) { give_up(c, status, 8); break; }
                tc_fence_after();
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
                    uint32_t o[16];
                    tmem_ld16(t_row + kOCol + part * 16, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    tmem_st16(t_row + kOCol + part * 16, o);
                    tmem_st_wait();
                }
            }
            // A 16-key box that straddles the last visible key brings rows of later positions with it: whatever the
            // cache holds there (it may be anything, also NaN) would meet its zero weight in the second product.
            // Those value rows (fewer than 16, in the last tile only) are zeroed here, after the tile has landed.
            const int t0 = kv_lo + tile * kBN;
            if (part == 0 && t0 + kBN - 1 > p_max) {
                ok = __all_sync(0xffffffffu, mbar_wait(&c->kv_full[tile % kStages], (tile / kStages) & 1, abort_flag));
                if (!ok) { give_up(c, status, 9); break; }
                const int last = p_max - t0;                        // last visible row of the tile
                if (r > last && r < (last / 16 + 1) * 16) {
                    uint4* row = reinterpret_cast<uint4*>(v_s + (size_t)(tile % kStages) * kTileBytes + (size_t)r * 128);
#pragma unroll
                    for (int i = 0; i < 8; ++i) row[i] = make_uint4(0, 0, 0, 0);
                }
            }
            tc_fence_before();
            fence_async_shared();                   // P (and those rows), written through the generic proxy, are read by the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&c->p_full[pb]);
        }
        // The parts' sums meet, then each part normalises and stores 16 of the row's 64 values.
        c->row_sum[part][r] = l;
        named_barrier(1, kSoftmaxThreads);
        if (*abort_flag == 0) {
            ok = __all_sync(0xffffffffu, mbar_wait(&c->o_done, (n_tiles - 1) & 1, abort_flag));
            if (!ok) give_up(c, status, 10);
        } else {
            ok = false;
        }
        if (ok) {
            tc_fence_after();
            float total = c->row_sum[0][r];
#pragma unroll
            for (int q = 1; q < kParts; ++q) total += c->row_sum[q][r];
            const float inv = 1.0f / total;
            __nv_bfloat16* dst = out + (size_t)(row0 + tile_q * kBM + r) * out_stride + (size_t)head * kHD + part * 16;
            uint32_t o[16];
            tmem_ld16(t_row + kOCol + part * 16, o);
            tmem_ld_wait();
            if (r < rows_here) {
#pragma unroll
                for (int q8 = 0; q8 < 2; ++q8) {
                    uint4 pk;
                    pk.x = pack2(__uint_as_float(o[q8 * 8]) * inv, __uint_as_float(o[q8 * 8 + 1]) * inv);
                    pk.y = pack2(__uint_as_float(o[q8 * 8 + 2]) * inv, __uint_as_float(o[q8 * 8 + 3]) * inv);
                    pk.z = pack2(__uint_as_float(o[q8 * 8 + 4]) * inv, __uint_as_float(o[q8 * 8 + 5]) * inv);
                    pk.w = pack2(__uint_as_float(o[q8 * 8 + 6]) * inv, __uint_as_float(o[q8 * 8 + 7]) * inv);
                    *reinterpret_cast<uint4*>(dst + q8 * 8) = pk;
                }
            }
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

// Whether the tcgen05 prefill kernel takes the shape: head size 64, pages of 16 positions or more (a power of two).
extern "C" int lb_prefill_attention_tc_supports(int n_head, int n_kv_head, int head_dim, int page_size) {
    return n_kv_head > 0 && n_head % n_kv_head == 0 && head_dim == kHD && page_size >= 16 && (page_size & (page_size - 1)) == 0;
}

extern "C" int lb_prefill_attention_tc(const void* q, int64_t q_stride, int n_tokens, const void* cache, int n_pages,
                                       const int32_t* q_start, const int32_t* n_past, const int32_t* block_table,
                                       int table_stride, void* out, int64_t out_stride, int n_seq, int max_q_len, int n_head,
                                       int n_kv_head, int head_dim, int page_size, float scale, int window, void* stream) {
    LB_CHECK_ARG(n_seq >= 0 && max_q_len >= 0 && n_tokens >= 0 && n_pages > 0, "prefill attention: bad sizes");
    if (!lb_prefill_attention_tc_supports(n_head, n_kv_head, head_dim, page_size))
        return lb_fail(LB_ERR_UNSUPPORTED, "prefill attention (tcgen05): unsupported shape heads %d/%d head_dim %d page_size %d",
                       n_head, n_kv_head, head_dim, page_size);
    LB_CHECK_ARG(q_stride % 8 == 0 && out_stride % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                     ((uintptr_t)cache & 15) == 0,
                 "prefill attention (tcgen05): q, out and cache rows must be 16-byte aligned");
    LB_CHECK_ARG((max_q_len + kBM - 1) / kBM <= 65535, "prefill attention: a portion of %d tokens is too long for one launch", max_q_len);
    const long long kv_rows = (long long)n_pages * 2 * n_kv_head * page_size;
    LB_CHECK_ARG(kv_rows < (1ll << 31), "prefill attention (tcgen05): the cache has too many rows for one tensor map");
    if (n_seq == 0 || max_q_len == 0 || n_tokens == 0) return LB_OK;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    CUtensorMap map_q, map_kv;
    int rc = lb_tensor_map_2d(&map_q, q, 2, n_tokens, n_head * kHD, q_stride, kBM);
    if (rc == LB_OK) rc = lb_tensor_map_2d(&map_kv, cache, 2, (int)kv_rows, kHD, kHD, 16);
    if (rc != LB_OK) return rc;
    int* status = nullptr;
    rc = lb_tc_status_word(&status);
    if (rc != LB_OK) return rc;
    constexpr size_t smem = 1024 + (size_t)(1 + 2 * kStages + 4) * kTileBytes + sizeof(Control);
    static bool configured = false;
    if (!configured) {
        LB_CHECK_CUDA(cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    dim3 grid(n_head * n_seq, (max_q_len + kBM - 1) / kBM);
    LB_CHECK_CUDA(lb_launch_overlapped(prefill_attention_tc_kernel, dim3(grid), dim3(kThreads), smem, static_cast<cudaStream_t>(stream), 
        map_q, map_kv, q_start, n_past, block_table, table_stride, (__nv_bfloat16*)out, out_stride, n_head, n_kv_head, page_shift,
        (int)kv_rows, scale, window, status));
    LB_CHECK_LAUNCH();
    return LB_OK;
}
