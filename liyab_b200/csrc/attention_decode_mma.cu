// Decode attention for bfloat16 with the products on the tensor cores: one new
// token per request against its paged keys and values, head sizes 64 and 128.
//
// The scalar decode kernel (attention_decode.cu) spends about 150 thread
// instructions per key and head and is bound by instruction issue at half the
// memory roofline.  Here the query heads that share a key/value head (1 to 16 of
// them) are the rows of a 16-row tile, keys come 16 at a time, and scores
// S = Q K^T and the update O += P V are mma.sync m16n8k16 products with 32-bit
// accumulators: a dozen tensor instructions replace a thousand scalar ones, and
// the kernel goes back to being bound by the bytes of the cache.
//
// One block serves (key range, key/value head, request), as in the scalar
// kernel and with the same split of the keys.  Each of its warps (four, or two
// where that fills the GPU's last wave of blocks better) takes every n-th 16-key
// tile of the range (a tile lies inside one page: its keys, and its values, are
// one contiguous run of the cache), brings it into its own two shared-memory
// buffers with cp.async one tile ahead (16-byte chunks XOR-swizzled by the row, so
// ldmatrix meets no bank twice and nothing is padded), and keeps its own running
// maximum, sum and output; the warps are merged at the end in warp order, the key
// ranges in range order: two to eight ranges are the blocks of one cluster and
// meet in its first block's shared memory (the launch carries the cluster size),
// more than eight go through global memory to the block that finishes last.  Softmax, sums and
// accumulators are 32-bit (exp2 of scores pre-scaled by log2 e).  Measured on
// B200, 12 heads of 64 over 768 keys: 27 us for 64 requests and 51 us for 128
// (5.5 and 5.9 TB/s of cache), where the scalar kernel takes 47 us for 64.
//
// Reference formulas: src/core/transformer.cpp:2303-2313, 2327-2341, 2344-2358, 2367-2385.
#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"

#include <math_constants.h>

namespace {

constexpr int kTile = 16;            // keys per tile
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16 bytes global -> shared; when `valid` is false nothing is read and the destination is filled with zeros.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// TMA: the tiles come as tensor-map boxes of 16 keys (head size 64: a row is the 128 bytes of the swizzle) instead
// of 16-byte cp.async pieces: two instructions per tile from one lane, completion on a per-warp mbarrier.
template <int HD, int kWarps, int kStages, bool TMA>
__global__ void __launch_bounds__(kWarps * 32)
decode_attention_mma_kernel(const __grid_constant__ CUtensorMap map_kv, int kv_rows, int* status,
                            const __nv_bfloat16* __restrict__ q, int64_t q_stride, const __nv_bfloat16* __restrict__ cache,
                            const int32_t* __restrict__ positions, const int32_t* __restrict__ block_table, int table_stride,
                            __nv_bfloat16* __restrict__ out, int64_t out_stride, float* __restrict__ partial,
                            int* __restrict__ counters, int n_head, int n_kv_head, int page_shift, float scale, int window,
                            int n_splits, int cluster_merge) {
    constexpr int kThreads = kWarps * 32;
    constexpr int LD = HD;                      // a tile's row in shared memory; its 16-byte chunks are XOR-swizzled by the row
    constexpr int CH = HD / 8;                  // 16-byte chunks per row
    constexpr int KS = HD / 16;                 // k-steps of Q K^T
    constexpr int OT = HD / 8;                  // output n-tiles
    constexpr int STATE = HD + 2;               // m, l, values of one query head
    // Dynamic shared memory: the warps' tile buffers [warp][stage][K|V][16 x LD]; once the key loop is over the
    // same bytes hold the warps' states per query row, red[warp][row][STATE].
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // TMA's swizzle counts rows from 1024-byte boundaries.
    uint8_t* smem_bytes = TMA ? reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023) : smem_raw;
    __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem_bytes);
    float* red = reinterpret_cast<float*>(smem_bytes);
    __shared__ int is_last;
    __shared__ uint64_t bars[kWarps][kStages];

    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    // Every block of the cluster has started before one of them writes into another's shared memory: arrive now, wait
    // just before those writes.
    if (cluster_merge) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int G = n_head / n_kv_head;           // query heads of this key/value head: the tile's valid rows
    const int page_size = 1 << page_shift;
    const size_t plane = (size_t)n_kv_head * page_size * HD;
    const int pos = positions[seq];
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_keys = pos + 1 - first;
    const int chunk = (n_keys + n_splits - 1) / n_splits;
    const int begin = first + split * chunk, end = min(pos + 1, begin + chunk);
    const int32_t* table = block_table + (size_t)seq * table_stride;
    const int tile0 = begin / kTile;                                                // first tile of the range
    const int n_tiles = end > begin ? (end - 1) / kTile + 1 - tile0 : 0;

    // Q as the A operand: row r = query head kvh * G + r (rows past G are zero).  Filled after the wait below.
    uint32_t qf[KS][4];
    auto load_queries = [&]() {
        const __nv_bfloat16* q_seq = q + (size_t)seq * q_stride + (size_t)kvh * G * HD;
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            const int c = kk * 16 + 2 * t;
            qf[kk][0] = g < G ? *reinterpret_cast<const uint32_t*>(q_seq + (size_t)g * HD + c) : 0u;
            qf[kk][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(q_seq + (size_t)(g + 8) * HD + c) : 0u;
            qf[kk][2] = g < G ? *reinterpret_cast<const uint32_t*>(q_seq + (size_t)g * HD + c + 8) : 0u;
            qf[kk][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(q_seq + (size_t)(g + 8) * HD + c + 8) : 0u;
        }
    };
    const int my_tiles = n_tiles > warp ? (n_tiles - warp + kWarps - 1) / kWarps : 0;
    // This warp's i-th tile (tile index tile0 + warp + kWarps i) -> stage.  Rows outside [begin, end) are not read
    // and arrive as zeros: their scores are masked, and a zero weight times whatever the cache holds there (it
    // may be anything, also NaN) must not reach the output.  Chunk c of row r lies at chunk c ^ (r & 7), which
    // keeps the eight rows of an ldmatrix on different banks without padding.  The page numbers of 32 tiles are
    // read at once, one per lane, so that no tile waits for its table entry.
    int page_reg = 0;
    auto load_tile = [&](int i, int stage) {
        if ((i & 31) == 0) {
            const int mine = tile0 + warp + kWarps * (i + lane);
            page_reg = i + lane < my_tiles ? table[(mine * kTile) >> page_shift] : 0;
        }
        const int page = __shfl_sync(0xffffffffu, page_reg, i & 31);
        const int j0 = (tile0 + warp + kWarps * i) * kTile;
        const __nv_bfloat16* src = cache + (size_t)page * 2 * plane + ((size_t)kvh * page_size + (j0 & (page_size - 1))) * HD;
        __nv_bfloat16* kd = tiles + (size_t)((warp * kStages + stage) * 2) * kTile * LD;
        __nv_bfloat16* vd = kd + kTile * LD;
        if constexpr (TMA) {
            // Rows of the cache as the tensor map counts them: ((page * 2 + K|V) * kv_heads + head) * page_size + slot.
            if (lane == 0) {
                const int row_k = ((page * 2) * n_kv_head + kvh) * page_size + (j0 & (page_size - 1));
                const int row_v = row_k + n_kv_head * page_size;
                lb_tc::fence_async_shared();              // the lanes' reads of the stage (ordered before by __syncwarp)
                lb_tc::mbar_expect_tx(&bars[warp][stage], 2 * kTile * HD * sizeof(__nv_bfloat16));
                lb_tc::tma_load_2d(kd, &map_kv, &bars[warp][stage], 0, row_k);
                lb_tc::tma_load_2d(vd, &map_kv, &bars[warp][stage], 0, row_v);
            }
            return;
        }
#pragma unroll
        for (int c = lane; c < kTile * CH; c += 32) {
            const int r = c / CH, ch = c - r * CH;
            const bool valid = j0 + r >= begin && j0 + r < end;
            const int at = r * LD + ((ch ^ (r & 7)) << 3);
            cp_async16(kd + at, src + r * HD + ch * 8, valid);
            cp_async16(vd + at, src + plane + r * HD + ch * 8, valid);
        }
    };

    float o[OT][4];
#pragma unroll
    for (int i = 0; i < OT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_lo = -CUDART_INF_F, m_hi = -CUDART_INF_F, l_lo = 0.0f, l_hi = 0.0f;
    const float sc = scale * kLog2e;

    if constexpr (TMA) {
        if (lane == 0) {
            for (int i = 0; i < kStages; ++i) lb_tc::mbar_init(&bars[warp][i], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
    }
    int gave_up_at = -1;
    // Positions and block table came from the host before any kernel of the step, and keys and values of earlier
    // positions from earlier steps: the first tiles travel before this kernel waits for the one before it, all but
    // a tile that holds the request's newest position, which that kernel writes (TMA tiles only: the other path counts
    // its copies in groups, in order).  Queries come from that kernel too.
    const int newest_tile = pos / kTile;
    bool held_back[kStages - 1 > 0 ? kStages - 1 : 1];
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {          // kStages - 1 tiles ahead; a group per tile, empty past the end
        held_back[i] = !TMA || tile0 + warp + kWarps * i == newest_tile;
        if (i < my_tiles && !held_back[i]) load_tile(i, i);
    }
    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    load_queries();
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {
        if (i < my_tiles && held_back[i]) load_tile(i, i);
        cp_async_commit();
    }
    for (int i = 0; i < my_tiles; ++i) {
        const int stage = i % kStages;
        if (i + kStages - 1 < my_tiles) load_tile(i + kStages - 1, (i + kStages - 1) % kStages);
        if constexpr (TMA) {
            // Bounded; one answer for the warp.  A wait that ran out ends the warp's walk (its result is then wrong
            // and the status word says so).
            if (!__all_sync(0xffffffffu, lb_tc::mbar_wait(&bars[warp][stage], (uint32_t)(i / kStages) & 1u, nullptr))) {
                if (lane == 0) atomicCAS(status, 0, (0xD << 12) | 1);
                gave_up_at = i;
                break;
            }
            // Rows outside the range came with the box: values there (whatever the page holds, also NaN) would
            // meet a zero weight.  Zeroed here, in the tiles of the range's two ends only.
            const int j0z = (tile0 + warp + kWarps * i) * kTile;
            if (j0z < begin || j0z + kTile > end) {
                __nv_bfloat16* vz = tiles + (size_t)((warp * kStages + stage) * 2) * kTile * LD + kTile * LD;
                for (int c = lane; c < kTile * CH; c += 32) {
                    const int r = c / CH;
                    if (j0z + r < begin || j0z + r >= end) *reinterpret_cast<uint4*>(vz + r * LD + (c - r * CH) * 8) = make_uint4(0, 0, 0, 0);
                }
            }
        } else {
            cp_async_commit();
            cp_async_wait<kStages - 1>();
        }
        __syncwarp();
        const __nv_bfloat16* kt = tiles + (size_t)((warp * kStages + stage) * 2) * kTile * LD;
        const __nv_bfloat16* vt = kt + kTile * LD;
        const int j0 = (tile0 + warp + kWarps * i) * kTile;
        // S = Q K^T: 16 rows x 16 keys.
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const int mat = lane >> 3, r8 = lane & 7;
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            uint32_t b[4];
            ldmatrix_x4(b, smem_addr(kt + ((mat >> 1) * 8 + r8) * LD + (((kk * 2 + (mat & 1)) ^ r8) << 3)));
            mma_bf16(s[0], qf[kk], b[0], b[1]);
            mma_bf16(s[1], qf[kk], b[2], b[3]);
        }
        float mx_lo = -CUDART_INF_F, mx_hi = -CUDART_INF_F;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + nt * 8 + 2 * t + (e & 1);
                s[nt][e] = (j >= begin && j < end) ? s[nt][e] * sc : -CUDART_INF_F;
            }
            mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
            mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float base_lo = mn_lo == -CUDART_INF_F ? 0.0f : mn_lo, base_hi = mn_hi == -CUDART_INF_F ? 0.0f : mn_hi;
        const float corr_lo = exp2f(m_lo - base_lo), corr_hi = exp2f(m_hi - base_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        uint32_t pf[4];
        float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const float p0 = exp2f(s[nt][0] - base_lo), p1 = exp2f(s[nt][1] - base_lo);
            const float p2 = exp2f(s[nt][2] - base_hi), p3 = exp2f(s[nt][3] - base_hi);
            sum_lo += p0 + p1;
            sum_hi += p2 + p3;
            pf[nt * 2] = pack_bf16(p0, p1);
            pf[nt * 2 + 1] = pack_bf16(p2, p3);
        }
        l_lo = l_lo * corr_lo + sum_lo;          // per-thread partial sums; the quad is summed once at the end
        l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
        for (int ot = 0; ot < OT; ot += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, smem_addr(vt + ((mat & 1) * 8 + r8) * LD + (((ot + (mat >> 1)) ^ r8) << 3)));
            o[ot][0] *= corr_lo; o[ot][1] *= corr_lo; o[ot][2] *= corr_hi; o[ot][3] *= corr_hi;
            o[ot + 1][0] *= corr_lo; o[ot + 1][1] *= corr_lo; o[ot + 1][2] *= corr_hi; o[ot + 1][3] *= corr_hi;
            mma_bf16(o[ot], pf, b[0], b[1]);
            mma_bf16(o[ot + 1], pf, b[2], b[3]);
        }
        __syncwarp();        // the stage is overwritten by the load issued in the next trip
    }
    cp_async_wait<0>();
    if constexpr (TMA) {
        // After a wait that ran out the copies still in flight land before the block may leave (bounded as well).
        if (gave_up_at >= 0)
            for (int t2 = gave_up_at; t2 < my_tiles && t2 < gave_up_at + kStages; ++t2)
                lb_tc::mbar_wait(&bars[warp][t2 % kStages], (uint32_t)(t2 / kStages) & 1u, nullptr);
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    // The warps' states of every valid row -> shared memory (over the tile buffers) -> merged in warp order.
    __syncthreads();
    if (g < G) {
        float* st = red + (size_t)(warp * 16 + g) * STATE;
        if (t == 0) { st[0] = m_lo; st[1] = l_lo; }
#pragma unroll
        for (int ot = 0; ot < OT; ++ot) { st[2 + ot * 8 + 2 * t] = o[ot][0]; st[2 + ot * 8 + 2 * t + 1] = o[ot][1]; }
    }
    if (g + 8 < G) {
        float* st = red + (size_t)(warp * 16 + g + 8) * STATE;
        if (t == 0) { st[0] = m_hi; st[1] = l_hi; }
#pragma unroll
        for (int ot = 0; ot < OT; ++ot) { st[2 + ot * 8 + 2 * t] = o[ot][2]; st[2 + ot * 8 + 2 * t + 1] = o[ot][3]; }
    }
    __syncthreads();
    float* my_partial = partial + (((size_t)seq * n_kv_head + kvh) * n_splits + split) * (size_t)(G * STATE);
    // With the key ranges of a request and head as the blocks of one cluster, their states meet in the first block's
    // shared memory (an inbox past the tile buffers, one slot per range) instead of global memory.
    constexpr size_t kRegion = ((size_t)kWarps * kStages * 2 * kTile * HD * sizeof(__nv_bfloat16) > (size_t)kWarps * 16 * STATE * sizeof(float)
                                    ? (size_t)kWarps * kStages * 2 * kTile * HD * sizeof(__nv_bfloat16)
                                    : (size_t)kWarps * 16 * STATE * sizeof(float)) + (TMA ? 1024 : 0);
    uint32_t first_block = 0;
    if (cluster_merge) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    if (cluster_merge && n_splits > 1)
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                     : "=r"(first_block) : "r"(smem_addr(reinterpret_cast<float*>(smem_raw + kRegion) + (size_t)split * G * STATE)), "r"(0));
    for (int idx = threadIdx.x; idx < G * HD; idx += kThreads) {
        const int r = idx / HD, d = idx - r * HD;
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, red[(size_t)(w * 16 + r) * STATE]);
        float ll = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float* st = red + (size_t)(w * 16 + r) * STATE;
            const float f = mm == -CUDART_INF_F ? 0.0f : exp2f(st[0] - mm);
            ll += st[1] * f;
            a += st[2 + d] * f;
        }
        if (n_splits == 1) {
            out[(size_t)seq * out_stride + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(a / ll);
        } else if (cluster_merge) {
            const uint32_t at = first_block + (uint32_t)(r * STATE) * 4u;
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(at + (uint32_t)(2 + d) * 4u), "f"(a) : "memory");
            if (d == 0) {
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(at), "f"(mm) : "memory");
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(at + 4u), "f"(ll) : "memory");
            }
        } else {
            my_partial[r * STATE + 2 + d] = a;
            if (d == 0) {
                my_partial[r * STATE] = mm;
                my_partial[r * STATE + 1] = ll;
            }
        }
    }
    if (n_splits == 1) return;
    if (cluster_merge) {
        // The first block of the cluster merges the states, in range order as the other way does.
        float* inbox = reinterpret_cast<float*>(smem_raw + kRegion);
        uint32_t rank;
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (rank != 0) return;
        for (int idx = threadIdx.x; idx < G * HD; idx += kThreads) {
            const int r = idx / HD, d = idx - r * HD;
            float mm = -CUDART_INF_F;
            for (int sp = 0; sp < n_splits; ++sp) mm = fmaxf(mm, inbox[(size_t)sp * G * STATE + r * STATE]);
            float ll = 0.0f, a = 0.0f;
            for (int sp = 0; sp < n_splits; ++sp) {
                const float* st = inbox + (size_t)sp * G * STATE + r * STATE;
                const float f = exp2f(st[0] - mm);
                ll += st[1] * f;
                a += st[2 + d] * f;
            }
            out[(size_t)seq * out_stride + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(a / ll);
        }
        return;
    }
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
        const int r = idx / HD, d = idx - r * HD;
        float mm = -CUDART_INF_F;
        for (int sp = 0; sp < n_splits; ++sp) mm = fmaxf(mm, __ldcg(all + (size_t)sp * G * STATE + r * STATE));
        float ll = 0.0f, a = 0.0f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const float* st = all + (size_t)sp * G * STATE + r * STATE;
            const float f = exp2f(__ldcg(st) - mm);        // an empty range has m = -inf: factor 0
            ll += __ldcg(st + 1) * f;
            a += __ldcg(st + 2 + d) * f;
        }
        out[(size_t)seq * out_stride + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(a / ll);
    }
}

// LIYAB_B200_ATTN_CLUSTER=0 in the environment keeps the merge through global memory at every number of ranges
// (measurements: 8 requests x 12 heads at 650 keys in 3 ranges: 7.3 us that way, 5.8 us inside a cluster).
bool cluster_merge_enabled() {
    static const bool on = [] { const char* e = getenv("LIYAB_B200_ATTN_CLUSTER"); return e == nullptr || e[0] != '0'; }();
    return on;
}

// Shared memory of one block and how many blocks of an instantiation one SM holds (asked once).
template <int HD, int kWarps, int kStages, bool TMA>
struct Variant {
    static constexpr size_t tile_bytes = (size_t)kWarps * kStages * 2 * kTile * HD * sizeof(__nv_bfloat16);
    static constexpr size_t red_bytes = (size_t)kWarps * 16 * (HD + 2) * sizeof(float);
    static constexpr size_t smem = (tile_bytes > red_bytes ? tile_bytes : red_bytes) + (TMA ? 1024 : 0);
    static constexpr size_t kInboxMax = (size_t)8 * 16 * (HD + 2) * sizeof(float);       // eight ranges of sixteen query heads

    static int blocks_per_sm(int* out) {
        static int cached = 0;
        if (cached == 0) {
            LB_CHECK_CUDA(cudaFuncSetAttribute(decode_attention_mma_kernel<HD, kWarps, kStages, TMA>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(smem + kInboxMax)));
            int n = 0;
            LB_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_attention_mma_kernel<HD, kWarps, kStages, TMA>,
                                                                        kWarps * 32, smem));
            cached = n > 0 ? n : 1;
        }
        *out = cached;
        return LB_OK;
    }

    static int launch(const CUtensorMap& map_kv, int kv_rows, int* status, const void* q, int64_t q_stride, const void* cache, const int32_t* positions, const int32_t* block_table,
                      int table_stride, void* out, int64_t out_stride, float* partial, int* counters, int n_seq, int n_head,
                      int n_kv_head, int page_shift, float scale, int window, int n_splits, cudaStream_t s) {
        dim3 grid(n_splits, n_kv_head, n_seq);
        // Two to eight key ranges: the ranges of a request and head form a cluster and merge in shared memory.
        const int group = n_head / n_kv_head;
        const bool cluster = n_splits > 1 && n_splits <= 8 && cluster_merge_enabled();
        const size_t inbox = cluster ? (size_t)n_splits * group * (HD + 2) * sizeof(float) : 0;
        int per_sm = 0;
        const int rc = blocks_per_sm(&per_sm);              // sets the kernel's shared-memory limit
        if (rc != LB_OK) return rc;
        LB_CHECK_CUDA(lb_launch_overlapped_cluster(3, cluster ? n_splits : 1, decode_attention_mma_kernel<HD, kWarps, kStages, TMA>, grid,
                                                   dim3(kWarps * 32), smem + inbox, s, map_kv, kv_rows, status, (const __nv_bfloat16*)q,
                                                   q_stride, (const __nv_bfloat16*)cache, positions, block_table, table_stride,
                                                   (__nv_bfloat16*)out, out_stride, partial, counters, n_head, n_kv_head, page_shift,
                                                   scale, window, n_splits, cluster ? 1 : 0));
        return LB_OK;
    }
};

// Blocks of four warps or of two: the one whose last wave of blocks is fuller (four-warp blocks fill an SM with
// fewer blocks, so a count a little above one wave of them leaves a second wave nearly empty; two-warp blocks
// then fit in one).  A choice by the launch's shape only; it changes the order in which tiles are merged, which
// is rounding.
template <int HD, bool TMA>
int launch_for(const CUtensorMap& map_kv, int kv_rows, int* status, const void* q, int64_t q_stride, const void* cache, const int32_t* positions, const int32_t* block_table,
               int table_stride, void* out, int64_t out_stride, float* partial, int* counters, int n_seq, int n_head,
               int n_kv_head, int page_shift, float scale, int window, int n_splits, cudaStream_t s) {
    using Wide = Variant<HD, 4, 2, TMA>;
    using Narrow = Variant<HD, 2, 2, TMA>;
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        LB_CHECK_CUDA(cudaGetDevice(&dev));
        LB_CHECK_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
    }
    int per_wide = 1, per_narrow = 1;
    if (int rc = Wide::blocks_per_sm(&per_wide)) return rc;
    if (int rc = Narrow::blocks_per_sm(&per_narrow)) return rc;
    const long blocks = (long)n_splits * n_kv_head * n_seq;
    const long slots_wide = (long)per_wide * n_sm, slots_narrow = (long)per_narrow * n_sm;
    const long waves_wide = (blocks + slots_wide - 1) / slots_wide, waves_narrow = (blocks + slots_narrow - 1) / slots_narrow;
    // fill = blocks / (waves * slots); compared without division
    const bool narrow = blocks > slots_wide && waves_wide * slots_wide >= waves_narrow * slots_narrow;
    if (narrow)
        return Narrow::launch(map_kv, kv_rows, status, q, q_stride, cache, positions, block_table, table_stride, out, out_stride, partial, counters,
                              n_seq, n_head, n_kv_head, page_shift, scale, window, n_splits, s);
    return Wide::launch(map_kv, kv_rows, status, q, q_stride, cache, positions, block_table, table_stride, out, out_stride, partial, counters, n_seq,
                        n_head, n_kv_head, page_shift, scale, window, n_splits, s);
}

}  // namespace

// Whether the tensor-core decode kernel takes this shape: head size 64 or 128, up to 16 query heads per key/value
// head, pages of 16 positions or more (a power of two), and q rows on 4-byte boundaries.
extern "C" int lb_decode_attention_mma_supports(int n_head, int n_kv_head, int head_dim, int page_size) {
    if (n_kv_head <= 0 || n_head % n_kv_head != 0) return 0;
    const int g = n_head / n_kv_head;
    return (head_dim == 64 || head_dim == 128) && g >= 1 && g <= 16 && page_size >= 16 && (page_size & (page_size - 1)) == 0;
}

// n_pages: the pages of the cache (its first extent).  With head size 64 and a cache that a tensor map can
// describe, the tiles come through TMA; with n_pages 0, or otherwise, through cp.async.
extern "C" int lb_decode_attention_mma(const void* q, int64_t q_stride, const void* cache, int n_pages, const int32_t* positions,
                                       const int32_t* block_table, int table_stride, void* out, int64_t out_stride,
                                       float* partial, int* counters, int n_seq, int n_head, int n_kv_head, int head_dim,
                                       int page_size, float scale, int window, int n_splits, void* stream) {
    LB_CHECK_ARG(n_seq >= 0 && n_splits >= 1, "decode attention: bad sizes n_seq=%d n_splits=%d", n_seq, n_splits);
    if (!lb_decode_attention_mma_supports(n_head, n_kv_head, head_dim, page_size))
        return lb_fail(LB_ERR_UNSUPPORTED, "decode attention (tensor cores): unsupported shape heads %d/%d head_dim %d page_size %d",
                       n_head, n_kv_head, head_dim, page_size);
    LB_CHECK_ARG(n_splits == 1 || (partial != nullptr && counters != nullptr), "decode attention: scratch is missing");
    LB_CHECK_ARG(n_seq <= 65535 && n_kv_head <= 65535, "decode attention: too many requests or heads for one launch");
    LB_CHECK_ARG(q_stride % 2 == 0 && ((uintptr_t)q & 3) == 0, "decode attention: q rows must be 4-byte aligned");
    if (n_seq == 0) return LB_OK;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    auto s = static_cast<cudaStream_t>(stream);
    CUtensorMap none;
    memset(&none, 0, sizeof(none));
    if (head_dim == 64) {
        const int64_t kv_rows = (int64_t)n_pages * 2 * n_kv_head * page_size;
        if (n_pages > 0 && kv_rows < (int64_t)1 << 31 && ((uintptr_t)cache & 15) == 0) {
            CUtensorMap map_kv;
            int* status = nullptr;
            int rc = lb_tensor_map_2d(&map_kv, cache, 2, (int)kv_rows, 64, 64, kTile);
            if (rc == LB_OK) rc = lb_tc_status_word(&status);
            if (rc != LB_OK) return rc;
            return launch_for<64, true>(map_kv, (int)kv_rows, status, q, q_stride, cache, positions, block_table, table_stride,
                                        out, out_stride, partial, counters, n_seq, n_head, n_kv_head, page_shift, scale, window,
                                        n_splits, s);
        }
        return launch_for<64, false>(none, 0, nullptr, q, q_stride, cache, positions, block_table, table_stride, out, out_stride,
                                     partial, counters, n_seq, n_head, n_kv_head, page_shift, scale, window, n_splits, s);
    }
    return launch_for<128, false>(none, 0, nullptr, q, q_stride, cache, positions, block_table, table_stride, out, out_stride,
                                  partial, counters, n_seq, n_head, n_kv_head, page_shift, scale, window, n_splits, s);
}
