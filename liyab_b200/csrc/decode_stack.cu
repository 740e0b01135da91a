// A whole decode step of a stack of pre-norm blocks in ONE persistent kernel, for
// steps of at most 16 tokens (one per request) in bfloat16.
//
// Why: at this size a layer has to read about 14 MB of weights and a few MB of
// cache, two microseconds of HBM time, while a step run kernel by kernel pays a
// launch and a memory round trip for each of its hundred kernels.  Here one
// cooperative grid (one block per SM) walks the phases of every layer with a
// grid-wide barrier between them:
//
//   embed | per layer: [LayerNorm + QKV + cache write] [attention] [output
//   projection + residual] [LayerNorm + up + activation] [down + residual] |
//   final LayerNorm + head
//
// A matrix phase gives every block a slice of the output features and the whole
// reduction length: the (normalised) activations of all tokens sit in shared
// memory as bfloat16, each warp streams its part of the weight rows from HBM
// with 16-byte loads straight into mma.sync m16n8k16 fragments (tokens are the
// 16 rows, 8 features the columns), the eight warps split K and their partial
// tiles are summed in a fixed order.  So every weight byte is read once, all SMs
// stream together, and a row's result does not depend on the other rows.  The
// attention phase is the split-key scheme of attention_decode.cu with work items
// (token, head, key range) dealt round-robin to the blocks.
//
// LayerNorm statistics, softmax, the residual stream (float32 in global memory)
// and all accumulators are 32-bit.  Formulas and order are those of the
// part-by-part path (see elementwise.cu, attention_decode.cu, gemm_tcgen05.cu and
// the reference lines they cite).
//
// The grid barrier spins on a counter in global memory; the spin is bounded
// (about two seconds), after which the block records the phase in the status
// word, every block leaves at its next barrier, and the host sees the status.
#include "api.h"
#include "common.cuh"

#include <cooperative_groups.h>
#include <math_constants.h>

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kMaxTokens = 16;
constexpr int kGC = 8;                           // feature groups (of 8 features) a block handles per pass
constexpr long long kSpinLimit = 4000000000ll;   // cycles
constexpr float kLog2e = 1.4426950408889634f;

// One entry of the run order.  Python packs this with struct format "<13Q3f6i4x" (144 bytes).
struct StackLayer {
    const float* ln1_w;
    const float* ln1_b;
    const float* ln2_w;
    const float* ln2_b;
    const __nv_bfloat16* w_qkv;
    const float* b_qkv;
    const __nv_bfloat16* w_out;
    const float* b_out;
    const __nv_bfloat16* w_up;
    const float* b_up;
    const __nv_bfloat16* w_down;
    const float* b_down;
    __nv_bfloat16* cache;
    float ln1_eps, ln2_eps, scale;
    int n_head, n_kv_head, head_dim, inner, act, window;
    int pad_;
};
static_assert(sizeof(StackLayer) == 144, "StackLayer must match the layout the Python side packs");

struct StackParams {
    const StackLayer* layers;
    int n_layers, n_tokens, width, vocab;
    const __nv_bfloat16* embedding;
    const __nv_bfloat16* pos_table;
    float embed_scale;
    const float* lnf_w;
    const float* lnf_b;
    float lnf_eps;
    const __nv_bfloat16* head_w;
    const float* head_b;
    const int32_t* tokens;
    const int32_t* positions;
    const int32_t* block_table;
    int table_stride;
    const int32_t* slot_mapping;
    int page_shift;
    float* x;
    __nv_bfloat16* q;
    __nv_bfloat16* att;
    __nv_bfloat16* inner;
    float* partial;
    int* counters;
    float* logits;
    unsigned* barrier;
    int* status;
    int n_splits, act_ld;
    unsigned long long* timing;      // optional: block 0 stamps the global timer after every barrier
};

__device__ int g_stack_status = 0;

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Grid-wide barrier number `epoch` (1, 2, ...) on a counter that starts at zero.  False: gave up or told to.
__device__ bool grid_sync(const StackParams& p, unsigned& epoch, int phase_code) {
    __shared__ int ok_s;
    __syncthreads();
    if (threadIdx.x == 0) {
        ++epoch;
        const unsigned target = epoch * gridDim.x;
        // The release on the add publishes what this block wrote before the barrier (the block-wide
        // barrier above ordered its threads' writes before this thread); the acquire on the load makes
        // the other blocks' writes visible to everything after the barrier.
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.barrier) : "memory");
        int ok = 1;
        const long long t0 = clock64();
        for (unsigned spins = 1;; ++spins) {
            unsigned seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.barrier) : "memory");
            if (seen >= target) break;
            if ((spins & 1023u) == 0) {
                if (*(volatile int*)p.status != 0) { ok = 0; break; }
                if (clock64() - t0 > kSpinLimit) {
                    atomicCAS(p.status, 0, phase_code);
                    ok = 0;
                    break;
                }
            }
        }
        ok_s = ok;
        if (p.timing != nullptr && blockIdx.x == 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            p.timing[epoch] = now;
        }
    } else {
        ++epoch;
    }
    __syncthreads();
    return ok_s != 0;
}

// Optional fine-grained stamps of block 0 (work done before a barrier, staging done, ...), after the barrier stamps.
__device__ __forceinline__ void stamp(const StackParams& p, int slot) {
    if (p.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        p.timing[slot] = now;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Rows of x (float32, written by other blocks: read through L2) -> LayerNorm -> bfloat16 rows in shared memory.
// One warp per row.  Up to 1024 columns the row is fetched once, as 16-byte loads that are all in flight
// together, and kept in registers for both statistics and the output; wider rows are read three times.
__device__ void layernorm_to_smem(const float* x, const float* __restrict__ w, const float* __restrict__ b, float eps,
                                  int n_rows, int width, __nv_bfloat16* act_s, int ld, int k_pad) {
    constexpr int kVecs = 8;                        // float4 per lane held in registers (row, gains, offsets)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool in_regs = width % 4 == 0 && width <= kVecs * 32 * 4;
    for (int r = warp; r < n_rows; r += kWarps) {
        const float* row = x + (size_t)r * width;
        __nv_bfloat16* dst = act_s + r * ld;
        if (in_regs) {
            const int n_vec = width / 4;
            // The row, the gains and the offsets are all requested before anything is used: one round trip.
            float4 v[kVecs], gain[kVecs], offs[kVecs];
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int i = lane + 32 * j;
                const bool in = i < n_vec;
                v[j] = in ? __ldcg(reinterpret_cast<const float4*>(row) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                gain[j] = (in && w != nullptr) ? __ldg(reinterpret_cast<const float4*>(w) + i) : make_float4(1.f, 1.f, 1.f, 1.f);
                offs[j] = (in && b != nullptr) ? __ldg(reinterpret_cast<const float4*>(b) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < kVecs; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
            const float mean = warp_sum(sum) / (float)width;
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
            const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)width + eps);
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
            for (int i = width + lane; i < k_pad; i += 32) dst[i] = __float2bfloat16_rn(0.0f);
        } else {
            float sum = 0.0f;
            for (int i = lane; i < width; i += 32) sum += __ldcg(row + i);
            const float mean = warp_sum(sum) / (float)width;
            float ss = 0.0f;
            for (int i = lane; i < width; i += 32) {
                const float d = __ldcg(row + i) - mean;
                ss = fmaf(d, d, ss);
            }
            const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)width + eps);
            for (int i = lane; i < k_pad; i += 32) {
                float y = 0.0f;
                if (i < width) {
                    y = (__ldcg(row + i) - mean) * inv;
                    if (w != nullptr) y *= w[i];
                    if (b != nullptr) y += b[i];
                }
                dst[i] = __float2bfloat16_rn(y);
            }
        }
    }
}

// Asks L2 for this block's slice of a weight matrix (the rows gemm_phase will give it), one request per
// 128 bytes.  Issued a phase or two ahead, so that the slice streams from HBM while other work runs and the
// matrix phase finds it in L2.
__device__ void prefetch_slice(const __nv_bfloat16* __restrict__ W, int N, int K) {
    const int n_groups = (N + 7) / 8;
    const int per_cta = (n_groups + (int)gridDim.x - 1) / (int)gridDim.x;
    const int f0 = min(N, (int)blockIdx.x * per_cta * 8), f1 = min(N, f0 + per_cta * 8);
    const char* base = reinterpret_cast<const char*>(W + (size_t)f0 * K);
    const size_t bytes = (size_t)(f1 - f0) * K * sizeof(__nv_bfloat16);
    for (size_t off = (size_t)threadIdx.x * 128; off < bytes; off += (size_t)kThreads * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
}

// Rows of a bfloat16 matrix written by other blocks -> shared memory, the tail up to k_pad zeroed.
__device__ void rows_to_smem(const __nv_bfloat16* src, int n_rows, int width, __nv_bfloat16* act_s, int ld, int k_pad) {
    // Stores go to shared memory, so the compiler is free to request the loads of several trips ahead of them.
    const int chunks = k_pad / 8;
    for (int idx = threadIdx.x; idx < n_rows * chunks; idx += kThreads) {
        const int r = idx / chunks, c = idx - r * chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (c * 8 < width) v = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)r * width + c * 8));
        *reinterpret_cast<uint4*>(act_s + r * ld + c * 8) = v;
    }
}

__device__ __forceinline__ uint4 load_w(const __nv_bfloat16* __restrict__ W, int N, int K, int f, int k) {
    if (f < N && k < K) return __ldg(reinterpret_cast<const uint4*>(W + (size_t)f * K + k));
    return make_uint4(0, 0, 0, 0);
}

// out[b, f] = sum_k act[b, k] * W[f, k] for this block's slice of the features.  An element (b, f) is finished by
// post(b, f, value, pre(b, f)); pre() is called before the weights are streamed, so whatever it loads from global
// memory (a bias, the residual) travels together with the weights instead of after them.
template <typename Pre, typename Post>
__device__ void gemm_phase(const __nv_bfloat16* __restrict__ W, int N, int K, const __nv_bfloat16* act_s, int ld,
                           float* red_s, int n_tokens, Pre pre, Post post) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n_groups = (N + 7) / 8;
    const int per_cta = (n_groups + (int)gridDim.x - 1) / (int)gridDim.x;
    const int g_begin = blockIdx.x * per_cta, g_end = min(n_groups, g_begin + per_cta);
    const int n_kb = (K + 31) / 32, per_warp = (n_kb + kWarps - 1) / kWarps;
    const int kb0 = warp * per_warp, kb1 = min(n_kb, kb0 + per_warp);
    const __nv_bfloat16* a_lo = act_s + g * ld + t * 8;
    const __nv_bfloat16* a_hi = a_lo + 8 * ld;
    for (int gp = g_begin; gp < g_end; gp += kGC) {
        const int ng = min(kGC, g_end - gp);
        float2 early[kGC * 128 / kThreads];
#pragma unroll
        for (int e = 0; e < kGC * 128 / kThreads; ++e) {
            const int idx = threadIdx.x + e * kThreads;
            const int gi = idx >> 7, r = (idx >> 3) & 15, f = (gp + gi) * 8 + (idx & 7);
            early[e] = (idx < ng * 128 && r < n_tokens && f < N) ? pre(r, f) : make_float2(0.f, 0.f);
        }
        float acc[kGC][4];
#pragma unroll
        for (int i = 0; i < kGC; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
        if (ng == 1) {
            // One group, long K: eight k-blocks are requested before the first is used.
            for (int kb = kb0; kb < kb1; kb += 8) {
                uint4 w[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    w[u] = kb + u < kb1 ? load_w(W, N, K, gp * 8 + g, (kb + u) * 32 + t * 8) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (kb + u < kb1) {
                        const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + (kb + u) * 32);
                        const uint4 hi = *reinterpret_cast<const uint4*>(a_hi + (kb + u) * 32);
                        mma_bf16(acc[0], lo.x, hi.x, lo.y, hi.y, w[u].x, w[u].y);
                        mma_bf16(acc[0], lo.z, hi.z, lo.w, hi.w, w[u].z, w[u].w);
                    }
                }
            }
        } else if (ng == 2) {
            // Two groups: four k-blocks of both are requested before the first is used.
            for (int kb = kb0; kb < kb1; kb += 4) {
                uint4 w[2][4];
#pragma unroll
                for (int gi = 0; gi < 2; ++gi)
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        w[gi][u] = kb + u < kb1 ? load_w(W, N, K, (gp + gi) * 8 + g, (kb + u) * 32 + t * 8)
                                                : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (kb + u < kb1) {
                        const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + (kb + u) * 32);
                        const uint4 hi = *reinterpret_cast<const uint4*>(a_hi + (kb + u) * 32);
#pragma unroll
                        for (int gi = 0; gi < 2; ++gi) {
                            mma_bf16(acc[gi], lo.x, hi.x, lo.y, hi.y, w[gi][u].x, w[gi][u].y);
                            mma_bf16(acc[gi], lo.z, hi.z, lo.w, hi.w, w[gi][u].z, w[gi][u].w);
                        }
                    }
                }
            }
        } else if (ng <= 4) {
            // Up to four groups: two k-blocks of all of them are requested before the first is used.
            for (int kb = kb0; kb < kb1; kb += 2) {
                uint4 w[4][2];
#pragma unroll
                for (int gi = 0; gi < 4; ++gi)
#pragma unroll
                    for (int u = 0; u < 2; ++u)
                        w[gi][u] = (gi < ng && kb + u < kb1) ? load_w(W, N, K, (gp + gi) * 8 + g, (kb + u) * 32 + t * 8)
                                                            : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (kb + u < kb1) {
                        const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + (kb + u) * 32);
                        const uint4 hi = *reinterpret_cast<const uint4*>(a_hi + (kb + u) * 32);
#pragma unroll
                        for (int gi = 0; gi < 4; ++gi) {
                            if (gi < ng) {
                                mma_bf16(acc[gi], lo.x, hi.x, lo.y, hi.y, w[gi][u].x, w[gi][u].y);
                                mma_bf16(acc[gi], lo.z, hi.z, lo.w, hi.w, w[gi][u].z, w[gi][u].w);
                            }
                        }
                    }
                }
            }
        } else {
            // Many features: one k-block of up to eight groups per trip.
#pragma unroll 2
            for (int kb = kb0; kb < kb1; ++kb) {
                uint4 w[kGC];
#pragma unroll
                for (int gi = 0; gi < kGC; ++gi)
                    w[gi] = gi < ng ? load_w(W, N, K, (gp + gi) * 8 + g, kb * 32 + t * 8) : make_uint4(0, 0, 0, 0);
                const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + kb * 32);
                const uint4 hi = *reinterpret_cast<const uint4*>(a_hi + kb * 32);
#pragma unroll
                for (int gi = 0; gi < kGC; ++gi) {
                    if (gi < ng) {
                        mma_bf16(acc[gi], lo.x, hi.x, lo.y, hi.y, w[gi].x, w[gi].y);
                        mma_bf16(acc[gi], lo.z, hi.z, lo.w, hi.w, w[gi].z, w[gi].w);
                    }
                }
            }
        }
        // Partial tiles of the eight warps -> shared memory -> summed in warp order.
#pragma unroll
        for (int gi = 0; gi < kGC; ++gi) {
            if (gi < ng) {
                float* tile = red_s + (warp * kGC + gi) * 128;
                tile[g * 8 + 2 * t] = acc[gi][0];
                tile[g * 8 + 2 * t + 1] = acc[gi][1];
                tile[(g + 8) * 8 + 2 * t] = acc[gi][2];
                tile[(g + 8) * 8 + 2 * t + 1] = acc[gi][3];
            }
        }
        __syncthreads();
#pragma unroll
        for (int e = 0; e < kGC * 128 / kThreads; ++e) {
            const int idx = threadIdx.x + e * kThreads;
            if (idx < ng * 128) {
                const int gi = idx >> 7, r = (idx >> 3) & 15, c = idx & 7;
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) v += red_s[(w * kGC + gi) * 128 + r * 8 + c];
                const int f = (gp + gi) * 8 + c;
                if (r < n_tokens && f < N) post(r, f, v, early[e]);
            }
        }
        __syncthreads();
    }
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// Attention of every (token, head) over its pages; work items (token, head, key range) go round-robin to the blocks.
// `table_s` holds the block-table rows of this block's first kCachedItems work items and `pos_s` the tokens'
// positions, copied once per step (they are the same for every layer) when `cached_heads` equals the layer's heads.
constexpr int kCachedItems = 2;

template <int HD>
__device__ void attention_phase(const StackParams& p, const StackLayer& L, float* att_s, const int32_t* table_s,
                                const int32_t* pos_s, int cached_heads) {
    constexpr int TPK = HD / 8, KPW = 32 / TPK, STATE = HD + 2, U = 8;
    __shared__ int last_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane % TPK, kgroup = lane / TPK;
    const int B = p.n_tokens, H = L.n_head, G = H / L.n_kv_head, splits = p.n_splits;
    const int qd = H * HD, page_size = 1 << p.page_shift;
    const size_t plane = (size_t)L.n_kv_head * page_size * HD;
    int item_slot = 0;
    for (int item = blockIdx.x; item < B * H * splits; item += gridDim.x, ++item_slot) {
        const int split = item % splits, bh = item / splits, h = bh % H, b = bh / H, kvh = h / G;
        const int pos = pos_s[b];
        const int first = L.window > 0 ? max(0, pos - L.window + 1) : 0;
        const int n_keys = pos + 1 - first;
        const int chunk = (n_keys + splits - 1) / splits;
        const int begin = first + split * chunk, end = min(pos + 1, begin + chunk);
        const uint4 q_raw = __ldcg(reinterpret_cast<const uint4*>(p.q + (size_t)b * qd + (size_t)h * HD + sub * 8));
        // Page ids: from the rows copied to shared memory at the start of the step, else from global memory.
        const int32_t* table = (cached_heads == H && item_slot < kCachedItems)
                                   ? table_s + (size_t)item_slot * p.table_stride
                                   : p.block_table + (size_t)b * p.table_stride;
        float qf[8];
        unpack8(q_raw, qf);
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[i] *= L.scale * kLog2e;
        float m = -CUDART_INF_F, l = 0.0f, acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        for (int jb = begin + warp * KPW; jb < end; jb += kWarps * KPW * U) {
            uint4 kraw[U], vraw[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = jb + kgroup + u * kWarps * KPW;
                if (j < end) {
                    const int page = table[j >> p.page_shift];
                    const __nv_bfloat16* row = L.cache + (size_t)page * 2 * plane +
                                               ((size_t)kvh * page_size + (j & (page_size - 1))) * HD + sub * 8;
                    kraw[u] = __ldcg(reinterpret_cast<const uint4*>(row));
                    vraw[u] = __ldcg(reinterpret_cast<const uint4*>(row + plane));
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = jb + kgroup + u * kWarps * KPW;
                const bool live = j < end;
                float kf[8], vf[8];
                if (live) {
                    unpack8(kraw[u], kf);
                    unpack8(vraw[u], vf);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) kf[i] = vf[i] = 0.0f;
                }
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) s = fmaf(qf[i], kf[i], s);
#pragma unroll
                for (int o = TPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (live) {
                    const float m_new = fmaxf(m, s);
                    const float corr = exp2f(m - m_new), pj = exp2f(s - m_new);
                    l = l * corr + pj;
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = fmaf(pj, vf[i], acc[i] * corr);
                    m = m_new;
                }
            }
        }
        // Key groups of the warp, in a fixed pairing; both partners end with the same state.
#pragma unroll
        for (int o = TPK; o < 32; o <<= 1) {
            const float m_b = __shfl_xor_sync(0xffffffffu, m, o), l_b = __shfl_xor_sync(0xffffffffu, l, o);
            float acc_b[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc_b[i] = __shfl_xor_sync(0xffffffffu, acc[i], o);
            const bool low = (lane & o) == 0;
            const float m0 = low ? m : m_b, l0 = low ? l : l_b, m1 = low ? m_b : m, l1 = low ? l_b : l;
            const float mn = fmaxf(m0, m1);
            const float f0 = mn == -CUDART_INF_F ? 0.0f : exp2f(m0 - mn), f1 = mn == -CUDART_INF_F ? 0.0f : exp2f(m1 - mn);
            l = l0 * f0 + l1 * f1;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = (low ? acc[i] : acc_b[i]) * f0 + (low ? acc_b[i] : acc[i]) * f1;
            m = mn;
        }
        if (kgroup == 0) {
            float* st = att_s + warp * STATE;
            st[0] = m;
            st[1] = l;
#pragma unroll
            for (int i = 0; i < 8; ++i) st[2 + sub * 8 + i] = acc[i];
        }
        __syncthreads();
        float* mine = p.partial + (size_t)item * STATE;
        if (threadIdx.x < HD) {
            const int d = threadIdx.x;
            float mm = -CUDART_INF_F;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, att_s[w * STATE]);
            float ll = 0.0f, a = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float f = mm == -CUDART_INF_F ? 0.0f : exp2f(att_s[w * STATE] - mm);
                ll += att_s[w * STATE + 1] * f;
                a += att_s[w * STATE + 2 + d] * f;
            }
            if (splits == 1) {
                p.att[(size_t)b * qd + (size_t)h * HD + d] = __float2bfloat16_rn(a / ll);
            } else {
                mine[2 + d] = a;
                if (d == 0) {
                    mine[0] = mm;
                    mine[1] = ll;
                }
            }
        }
        if (splits > 1) {
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const int done = atomicAdd(&p.counters[bh], 1);
                last_s = done == splits - 1;
                if (last_s) p.counters[bh] = 0;
            }
            __syncthreads();
            if (last_s) {
                __threadfence();
                const float* all = p.partial + (size_t)bh * splits * STATE;
                if (threadIdx.x < HD) {
                    const int d = threadIdx.x;
                    float mm = -CUDART_INF_F;
                    for (int sp = 0; sp < splits; ++sp) mm = fmaxf(mm, __ldcg(all + (size_t)sp * STATE));
                    float ll = 0.0f, a = 0.0f;
                    for (int sp = 0; sp < splits; ++sp) {
                        const float f = exp2f(__ldcg(all + (size_t)sp * STATE) - mm);
                        ll += __ldcg(all + (size_t)sp * STATE + 1) * f;
                        a += __ldcg(all + (size_t)sp * STATE + 2 + d) * f;
                    }
                    p.att[(size_t)b * qd + (size_t)h * HD + d] = __float2bfloat16_rn(a / ll);
                }
            }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kThreads, 1) decode_stack_kernel(const StackParams p) {
    extern __shared__ __align__(16) uint8_t smem_bytes[];
    __nv_bfloat16* act_s = reinterpret_cast<__nv_bfloat16*>(smem_bytes);
    float* red_s = reinterpret_cast<float*>(smem_bytes + (size_t)kMaxTokens * p.act_ld * sizeof(__nv_bfloat16));
    float* att_s = red_s + kWarps * kGC * 128;
    int32_t* pos_s = reinterpret_cast<int32_t*>(att_s + kWarps * (128 + 2));       // [kMaxTokens] positions
    int32_t* table_s = pos_s + kMaxTokens;                                          // [kCachedItems][table_stride] page ids
    const int B = p.n_tokens, d = p.width, ld = p.act_ld;
    unsigned epoch = 0;
    if (p.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        p.timing[0] = now;
    }

    // Positions and the block-table rows of this block's attention work items: the same for every layer.
    const int cached_heads = p.n_layers > 0 ? p.layers[0].n_head : 0;
    for (int i = threadIdx.x; i < B; i += kThreads) pos_s[i] = p.positions[i];
    for (int slot = 0; slot < kCachedItems; ++slot) {
        const int item = blockIdx.x + slot * gridDim.x;
        if (item < B * cached_heads * p.n_splits) {
            const int b = item / p.n_splits / cached_heads;
            for (int i = threadIdx.x; i < p.table_stride; i += kThreads)
                table_s[(size_t)slot * p.table_stride + i] = p.block_table[(size_t)b * p.table_stride + i];
        }
    }

    // Embedding (+ learned position) into the residual stream.
    for (int idx = blockIdx.x * kThreads + threadIdx.x; idx < B * d; idx += gridDim.x * kThreads) {
        const int b = idx / d, i = idx - b * d;
        float v = __bfloat162float(p.embedding[(size_t)p.tokens[b] * d + i]) * p.embed_scale;
        if (p.pos_table != nullptr) v += __bfloat162float(p.pos_table[(size_t)p.positions[b] * d + i]);
        p.x[idx] = v;
    }
    if (!grid_sync(p, epoch, 1)) return;

    for (int li = 0; li < p.n_layers; ++li) {
        const StackLayer L = p.layers[li];
        const int hd = L.head_dim, qd = L.n_head * hd, kvd = L.n_kv_head * hd, page_size = 1 << p.page_shift;
        const size_t plane = (size_t)L.n_kv_head * page_size * hd;
        const int code = (li + 1) << 4;

        // LayerNorm 1, fused projection, keys and values into their pages.
        stamp(p, 128 + li * 8 + 4);
        prefetch_slice(L.w_qkv, qd + 2 * kvd, d);
        prefetch_slice(L.w_out, d, qd);
        stamp(p, 128 + li * 8 + 5);
        layernorm_to_smem(p.x, L.ln1_w, L.ln1_b, L.ln1_eps, B, d, act_s, ld, (d + 63) / 64 * 64);
        __syncthreads();
        stamp(p, 128 + li * 8 + 0);
        gemm_phase(L.w_qkv, qd + 2 * kvd, d, act_s, ld, red_s, B, [&](int b, int f) {
            return make_float2(L.b_qkv != nullptr ? __ldg(L.b_qkv + f) : 0.0f, __int_as_float(f >= qd ? __ldg(p.slot_mapping + b) : 0));
        }, [&](int b, int f, float v, float2 e) {
            v += e.x;
            if (f < qd) {
                p.q[(size_t)b * qd + f] = __float2bfloat16_rn(v);
            } else {
                const int kvf = f - qd, which = kvf >= kvd ? 1 : 0, within = kvf - which * kvd;
                const int head = within / hd, dd = within - head * hd;
                const int slot = __float_as_int(e.y);
                if (slot >= 0) {
                    const int page = slot >> p.page_shift, off = slot & (page_size - 1);
                    L.cache[(size_t)page * 2 * plane + (size_t)which * plane + ((size_t)head * page_size + off) * hd + dd] =
                        __float2bfloat16_rn(v);
                }
            }
        });
        stamp(p, 128 + li * 8 + 1);
        if (!grid_sync(p, epoch, code | 1)) return;

        if (hd == 64) attention_phase<64>(p, L, att_s, table_s, pos_s, cached_heads);
        else attention_phase<128>(p, L, att_s, table_s, pos_s, cached_heads);
        stamp(p, 128 + li * 8 + 2);
        if (!grid_sync(p, epoch, code | 2)) return;

        // Output projection + residual.
        rows_to_smem(p.att, B, qd, act_s, ld, (qd + 63) / 64 * 64);
        __syncthreads();
        gemm_phase(L.w_out, d, qd, act_s, ld, red_s, B, [&](int b, int f) {
            return make_float2(L.b_out != nullptr ? __ldg(L.b_out + f) : 0.0f, __ldcg(p.x + (size_t)b * d + f));
        }, [&](int b, int f, float v, float2 e) { p.x[(size_t)b * d + f] = e.y + (v + e.x); });
        stamp(p, 128 + li * 8 + 3);
        if (!grid_sync(p, epoch, code | 3)) return;

        // LayerNorm 2, up projection, activation.
        prefetch_slice(L.w_up, L.inner, d);
        prefetch_slice(L.w_down, d, L.inner);
        if (li + 1 == p.n_layers) prefetch_slice(p.head_w, p.vocab, d);
        layernorm_to_smem(p.x, L.ln2_w, L.ln2_b, L.ln2_eps, B, d, act_s, ld, (d + 63) / 64 * 64);
        __syncthreads();
        gemm_phase(L.w_up, L.inner, d, act_s, ld, red_s, B, [&](int b, int f) {
            return make_float2(L.b_up != nullptr ? __ldg(L.b_up + f) : 0.0f, 0.0f);
        }, [&](int b, int f, float v, float2 e) {
            p.inner[(size_t)b * L.inner + f] = __float2bfloat16_rn(lb_activate(v + e.x, L.act));
        });
        if (!grid_sync(p, epoch, code | 4)) return;

        // Down projection + residual.
        rows_to_smem(p.inner, B, L.inner, act_s, ld, (L.inner + 63) / 64 * 64);
        __syncthreads();
        gemm_phase(L.w_down, d, L.inner, act_s, ld, red_s, B, [&](int b, int f) {
            return make_float2(L.b_down != nullptr ? __ldg(L.b_down + f) : 0.0f, __ldcg(p.x + (size_t)b * d + f));
        }, [&](int b, int f, float v, float2 e) { p.x[(size_t)b * d + f] = e.y + (v + e.x); });
        if (!grid_sync(p, epoch, code | 5)) return;
    }

    // Final norm and the head.
    layernorm_to_smem(p.x, p.lnf_w, p.lnf_b, p.lnf_eps, B, d, act_s, ld, (d + 63) / 64 * 64);
    __syncthreads();
    gemm_phase(p.head_w, p.vocab, d, act_s, ld, red_s, B, [&](int b, int f) {
        return make_float2(p.head_b != nullptr ? __ldg(p.head_b + f) : 0.0f, 0.0f);
    }, [&](int b, int f, float v, float2 e) { p.logits[(size_t)b * p.vocab + f] = v + e.x; });
}

int g_sm_count = 0;

}  // namespace

// Bytes of one packed layer record (for the Python side to check its struct format against).
extern "C" int lb_decode_stack_layer_bytes(void) { return (int)sizeof(StackLayer); }

// Floats of attention scratch for n_tokens tokens, n_head heads, head_dim and n_splits key ranges.
extern "C" int64_t lb_decode_stack_scratch_floats(int n_tokens, int n_head, int head_dim, int n_splits) {
    return (int64_t)n_tokens * n_head * n_splits * (head_dim + 2);
}

extern "C" int lb_decode_stack(const void* layers_dev, int n_layers, int n_tokens, int width, int vocab,
                               const void* embedding, const void* pos_table, float embed_scale, const float* lnf_w,
                               const float* lnf_b, float lnf_eps, const void* head_w, const float* head_b,
                               const int32_t* tokens, const int32_t* positions, const int32_t* block_table,
                               int table_stride, const int32_t* slot_mapping, int page_size, float* x, void* q, void* att,
                               void* inner, float* partial, int* counters, float* logits, unsigned* barrier, int max_k,
                               int head_dim, int n_splits, unsigned long long* timing, void* stream) {
    LB_CHECK_ARG(n_layers >= 0 && n_tokens >= 1 && n_tokens <= kMaxTokens, "decode stack: %d tokens (1..%d are taken)", n_tokens,
                 kMaxTokens);
    LB_CHECK_ARG(width > 0 && width % 8 == 0 && max_k >= width && max_k % 8 == 0 && vocab > 0,
                 "decode stack: width %d and the largest reduction length %d must be multiples of 8", width, max_k);
    LB_CHECK_ARG(head_dim == 64 || head_dim == 128, "decode stack: head_dim %d (64 and 128 are taken)", head_dim);
    LB_CHECK_ARG(page_size > 0 && (page_size & (page_size - 1)) == 0, "decode stack: page_size %d is not a power of two", page_size);
    LB_CHECK_ARG(n_splits >= 1 && n_splits <= 64, "decode stack: n_splits %d", n_splits);
    auto s = static_cast<cudaStream_t>(stream);
    if (g_sm_count == 0) {
        int dev = 0, coop = 0;
        LB_CHECK_CUDA(cudaGetDevice(&dev));
        LB_CHECK_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
        if (!coop) return lb_fail(LB_ERR_UNSUPPORTED, "decode stack: the device does not launch cooperative kernels");
        LB_CHECK_CUDA(cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev));
    }
    StackParams p;
    p.layers = static_cast<const StackLayer*>(layers_dev);
    p.n_layers = n_layers;
    p.n_tokens = n_tokens;
    p.width = width;
    p.vocab = vocab;
    p.embedding = static_cast<const __nv_bfloat16*>(embedding);
    p.pos_table = static_cast<const __nv_bfloat16*>(pos_table);
    p.embed_scale = embed_scale;
    p.lnf_w = lnf_w;
    p.lnf_b = lnf_b;
    p.lnf_eps = lnf_eps;
    p.head_w = static_cast<const __nv_bfloat16*>(head_w);
    p.head_b = head_b;
    p.tokens = tokens;
    p.positions = positions;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.slot_mapping = slot_mapping;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.x = x;
    p.q = static_cast<__nv_bfloat16*>(q);
    p.att = static_cast<__nv_bfloat16*>(att);
    p.inner = static_cast<__nv_bfloat16*>(inner);
    p.partial = partial;
    p.counters = counters;
    p.logits = logits;
    p.barrier = barrier;
    int* status = nullptr;
    LB_CHECK_CUDA(cudaGetSymbolAddress((void**)&status, g_stack_status));
    p.status = status;
    p.n_splits = n_splits;
    p.timing = timing;
    p.act_ld = (max_k + 63) / 64 * 64 + 32;       // row stride = 64 bytes mod 128: conflict-free 16-byte reads
    const size_t smem = (size_t)kMaxTokens * p.act_ld * sizeof(__nv_bfloat16) + (size_t)kWarps * kGC * 128 * sizeof(float) +
                        (size_t)kWarps * (128 + 2) * sizeof(float) + (size_t)(kMaxTokens + kCachedItems * table_stride) * sizeof(int32_t);
    LB_CHECK_ARG(smem <= 227 * 1024, "decode stack: a reduction length of %d needs %zu bytes of shared memory, the SM has 232448",
                 max_k, smem);
    static size_t configured = 0;
    if (smem > configured) {
        LB_CHECK_CUDA(cudaFuncSetAttribute(decode_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    LB_CHECK_CUDA(cudaMemsetAsync(barrier, 0, sizeof(unsigned), s));
    void* args[] = {&p};
    LB_CHECK_CUDA(cudaLaunchCooperativeKernel((const void*)decode_stack_kernel, dim3(g_sm_count), dim3(kThreads), args, smem, s));
    return LB_OK;
}

// Reads and clears the status word of the grid barrier (0: every barrier so far completed).  Synchronises the device.
extern "C" int lb_decode_stack_status(int* status) {
    int zero = 0;
    LB_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_stack_status, sizeof(int)));
    LB_CHECK_CUDA(cudaMemcpyToSymbol(g_stack_status, &zero, sizeof(int)));
    return LB_OK;
}
