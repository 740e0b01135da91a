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
// memory as bfloat16, each warp takes its part of the weight rows with 16-byte
// loads straight into mma.sync m16n8k16 fragments (tokens are the 16 rows, 8
// features the columns), the eight warps split K and their partial tiles are
// summed in a fixed order.  So every weight byte is read once, all SMs stream
// together, and a row's result does not depend on the other rows.  Weights do not
// depend on what the phase before computed, so a block asks for its slice of the
// NEXT matrix phase before it enters the barrier that ends the current one (into
// registers, where the slice is a dozen 16-byte pieces per thread, which it is for
// the layers of models up to GPT-2 medium; L2 prefetches go out two phases ahead):
// the weights' latency hides behind the barrier and the staging of the
// activations, and a phase is little more than barrier + one round trip for the
// activations + the products.
//
// The attention phase deals work items (token, key/value head, key range) to the
// 2 x blocks groups of four warps; a group runs the tensor-core scheme of
// attention_decode_mma.cu (16-key tiles through a cp.async ring per warp, scores
// and weighted values as mma.sync, running softmax per warp, merge in shared
// memory, key ranges merged by the group that finishes last).  The head is
// streamed without any block-wide barrier: every warp owns whole groups of eight
// vocabulary rows and walks K in double-buffered chunks.
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
constexpr int kWRegs = 16;                       // 16-byte weight pieces a thread holds for the next matrix phase
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
static_assert(sizeof(StackLayer) == 144, "StackLayer must match the layout the host packs");

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
    unsigned* barrier;               // this launch's grid-barrier counter (starts at zero)
    unsigned* other_barrier;         // the one the launch before used: block 0 zeroes it for the launch after
    int* status;
    int n_splits, act_ld;
    int unit_warps;                  // warps that share an attention work item: 4 (two items per block at a time) or 8
    int bars_offset;                         // 8 x 4 mbarriers of the head's rings
    int head_ring_offset, head_ring_bytes;   // the head's cp.async ring: shared memory after the activations
    int pos_offset;                  // byte offset of the positions in shared memory (after what the phases share)
    unsigned long long* timing;      // optional: block 0 stamps the global timer after every barrier
    int withhold_arrival;            // a test's launch: block 0 is not counted at the first barrier, which then runs out
};

__device__ int g_stack_status = 0;
static int g_withhold_next = 0;      // host side: the next launch's block 0 skips its first arrival (tests)

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Grid-wide barrier number `epoch` (1, 2, ...) on a counter that starts at zero, in two halves.  grid_arrive:
// everything this block wrote is published and the block is counted.  grid_wait: until every block is counted;
// false: gave up or told to.  Between the two a block may issue loads of data that no block writes (the next
// phase's weights): they travel while the block waits.  (Issued before the arrival they would delay it: the
// arriving thread's release waits for its own earlier loads.)
__device__ void grid_arrive(const StackParams& p, unsigned& epoch) {
    __syncthreads();
    ++epoch;
    if (threadIdx.x == 0) {
        if (p.timing != nullptr && epoch >= 27 && epoch <= 31) {       // arrival of every block at the five barriers of layer 5
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            p.timing[256 + (epoch - 27) * 160 + blockIdx.x] = now;
        }
        // The release on the add publishes what this block wrote before the barrier (the block-wide
        // barrier above ordered its threads' writes before this thread).
        if (p.withhold_arrival != 0 && epoch == 1 && blockIdx.x == 0) return;
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.barrier) : "memory");
    }
}

__device__ bool grid_wait(const StackParams& p, unsigned epoch, int phase_code) {
    __shared__ int ok_s;
    if (threadIdx.x == 0) {
        const unsigned target = epoch * gridDim.x;
        // The acquire on the load makes the other blocks' writes visible to everything after the barrier.
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
    }
    __syncthreads();
    return ok_s != 0;
}

__device__ bool grid_sync(const StackParams& p, unsigned& epoch, int phase_code) {
    grid_arrive(p, epoch);
    return grid_wait(p, epoch, phase_code);
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

// Asks L2 for this block's slice of a weight matrix (the rows gemm_phase will give it), one request per 128
// bytes.  Only for matrices whose slice does not fit the registers set aside for the next phase's weights (those
// are asked for a phase ahead anyway) and for the head: issuing the requests costs the block about a microsecond
// per 50 KB (measured; bulk prefetches cost more), which is only worth it where the data would otherwise be
// waited for.
__device__ void prefetch_slice(const __nv_bfloat16* __restrict__ W, int N, int K) {
    const int n_groups = (N + 7) / 8;
    const int per_cta = (n_groups + (int)gridDim.x - 1) / (int)gridDim.x;
    const int f0 = min(N, (int)blockIdx.x * per_cta * 8), f1 = min(N, f0 + per_cta * 8);
    const char* base = reinterpret_cast<const char*>(W + (size_t)f0 * K);
    const size_t bytes = (size_t)(f1 - f0) * K * sizeof(__nv_bfloat16);
    for (size_t off = (size_t)threadIdx.x * 128; off < bytes; off += (size_t)kThreads * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16 bytes global -> shared (through L2, not through registers); when `valid` is false nothing is read and the
// destination is filled with zeros.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Rows of a bfloat16 matrix written by other blocks -> shared memory, the tail up to k_pad zeroed.  Every piece is
// an asynchronous copy and all of them are in flight together: one round trip to L2, whatever the row length.
// The caller's block-wide barrier follows.
__device__ void rows_to_smem(const __nv_bfloat16* src, int n_rows, int width, __nv_bfloat16* act_s, int ld, int k_pad) {
    const int chunks = k_pad / 8;
    for (int idx = threadIdx.x; idx < n_rows * chunks; idx += kThreads) {
        const int r = idx / chunks, c = idx - r * chunks;
        const bool valid = c * 8 < width;
        cp_async16(act_s + r * ld + c * 8, src + (size_t)r * width + (valid ? c * 8 : 0), valid);
    }
    cp_async_commit();
    cp_async_wait<0>();
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

// ---- a matrix phase whose weights were asked for before the barrier ----

// This block's feature groups [g_begin, g_begin + ng) of a matrix with N rows, and this warp's k-blocks [kb0, kb1).
struct Slice {
    int g_begin, ng, kb0, kb1;
};

__device__ __forceinline__ Slice slice_of(int N, int K) {
    const int n_groups = (N + 7) / 8;
    const int per_cta = (n_groups + (int)gridDim.x - 1) / (int)gridDim.x;
    const int n_kb = (K + 31) / 32, per_warp = (n_kb + kWarps - 1) / kWarps;
    const int warp = threadIdx.x >> 5;
    Slice sl;
    sl.g_begin = min(n_groups, (int)blockIdx.x * per_cta);
    sl.ng = min(n_groups, sl.g_begin + per_cta) - sl.g_begin;
    sl.kb0 = warp * per_warp;
    sl.kb1 = min(n_kb, sl.kb0 + per_warp);
    return sl;
}

// How a thread's kWRegs pieces are laid out for a matrix: 1 = one group x 16 k-blocks, 2 = two groups x 8, 3 = four
// groups x 4; 0 = the slice does not fit, the phase streams its weights (gemm_phase).  The same for every block.
__device__ __forceinline__ int pick_shape(int N, int K) {
    const int n_groups = (N + 7) / 8;
    const int per_cta = (n_groups + (int)gridDim.x - 1) / (int)gridDim.x;
    const int per_warp = ((K + 31) / 32 + kWarps - 1) / kWarps;
    if (per_cta == 1 && per_warp <= 16) return 1;
    if (per_cta <= 2 && per_warp <= 8) return 2;
    if (per_cta <= 4 && per_warp <= 4) return 3;
    return 0;
}

template <int NG, int KB>
__device__ __forceinline__ void preload_weights(const __nv_bfloat16* __restrict__ W, int N, int K, uint4 (&w)[kWRegs]) {
    static_assert(NG * KB <= kWRegs, "the pieces fit the registers set aside");
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const Slice sl = slice_of(N, K);
#pragma unroll
    for (int gi = 0; gi < NG; ++gi)
#pragma unroll
        for (int u = 0; u < KB; ++u)
            w[gi * KB + u] = (gi < sl.ng && sl.kb0 + u < sl.kb1) ? load_w(W, N, K, (sl.g_begin + gi) * 8 + g, (sl.kb0 + u) * 32 + t * 8)
                                                             : make_uint4(0, 0, 0, 0);
}

__device__ __forceinline__ void preload(int shape, const __nv_bfloat16* __restrict__ W, int N, int K, uint4 (&w)[kWRegs]) {
    if (shape == 1) preload_weights<1, 16>(W, N, K, w);
    else if (shape == 2) preload_weights<2, 8>(W, N, K, w);
    else if (shape == 3) preload_weights<4, 4>(W, N, K, w);
}

// The elements (token r, feature f) that this thread finishes in a phase: element e is number threadIdx.x + 256 e of
// the block's [groups][16 tokens][8 features].  False where there is none.
__device__ __forceinline__ bool post_element(const Slice& sl, int N, int n_tokens, int e, int& r, int& f) {
    const int idx = threadIdx.x + e * kThreads;
    const int gi = idx >> 7;
    r = (idx >> 3) & 15;
    f = (sl.g_begin + gi) * 8 + (idx & 7);
    return gi < sl.ng && r < n_tokens && f < N;
}

template <int NG, int KB, typename Post>
__device__ __forceinline__ void gemm_preloaded(const uint4 (&w)[kWRegs], int N, int K, const __nv_bfloat16* act_s, int ld,
                                               float* red_s, int n_tokens, const float2 (&early)[2], Post post) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const Slice sl = slice_of(N, K);
    const __nv_bfloat16* a_lo = act_s + g * ld + t * 8;
    const __nv_bfloat16* a_hi = a_lo + 8 * ld;
    float acc[NG][4];
#pragma unroll
    for (int i = 0; i < NG; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
#pragma unroll
    for (int u = 0; u < KB; ++u) {
        if (sl.kb0 + u < sl.kb1) {
            const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + (sl.kb0 + u) * 32);
            const uint4 hi = *reinterpret_cast<const uint4*>(a_hi + (sl.kb0 + u) * 32);
#pragma unroll
            for (int gi = 0; gi < NG; ++gi) {
                if (gi < sl.ng) {
                    mma_bf16(acc[gi], lo.x, hi.x, lo.y, hi.y, w[gi * KB + u].x, w[gi * KB + u].y);
                    mma_bf16(acc[gi], lo.z, hi.z, lo.w, hi.w, w[gi * KB + u].z, w[gi * KB + u].w);
                }
            }
        }
    }
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
        if (gi < sl.ng) {
            float* tile = red_s + (warp * kGC + gi) * 128;
            tile[g * 8 + 2 * t] = acc[gi][0];
            tile[g * 8 + 2 * t + 1] = acc[gi][1];
            tile[(g + 8) * 8 + 2 * t] = acc[gi][2];
            tile[(g + 8) * 8 + 2 * t + 1] = acc[gi][3];
        }
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 2; ++e) {                   // at most four groups: 512 elements, two per thread
        int r, f;
        if (post_element(sl, N, n_tokens, e, r, f)) {
            const int idx = threadIdx.x + e * kThreads;
            const int gi = idx >> 7, c = idx & 7;
            float v = 0.0f;
#pragma unroll
            for (int wp = 0; wp < kWarps; ++wp) v += red_s[(wp * kGC + gi) * 128 + r * 8 + c];
            post(r, f, v, early[e]);
        }
    }
    __syncthreads();
}

// One matrix phase: with the weights in `w` (shape 1..3) or streamed (shape 0).  early[e] belongs to post element e.
template <typename Post>
__device__ __forceinline__ void gemm_run(int shape, const uint4 (&w)[kWRegs], const __nv_bfloat16* __restrict__ W, int N, int K,
                                         const __nv_bfloat16* act_s, int ld, float* red_s, int n_tokens,
                                         const float2 (&early)[2], Post post) {
    if (shape == 1) gemm_preloaded<1, 16>(w, N, K, act_s, ld, red_s, n_tokens, early, post);
    else if (shape == 2) gemm_preloaded<2, 8>(w, N, K, act_s, ld, red_s, n_tokens, early, post);
    else if (shape == 3) gemm_preloaded<4, 4>(w, N, K, act_s, ld, red_s, n_tokens, early, post);
}

// ---- bulk copies (TMA, untiled) with an mbarrier, for the head's stream ----

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for the barrier's phase; false when about two seconds passed without it.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
#pragma unroll 1
    for (int i = 0; i < 1024; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > kSpinLimit) return false;
    }
}
// `bytes` (a multiple of 16) from global to shared memory, both 16-byte aligned; completion is counted on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// The head: every warp owns whole groups of eight vocabulary rows (no sum across warps, no block-wide barrier) and
// streams them through its own ring of buffers in shared memory with bulk copies (one per row of a step, issued
// by the warp's first lane, completion counted on the stage's mbarrier).  A step is eight rows x `kc` columns and
// up to four steps (some 20 KB) are in flight per warp: ordinary loads and cp.async keep only about 32 KB per SM
// in flight (measured: 3 TB/s over the GPU, however many were issued), bulk copies are not bound by that.  Rows
// lie 64 bytes (mod 128) apart in a buffer, so the 16-byte fragment reads of a quarter warp meet no bank twice.
// logits[b, f] = sum_k act[b, k] W[f, k] + bias[f].  A wait that runs out records `code` in the status word and
// ends the warp's stream (after waiting, as boundedly, for the copies it still has in flight).
__device__ void head_phase(const __nv_bfloat16* __restrict__ W, const float* __restrict__ bias, int N, int K,
                           const __nv_bfloat16* act_s, int ld, int n_tokens, float* logits, uint8_t* ring, int ring_bytes,
                           uint64_t* bars, int* status, int code) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n_groups = (N + 7) / 8;
    const int per_cta = (n_groups + (int)gridDim.x - 1) / (int)gridDim.x;
    const int g_begin = min(n_groups, (int)blockIdx.x * per_cta), g_end = min(n_groups, g_begin + per_cta);
    const int k_pad = (K + 31) / 32 * 32;
    // A step is eight rows x kc columns (row stride kc * 2 + 64 bytes).  K is cut into the fewest equal chunks of
    // which at least two fit the warp's share of the ring; up to four steps are in flight.
    const int share = ring_bytes / kWarps;
    int n_chunks = 1, kc = k_pad;
    while (2 * 8 * (kc * 2 + 64) > share && kc > 32) {
        ++n_chunks;
        kc = ((k_pad + n_chunks - 1) / n_chunks + 31) / 32 * 32;
    }
    const int stage_bytes = 8 * (kc * 2 + 64);
    const int n_stages = min(4, max(2, share / stage_bytes));
    const int stride = kc + 32;                                          // elements
    const int my_groups = g_end - g_begin > warp ? (g_end - g_begin - warp + kWarps - 1) / kWarps : 0;
    const int total = my_groups * n_chunks;
    __nv_bfloat16* my_ring = reinterpret_cast<__nv_bfloat16*>(ring + (size_t)warp * share);
    uint64_t* my_bars = bars + warp * 4;
    // Columns past K in a buffer are multiplied by zero activations; what they hold must be finite, so where a
    // step is not filled to its last column the ring starts as zeros (bulk copies never touch those columns).
    if (n_chunks * kc != K) {
        uint4* z = reinterpret_cast<uint4*>(my_ring);
        for (int i = lane; i < n_stages * stage_bytes / 16; i += 32) z[i] = make_uint4(0, 0, 0, 0);
    }
    if (lane == 0) {
        for (int i = 0; i < 4; ++i) mbar_init(&my_bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the zeros above, before any bulk copy
    }
    __syncwarp();
    const __nv_bfloat16* a_lo = act_s + g * ld + t * 8;
    const __nv_bfloat16* a_hi = a_lo + 8 * ld;
    // Steps are counted as (group, chunk) and stage by running counters, with no division.
    int f_group = 0, f_chunk = 0, f_stage = 0;                           // the next step to fetch (first lane only)
    auto fetch = [&]() {
        const int gp = g_begin + warp + kWarps * f_group, k0 = f_chunk * kc;
        __nv_bfloat16* dst = my_ring + (size_t)f_stage * (stage_bytes / 2);
        const int rows = min(8, N - gp * 8);
        const uint32_t row_bytes = (uint32_t)(min(kc, K - k0) * 2);
        mbar_expect_tx(&my_bars[f_stage], row_bytes * rows);
        for (int r = 0; r < rows; ++r) bulk_load(dst + r * stride, W + (size_t)(gp * 8 + r) * K + k0, row_bytes, &my_bars[f_stage]);
        if (++f_chunk == n_chunks) { f_chunk = 0; ++f_group; }
        if (++f_stage == n_stages) f_stage = 0;
    };
    float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
    int fetched = 0;
    if (lane == 0)
        for (; fetched < n_stages && fetched < total; ++fetched) fetch();
    int c_group = 0, c_chunk = 0, c_stage = 0;                           // the step being consumed
    uint32_t parity = 0;                                                 // of the ring's current round
    int step = 0;
    for (; step < total; ++step) {
        if (!__all_sync(0xffffffffu, mbar_wait(&my_bars[c_stage], parity))) {      // one answer for the warp
            if (lane == 0) atomicCAS(status, 0, code);
            break;
        }
        const int gp = g_begin + warp + kWarps * c_group, k0 = c_chunk * kc;
        const __nv_bfloat16* src = my_ring + (size_t)c_stage * (stage_bytes / 2) + g * stride + t * 8;
        const int n_kb = min(kc, k_pad - k0) / 32;
#pragma unroll 4
        for (int kb = 0; kb < n_kb; kb += 2) {
            {
                const uint4 w = *reinterpret_cast<const uint4*>(src + kb * 32);
                const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + k0 + kb * 32);
                const uint4 hi = *reinterpret_cast<const uint4*>(a_hi + k0 + kb * 32);
                mma_bf16(acc0, lo.x, hi.x, lo.y, hi.y, w.x, w.y);
                mma_bf16(acc0, lo.z, hi.z, lo.w, hi.w, w.z, w.w);
            }
            if (kb + 1 < n_kb) {
                const uint4 w = *reinterpret_cast<const uint4*>(src + (kb + 1) * 32);
                const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + k0 + (kb + 1) * 32);
                const uint4 hi = *reinterpret_cast<const uint4*>(a_hi + k0 + (kb + 1) * 32);
                mma_bf16(acc1, lo.x, hi.x, lo.y, hi.y, w.x, w.y);
                mma_bf16(acc1, lo.z, hi.z, lo.w, hi.w, w.z, w.w);
            }
        }
        __syncwarp();                       // every lane has read the buffer: the step n_stages further on goes into it
        if (lane == 0 && fetched < total) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            fetch();
            ++fetched;
        }
        if (c_chunk == n_chunks - 1) {
            const int f = gp * 8 + 2 * t;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = g + (e >> 1) * 8, ff = f + (e & 1);
                if (r < n_tokens && ff < N) logits[(size_t)r * N + ff] = acc0[e] + acc1[e] + (bias != nullptr ? __ldg(bias + ff) : 0.0f);
                acc0[e] = acc1[e] = 0.0f;
            }
        }
        if (++c_chunk == n_chunks) { c_chunk = 0; ++c_group; }
        if (++c_stage == n_stages) { c_stage = 0; parity ^= 1; }
    }
    // After a wait that ran out: the copies still in flight land before the block may leave (bounded as well).
    fetched = __shfl_sync(0xffffffffu, fetched, 0);
    for (; step < fetched; ++step) {
        mbar_wait(&my_bars[c_stage], parity);
        if (++c_stage == n_stages) { c_stage = 0; parity ^= 1; }
    }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// Barrier among the `threads` threads of one group of warps (barrier 0 is the block's).
__device__ __forceinline__ void group_barrier(int group, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(threads) : "memory");
}

// Attention of every (token, key/value head) over its pages.  Work items (token, key/value head, key range) go
// round-robin to groups of UW warps (the two halves of every block, or whole blocks).  Within a group, warp w takes
// the 32-key steps w, w + UW, ... of the range through its own ring of S buffers in `ring` (the block's shared
// memory, free during this phase), all S copies in flight at once; the query heads that share the key/value head are the rows of the
// mma.sync tiles.  Formulas and merge order are those of attention_decode_mma.cu.
template <int HD, int S, int UW>
__device__ void attention_phase(const StackParams& p, const StackLayer& L, uint8_t* ring, const int32_t* pos_s) {
    static_assert(UW == 4 || UW == 8, "a work item is served by four or by all eight warps of a block");
    constexpr int kUnits = kWarps / UW, kUnitThreads = UW * 32;
    // A warp's step is 32 keys, two 16-key tiles (each inside one page): with only eight warps on the SM a warp's
    // chain of dependent instructions sets the pace, and it is as long for 32 keys as for 16.
    constexpr int kStep = 32, kTile = 16, CH = HD / 8, KS = HD / 16, OT = HD / 8, STATE = HD + 2;
    constexpr int kTileElems = kTile * HD;                         // one 16-key tile of keys (or of values)
    constexpr int kStageElems = 4 * kTileElems;                    // [tile 0: K, V][tile 1: K, V]
    __shared__ int last_s[2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int group = warp / UW, gw = warp % UW, gt = threadIdx.x % kUnitThreads;
    const int B = p.n_tokens, H = L.n_head, n_kv = L.n_kv_head, G = H / n_kv, splits = p.n_splits;
    const int qd = H * HD, page_size = 1 << p.page_shift;
    const size_t plane = (size_t)n_kv * page_size * HD;
    __nv_bfloat16* group_ring = reinterpret_cast<__nv_bfloat16*>(ring) + (size_t)group * UW * S * kStageElems;
    __nv_bfloat16* my_ring = group_ring + (size_t)gw * S * kStageElems;
    float* red = reinterpret_cast<float*>(group_ring);             // the group's states, over its ring, after the key loop
    const float sc = L.scale * kLog2e;
    const int n_items = B * n_kv * splits, n_units = kUnits * (int)gridDim.x;
    for (int item = (int)blockIdx.x * kUnits + group; item < n_items; item += n_units) {
        const int split = item % splits, pair = item / splits, kvh = pair % n_kv, b = pair / n_kv;
        const int pos = pos_s[b];
        const int first = L.window > 0 ? max(0, pos - L.window + 1) : 0;
        const int n_keys = pos + 1 - first;
        const int chunk = (n_keys + splits - 1) / splits;
        const int begin = first + split * chunk, end = min(pos + 1, begin + chunk);
        const int32_t* table = p.block_table + (size_t)b * p.table_stride;
        const int tile0 = begin / kStep;
        const int n_tiles = end > begin ? (end - 1) / kStep + 1 - tile0 : 0;
        const int my_tiles = n_tiles > gw ? (n_tiles - gw + UW - 1) / UW : 0;
        // Q as the A operand: row r = query head kvh * G + r (rows past G are zero).  Written by other blocks in the
        // phase before: read through L2.
        uint32_t qf[KS][4];
        {
            const uint32_t* q_seq = reinterpret_cast<const uint32_t*>(p.q + (size_t)b * qd + (size_t)kvh * G * HD);
#pragma unroll
            for (int kk = 0; kk < KS; ++kk) {
                const int c = (kk * 16 + 2 * t) / 2;
                qf[kk][0] = g < G ? __ldcg(q_seq + (g * HD) / 2 + c) : 0u;
                qf[kk][1] = g + 8 < G ? __ldcg(q_seq + ((g + 8) * HD) / 2 + c) : 0u;
                qf[kk][2] = g < G ? __ldcg(q_seq + (g * HD) / 2 + c + 4) : 0u;
                qf[kk][3] = g + 8 < G ? __ldcg(q_seq + ((g + 8) * HD) / 2 + c + 4) : 0u;
            }
        }
        stamp(p, 1100);
        // This warp's i-th step (keys (tile0 + gw + UW i) * 32 ...) -> stage.  Rows outside [begin, end) are not read
        // and arrive as zeros.  16-byte chunk c of row r lies at chunk c ^ (r & 7): ldmatrix meets no bank twice.
        auto load_tile = [&](int i, int stage) {
            const int j_step = (tile0 + gw + UW * i) * kStep;
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                const int j0 = j_step + sub * kTile;
                const bool any = j0 < end && j0 + kTile > begin;
                const int page = any ? __ldg(table + (j0 >> p.page_shift)) : 0;
                const __nv_bfloat16* src = L.cache + (size_t)page * 2 * plane + ((size_t)kvh * page_size + (j0 & (page_size - 1))) * HD;
                __nv_bfloat16* kd = my_ring + (size_t)stage * kStageElems + (size_t)sub * 2 * kTileElems;
                __nv_bfloat16* vd = kd + kTileElems;
#pragma unroll
                for (int c = lane; c < kTile * CH; c += 32) {
                    const int r = c / CH, ch = c - r * CH;
                    const bool valid = j0 + r >= begin && j0 + r < end;
                    const int at = r * HD + ((ch ^ (r & 7)) << 3);
                    cp_async16(kd + at, src + r * HD + ch * 8, valid);
                    cp_async16(vd + at, src + plane + r * HD + ch * 8, valid);
                }
            }
        };
        float o[OT][4];
#pragma unroll
        for (int i = 0; i < OT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
        float m_lo = -CUDART_INF_F, m_hi = -CUDART_INF_F, l_lo = 0.0f, l_hi = 0.0f;
#pragma unroll
        for (int i = 0; i < S; ++i) {
            if (i < my_tiles) load_tile(i, i);
            cp_async_commit();
        }
        for (int i = 0; i < my_tiles; ++i) {
            const int stage = i % S;
            cp_async_wait<S - 1>();
            __syncwarp();
            const __nv_bfloat16* st_base = my_ring + (size_t)stage * kStageElems;
            const int j_step = (tile0 + gw + UW * i) * kStep;
            float s[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
            const int mat = lane >> 3, r8 = lane & 7;
#pragma unroll
            for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    const __nv_bfloat16* kt = st_base + (size_t)sub * 2 * kTileElems;
                    uint32_t bf[4];
                    ldmatrix_x4(bf, smem_addr(kt + ((mat >> 1) * 8 + r8) * HD + (((kk * 2 + (mat & 1)) ^ r8) << 3)));
                    mma_bf16(s[2 * sub], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], bf[0], bf[1]);
                    mma_bf16(s[2 * sub + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], bf[2], bf[3]);
                }
            }
            float mx_lo = -CUDART_INF_F, mx_hi = -CUDART_INF_F;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = j_step + nt * 8 + 2 * t + (e & 1);
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
            uint32_t pf[2][4];
            float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const float p0 = exp2f(s[nt][0] - base_lo), p1 = exp2f(s[nt][1] - base_lo);
                const float p2 = exp2f(s[nt][2] - base_hi), p3 = exp2f(s[nt][3] - base_hi);
                sum_lo += p0 + p1;
                sum_hi += p2 + p3;
                pf[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            l_lo = l_lo * corr_lo + sum_lo;          // per-thread partial sums; the quad is summed once at the end
            l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
            for (int ot = 0; ot < OT; ++ot) {
                o[ot][0] *= corr_lo; o[ot][1] *= corr_lo; o[ot][2] *= corr_hi; o[ot][3] *= corr_hi;
            }
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                const __nv_bfloat16* vt = st_base + (size_t)sub * 2 * kTileElems + kTileElems;
#pragma unroll
                for (int ot = 0; ot < OT; ot += 2) {
                    uint32_t bf[4];
                    ldmatrix_x4_trans(bf, smem_addr(vt + ((mat & 1) * 8 + r8) * HD + (((ot + (mat >> 1)) ^ r8) << 3)));
                    mma_bf16(o[ot], pf[sub][0], pf[sub][1], pf[sub][2], pf[sub][3], bf[0], bf[1]);
                    mma_bf16(o[ot + 1], pf[sub][0], pf[sub][1], pf[sub][2], pf[sub][3], bf[2], bf[3]);
                }
            }
            __syncwarp();        // the stage is free: the step S further on goes into it
            if (i + S < my_tiles) load_tile(i + S, stage);
            cp_async_commit();
        }
        cp_async_wait<0>();
        stamp(p, 1101);
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
        // The warps' states of every valid row -> shared memory (over the group's ring) -> merged in warp order.
        group_barrier(group, kUnitThreads);
        if (g < G) {
            float* st = red + (size_t)(gw * 16 + g) * STATE;
            if (t == 0) { st[0] = m_lo; st[1] = l_lo; }
#pragma unroll
            for (int ot = 0; ot < OT; ++ot) { st[2 + ot * 8 + 2 * t] = o[ot][0]; st[2 + ot * 8 + 2 * t + 1] = o[ot][1]; }
        }
        if (g + 8 < G) {
            float* st = red + (size_t)(gw * 16 + g + 8) * STATE;
            if (t == 0) { st[0] = m_hi; st[1] = l_hi; }
#pragma unroll
            for (int ot = 0; ot < OT; ++ot) { st[2 + ot * 8 + 2 * t] = o[ot][2]; st[2 + ot * 8 + 2 * t + 1] = o[ot][3]; }
        }
        group_barrier(group, kUnitThreads);
        float* my_partial = p.partial + ((size_t)pair * splits + split) * (size_t)(G * STATE);
        for (int idx = gt; idx < G * HD; idx += kUnitThreads) {
            const int r = idx / HD, d = idx - r * HD;
            float mm = -CUDART_INF_F;
#pragma unroll
            for (int w = 0; w < UW; ++w) mm = fmaxf(mm, red[(size_t)(w * 16 + r) * STATE]);
            float ll = 0.0f, a = 0.0f;
#pragma unroll
            for (int w = 0; w < UW; ++w) {
                const float* st = red + (size_t)(w * 16 + r) * STATE;
                const float f = mm == -CUDART_INF_F ? 0.0f : exp2f(st[0] - mm);
                ll += st[1] * f;
                a += st[2 + d] * f;
            }
            if (splits == 1) {
                p.att[(size_t)b * qd + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(a / ll);
            } else {
                my_partial[r * STATE + 2 + d] = a;
                if (d == 0) {
                    my_partial[r * STATE] = mm;
                    my_partial[r * STATE + 1] = ll;
                }
            }
        }
        if (splits > 1) {
            __threadfence();
            group_barrier(group, kUnitThreads);
            if (gt == 0) {
                const int done = atomicAdd(&p.counters[pair], 1);
                last_s[group] = done == splits - 1;
                if (done == splits - 1) p.counters[pair] = 0;      // ready for the next layer
            }
            group_barrier(group, kUnitThreads);
            if (last_s[group]) {
                __threadfence();
                const float* all = p.partial + (size_t)pair * splits * (size_t)(G * STATE);
                for (int idx = gt; idx < G * HD; idx += kUnitThreads) {
                    const int r = idx / HD, d = idx - r * HD;
                    float mm = -CUDART_INF_F;
#pragma unroll 4
                    for (int sp = 0; sp < splits; ++sp) mm = fmaxf(mm, __ldcg(all + (size_t)sp * G * STATE + r * STATE));
                    float ll = 0.0f, a = 0.0f;
#pragma unroll 4
                    for (int sp = 0; sp < splits; ++sp) {
                        const float* st = all + (size_t)sp * G * STATE + r * STATE;
                        const float f = exp2f(__ldcg(st) - mm);        // an empty range has m = -inf: factor 0
                        ll += __ldcg(st + 1) * f;
                        a += __ldcg(st + 2 + d) * f;
                    }
                    p.att[(size_t)b * qd + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(a / ll);
                }
            }
        }
        group_barrier(group, kUnitThreads);        // the ring (and the states over it) are free for the group's next item
    }
}

__global__ void __launch_bounds__(kThreads, 1) decode_stack_kernel(const StackParams p) {
    extern __shared__ __align__(16) uint8_t smem_bytes[];
    __nv_bfloat16* act_s = reinterpret_cast<__nv_bfloat16*>(smem_bytes);
    float* red_s = reinterpret_cast<float*>(smem_bytes + (size_t)kMaxTokens * p.act_ld * sizeof(__nv_bfloat16));
    int32_t* pos_s = reinterpret_cast<int32_t*>(smem_bytes + p.pos_offset);        // [kMaxTokens] positions
    const StackLayer* layers_s = reinterpret_cast<const StackLayer*>(pos_s + kMaxTokens);   // every layer's record
    const int B = p.n_tokens, d = p.width, ld = p.act_ld;
    unsigned epoch = 0;
    if (p.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        p.timing[0] = now;
    }
    for (int i = threadIdx.x; i < B; i += kThreads) pos_s[i] = p.positions[i];
    if (blockIdx.x == 0 && threadIdx.x == 0) *p.other_barrier = 0u;
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.layers);
        uint4* dst = reinterpret_cast<uint4*>(pos_s + kMaxTokens);
        for (int i = threadIdx.x; i < p.n_layers * (int)(sizeof(StackLayer) / 16); i += kThreads) dst[i] = src[i];
    }
    __syncthreads();

    uint4 wreg[kWRegs];              // this thread's pieces of the next matrix phase's weights
    float2 early[2];                 // what belongs to its two post elements: .x before the barrier (bias), .y after
    early[0] = early[1] = make_float2(0.f, 0.f);
    int shape = 0;
    if (p.n_layers > 0) {
        const StackLayer& L0 = layers_s[0];
        const int qkv_n = (L0.n_head + 2 * L0.n_kv_head) * L0.head_dim;
        shape = pick_shape(qkv_n, d);
        if (shape == 0) prefetch_slice(L0.w_qkv, qkv_n, d);
        if (pick_shape(d, L0.n_head * L0.head_dim) == 0) prefetch_slice(L0.w_out, d, L0.n_head * L0.head_dim);
        preload(shape, L0.w_qkv, qkv_n, d, wreg);
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
        const StackLayer& L = layers_s[li];
        const int hd = L.head_dim, qd = L.n_head * hd, kvd = L.n_kv_head * hd, page_size = 1 << p.page_shift;
        const size_t plane = (size_t)L.n_kv_head * page_size * hd;
        const int code = (li + 1) << 4;
        const int qkv_n = qd + 2 * kvd;
        // Weights held in registers across the attention phase would push its wider head size over the register file.
        const bool hold_over_attention = hd == 64;

        // ---- LayerNorm 1, fused projection, keys and values into their pages (weights: asked for before the barrier).
        stamp(p, 128 + li * 8 + 4);
        {
            const Slice sl = slice_of(qkv_n, d);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                int r, f;
                early[e] = post_element(sl, qkv_n, B, e, r, f)
                               ? make_float2(L.b_qkv != nullptr ? __ldg(L.b_qkv + f) : 0.0f, __int_as_float(f >= qd ? __ldg(p.slot_mapping + r) : 0))
                               : make_float2(0.f, 0.f);
            }
        }
        stamp(p, 128 + li * 8 + 5);
        layernorm_to_smem(p.x, L.ln1_w, L.ln1_b, L.ln1_eps, B, d, act_s, ld, (d + 63) / 64 * 64);
        __syncthreads();
        stamp(p, 128 + li * 8 + 0);
        {
            auto post = [&](int b, int f, float v, float2 e) {
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
            };
            if (shape != 0) {
                gemm_run(shape, wreg, L.w_qkv, qkv_n, d, act_s, ld, red_s, B, early, post);
            } else {
                gemm_phase(L.w_qkv, qkv_n, d, act_s, ld, red_s, B, [&](int b, int f) {
                    return make_float2(L.b_qkv != nullptr ? __ldg(L.b_qkv + f) : 0.0f, __int_as_float(f >= qd ? __ldg(p.slot_mapping + b) : 0));
                }, post);
            }
        }
        stamp(p, 128 + li * 8 + 1);
        grid_arrive(p, epoch);
        shape = pick_shape(d, qd);
        if (hold_over_attention) preload(shape, L.w_out, d, qd, wreg);
        if (pick_shape(L.inner, d) == 0) prefetch_slice(L.w_up, L.inner, d);
        if (pick_shape(d, L.inner) == 0) prefetch_slice(L.w_down, d, L.inner);
        if (!grid_wait(p, epoch, code | 1)) return;

        // ---- Attention.
        if (hd == 64) {
            if (p.unit_warps == 8) attention_phase<64, 2, 8>(p, L, smem_bytes, pos_s);
            else attention_phase<64, 2, 4>(p, L, smem_bytes, pos_s);
        } else {
            if (p.unit_warps == 8) attention_phase<128, 1, 8>(p, L, smem_bytes, pos_s);
            else attention_phase<128, 1, 4>(p, L, smem_bytes, pos_s);
        }
        stamp(p, 128 + li * 8 + 2);
        if (!grid_sync(p, epoch, code | 2)) return;

        // ---- Output projection + residual.
        if (!hold_over_attention) preload(shape, L.w_out, d, qd, wreg);
        {
            const Slice sl = slice_of(d, qd);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                int r, f;
                early[e] = post_element(sl, d, B, e, r, f)
                               ? make_float2(L.b_out != nullptr ? __ldg(L.b_out + f) : 0.0f, __ldcg(p.x + (size_t)r * d + f))
                               : make_float2(0.f, 0.f);
            }
        }
        rows_to_smem(p.att, B, qd, act_s, ld, (qd + 63) / 64 * 64);
        __syncthreads();
        stamp(p, 128 + li * 8 + 6);
        {
            auto post = [&](int b, int f, float v, float2 e) { p.x[(size_t)b * d + f] = e.y + (v + e.x); };
            if (shape != 0) {
                gemm_run(shape, wreg, L.w_out, d, qd, act_s, ld, red_s, B, early, post);
            } else {
                gemm_phase(L.w_out, d, qd, act_s, ld, red_s, B, [&](int b, int f) {
                    return make_float2(L.b_out != nullptr ? __ldg(L.b_out + f) : 0.0f, __ldcg(p.x + (size_t)b * d + f));
                }, post);
            }
        }
        stamp(p, 128 + li * 8 + 3);
        grid_arrive(p, epoch);
        shape = pick_shape(L.inner, d);
        preload(shape, L.w_up, L.inner, d, wreg);
        if (li + 1 < p.n_layers) {
            const StackLayer& Ln = layers_s[li + 1];
            const int next_n = (Ln.n_head + 2 * Ln.n_kv_head) * Ln.head_dim, next_qd = Ln.n_head * Ln.head_dim;
            if (pick_shape(next_n, d) == 0) prefetch_slice(Ln.w_qkv, next_n, d);
            if (pick_shape(d, next_qd) == 0) prefetch_slice(Ln.w_out, d, next_qd);
        } else {
            if (p.timing == nullptr || p.timing[2040] == 0) prefetch_slice(p.head_w, p.vocab, d);
        }
        if (!grid_wait(p, epoch, code | 3)) return;

        // ---- LayerNorm 2, up projection, activation.
        {
            const Slice sl = slice_of(L.inner, d);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                int r, f;
                early[e] = post_element(sl, L.inner, B, e, r, f) ? make_float2(L.b_up != nullptr ? __ldg(L.b_up + f) : 0.0f, 0.0f)
                                                                 : make_float2(0.f, 0.f);
            }
        }
        layernorm_to_smem(p.x, L.ln2_w, L.ln2_b, L.ln2_eps, B, d, act_s, ld, (d + 63) / 64 * 64);
        __syncthreads();
        {
            auto post = [&](int b, int f, float v, float2 e) {
                p.inner[(size_t)b * L.inner + f] = __float2bfloat16_rn(lb_activate(v + e.x, L.act));
            };
            if (shape != 0) {
                gemm_run(shape, wreg, L.w_up, L.inner, d, act_s, ld, red_s, B, early, post);
            } else {
                gemm_phase(L.w_up, L.inner, d, act_s, ld, red_s, B, [&](int b, int f) {
                    return make_float2(L.b_up != nullptr ? __ldg(L.b_up + f) : 0.0f, 0.0f);
                }, post);
            }
        }
        grid_arrive(p, epoch);
        shape = pick_shape(d, L.inner);
        preload(shape, L.w_down, d, L.inner, wreg);
        if (!grid_wait(p, epoch, code | 4)) return;

        // ---- Down projection + residual.
        {
            const Slice sl = slice_of(d, L.inner);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                int r, f;
                early[e] = post_element(sl, d, B, e, r, f)
                               ? make_float2(L.b_down != nullptr ? __ldg(L.b_down + f) : 0.0f, __ldcg(p.x + (size_t)r * d + f))
                               : make_float2(0.f, 0.f);
            }
        }
        rows_to_smem(p.inner, B, L.inner, act_s, ld, (L.inner + 63) / 64 * 64);
        __syncthreads();
        {
            auto post = [&](int b, int f, float v, float2 e) { p.x[(size_t)b * d + f] = e.y + (v + e.x); };
            if (shape != 0) {
                gemm_run(shape, wreg, L.w_down, d, L.inner, act_s, ld, red_s, B, early, post);
            } else {
                gemm_phase(L.w_down, d, L.inner, act_s, ld, red_s, B, [&](int b, int f) {
                    return make_float2(L.b_down != nullptr ? __ldg(L.b_down + f) : 0.0f, __ldcg(p.x + (size_t)b * d + f));
                }, post);
            }
        }
        grid_arrive(p, epoch);
        if (li + 1 < p.n_layers) {
            const StackLayer& Ln = layers_s[li + 1];
            const int next_n = (Ln.n_head + 2 * Ln.n_kv_head) * Ln.head_dim;
            shape = pick_shape(next_n, d);
            preload(shape, Ln.w_qkv, next_n, d, wreg);
        }
        if (!grid_wait(p, epoch, code | 5)) return;
    }

    // ---- Final norm and the head.
    const int ld_head = (d + 63) / 64 * 64 + 32;          // the head's activations lie compactly: the rest is its ring
    layernorm_to_smem(p.x, p.lnf_w, p.lnf_b, p.lnf_eps, B, d, act_s, ld_head, (d + 63) / 64 * 64);
    __syncthreads();
    stamp(p, 126);
    head_phase(p.head_w, p.head_b, p.vocab, d, act_s, ld_head, B, p.logits, smem_bytes + p.head_ring_offset, p.head_ring_bytes,
               reinterpret_cast<uint64_t*>(smem_bytes + p.bars_offset), p.status, 0xF0);
    stamp(p, 127);
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
                               int head_dim, int n_splits, int unit_warps, unsigned long long* timing, void* stream) {
    LB_CHECK_ARG(n_layers >= 0 && n_tokens >= 1 && n_tokens <= kMaxTokens, "decode stack: %d tokens (1..%d are taken)", n_tokens,
                 kMaxTokens);
    LB_CHECK_ARG(width > 0 && width % 8 == 0 && max_k >= width && max_k % 8 == 0 && vocab > 0,
                 "decode stack: width %d and the largest reduction length %d must be multiples of 8", width, max_k);
    LB_CHECK_ARG(head_dim == 64 || head_dim == 128, "decode stack: head_dim %d (64 and 128 are taken)", head_dim);
    LB_CHECK_ARG(page_size >= 16 && (page_size & (page_size - 1)) == 0, "decode stack: page_size %d (a power of two, 16 or more)", page_size);
    LB_CHECK_ARG(n_splits >= 1 && n_splits <= 64, "decode stack: n_splits %d", n_splits);
    LB_CHECK_ARG(unit_warps == 4 || unit_warps == 8, "decode stack: unit_warps %d (4 or 8)", unit_warps);
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
    // `barrier` points at one of a pair of counters (8-byte aligned pair, both zero at first) and the caller
    // alternates between the two from launch to launch: a launch zeroes the other one (its only other user, the
    // launch before, has ended), so the step needs no memset of its own.
    p.barrier = barrier;
    p.other_barrier = reinterpret_cast<unsigned*>(reinterpret_cast<uintptr_t>(barrier) ^ (uintptr_t)4);
    int* status = nullptr;
    LB_CHECK_CUDA(cudaGetSymbolAddress((void**)&status, g_stack_status));
    p.status = status;
    p.n_splits = n_splits;
    p.unit_warps = unit_warps;
    p.timing = timing;
    p.withhold_arrival = g_withhold_next;
    g_withhold_next = 0;
    p.act_ld = (max_k + 63) / 64 * 64 + 32;       // row stride = 64 bytes mod 128: conflict-free 16-byte reads
    // Shared memory: the matrix phases' activations and partial tiles, or the attention phase's tile rings
    // (8 warps x S stages x K and V tiles of 16 keys), whichever is larger; then the positions.
    const size_t gemm_bytes = (size_t)kMaxTokens * p.act_ld * sizeof(__nv_bfloat16) + (size_t)kWarps * kGC * 128 * sizeof(float);
    const size_t ring_bytes = (size_t)kWarps * (head_dim == 64 ? 2 : 1) * 4 * 16 * head_dim * sizeof(__nv_bfloat16);
    // The head's ring follows the head's (compactly laid out) activations and takes what is left of 200 KB.
    const size_t head_act = ((size_t)kMaxTokens * ((width + 63) / 64 * 64 + 32) * sizeof(__nv_bfloat16) + 127) / 128 * 128;
    size_t head_ring = 200 * 1024 - head_act;
    head_ring = head_ring / (kWarps * 16) * (kWarps * 16);
    const size_t act_bytes = head_act;
    p.head_ring_offset = (int)head_act;
    p.head_ring_bytes = (int)head_ring;
    size_t most = gemm_bytes > ring_bytes ? gemm_bytes : ring_bytes;
    if (act_bytes + head_ring > most) most = act_bytes + head_ring;
    const size_t shared_bytes = (most + 15) / 16 * 16;
    p.pos_offset = (int)shared_bytes;
    const size_t after_layers = shared_bytes + (size_t)kMaxTokens * sizeof(int32_t) + (size_t)n_layers * sizeof(StackLayer);
    p.bars_offset = (int)((after_layers + 15) / 16 * 16);
    const size_t smem = (size_t)p.bars_offset + kWarps * 4 * sizeof(uint64_t);
    LB_CHECK_ARG(smem <= 227 * 1024, "decode stack: a reduction length of %d needs %zu bytes of shared memory, the SM has 232448",
                 max_k, smem);
    static size_t configured = 0;
    if (smem > configured) {
        LB_CHECK_CUDA(cudaFuncSetAttribute(decode_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
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

// The same word without a device synchronisation: copies it into `host` (pinned memory) on `stream`;
// lb_decode_stack_status_clear zeroes it on `stream`.
extern "C" int lb_decode_stack_status_async(int* host, void* stream) {
    int* word = nullptr;
    LB_CHECK_CUDA(cudaGetSymbolAddress((void**)&word, g_stack_status));
    LB_CHECK_CUDA(cudaMemcpyAsync(host, word, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    return LB_OK;
}

extern "C" int lb_decode_stack_status_clear(void* stream) {
    int* word = nullptr;
    LB_CHECK_CUDA(cudaGetSymbolAddress((void**)&word, g_stack_status));
    LB_CHECK_CUDA(cudaMemsetAsync(word, 0, sizeof(int), static_cast<cudaStream_t>(stream)));
    return LB_OK;
}

// The next launch's first grid barrier is one arrival short, so every block's wait runs to its limit (about
// two seconds), reports it in the status word and returns: a test of the give-up path that faults nothing.
extern "C" int lb_decode_stack_withhold_next(int on) {
    g_withhold_next = on != 0 ? 1 : 0;
    return LB_OK;
}

// Writes the word (tests of the host's handling of a reported barrier; synchronises).
extern "C" int lb_decode_stack_status_set(int value) {
    LB_CHECK_CUDA(cudaMemcpyToSymbol(g_stack_status, &value, sizeof(int)));
    return LB_OK;
}
