// Next-token choice on the device: greedy, or temperature -> top-k -> top-p ->
// draw, one thread block per row of logits, each row with its own options.
//
// The distribution is the reference sampler's (src/core/sampling.cpp:16-61):
// keep the top_k largest logits, p_i = exp((l_i - l_max) / T) in float, total in
// double, keep the shortest prefix of the candidates sorted by logit whose
// cumulative p_i / total reaches top_p, renormalise by the kept mass; then walk
// the ids in index order subtracting p_i from r = u * total until r < 0
// (sampling.cpp:66-79).  Greedy takes the first maximum (sampling.cpp:12-14).
// Where the reference's order among equal logits is left to std::nth_element and
// std::sort, ties here go to the lower index.  In general nothing is sorted: the
// k-th largest logit and the top-p cut are found by radix selection over the
// logits' bit patterns (four passes of eight bits), by count for top-k and by
// probability mass for top-p.  A top-k of up to 256 (the usual case: 40) takes a
// short way instead: a threshold that at least k logits reach comes from the
// block's 1,024 per-thread maxima (radix selection among them), the few logits
// that reach it are listed in shared memory and the rest happens among them
// (16 us instead of 94 us per step at a vocabulary of 50,257; one block per row
// walks the row twice).  Top-p without top-k takes the same way with the 256
// largest logits as candidates whenever they hold the asked share of the whole
// row's mass (34 us instead of 320 us), and the general path otherwise (whose
// histograms are built by warps that add their lanes' terms first, in fixed point,
// and read by one warp in parallel).
#include "api.h"
#include "common.cuh"

#include <math_constants.h>

namespace {

constexpr int kThreads = 1024;
constexpr int kSmallK = 256;       // a top-k up to this takes the short way: a threshold, then a list of candidates
constexpr int kMaxList = 1024;     // candidates (logits that reach the threshold) the short way takes
// The general path's histograms of probability mass are sums of exp((l - max) / T) <= 1 in fixed point (the unit is
// 2^-(62 - floor(log2 vocab)), at most 2^-47: a row of ones still fits 64 bits, and what a term loses is far below the
// float probabilities' own rounding).  Thousands of logits share a few buckets (sign and exponent), so the lanes of a
// warp that meet in a bucket add their terms first (three 16-bit limbs through the warp's integer reduction) and one
// of them adds the sum to shared memory; integer sums do not depend on the order of the additions.

// Monotone map from float to uint32: a larger float gives a larger key.
__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct ArgMax {
    float v;
    int i;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ ArgMax block_argmax(ArgMax a, ArgMax* scratch /* 33 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
        a = better(a, b);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = a;
    __syncthreads();
    if (warp == 0) {
        ArgMax t = lane < (int)(blockDim.x >> 5) ? scratch[lane] : ArgMax{-CUDART_INF_F, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax b{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
            t = better(t, b);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Exclusive prefix sum of one value per thread, in thread order; returns the
// block total through *total.  T is int or double.
template <typename T>
__device__ T block_exclusive_scan(T v, T* scratch /* 33 */, T* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    T inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T up = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += up;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        T w = lane < n_warps ? scratch[lane] : T(0);
        T winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const T up = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += up;
        }
        scratch[lane] = winc - w;           // exclusive offset of each warp
        if (lane == 31) scratch[32] = winc;  // block total
    }
    __syncthreads();
    *total = scratch[32];
    return scratch[warp] + inc - v;
}

// Sums over a short array in shared memory by one warp: every lane adds its run of consecutive elements in order, the
// lanes' sums are scanned in lane order.  Returns the lane's offset (the sum of everything before its run) and the
// total through *total; `value(i)` gives element i as a double.  The order of the additions is fixed.
template <typename F>
__device__ __forceinline__ double warp_ordered_offsets(int n, F value, double* mine, double* total, int* first, int* last) {
    const int lane = threadIdx.x & 31, per = (n + 31) / 32;
    const int a = min(n, lane * per), b = min(n, a + per);
    double s = 0.0;
    for (int i = a; i < b; ++i) s += value(i);
    double inc = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += up;
    }
    *mine = s;
    *total = __shfl_sync(0xffffffffu, inc, 31);
    *first = a;
    *last = b;
    return inc - s;
}

// One warp finds, from the top bucket down, the bucket that holds the `remaining`-th largest key of a 256-bucket
// histogram of counts, and the rank that is left inside it (lane l holds buckets 255 - 8 l down to 248 - 8 l; the
// lanes' sums are scanned).  The histogram holds at least `remaining` keys.  The answer is the same on every lane.
__device__ __forceinline__ void warp_bucket_by_count(const int* hist, int remaining, int* digit_out, int* rem_out) {
    const int lane = threadIdx.x & 31;
    int c[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        c[j] = hist[255 - 8 * lane - j];
        sum += c[j];
    }
    int inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += up;
    }
    const unsigned reached = __ballot_sync(0xffffffffu, inc >= remaining);
    const int owner = reached != 0u ? __ffs(reached) - 1 : 31;
    int rem = remaining - (inc - sum), digit = 255 - 8 * lane;
#pragma unroll
    for (int j = 0; j < 7; ++j) {
        if (rem > c[j] && digit == 255 - 8 * lane - j) {
            rem -= c[j];
            --digit;
        }
    }
    *digit_out = __shfl_sync(0xffffffffu, digit, owner);
    *rem_out = __shfl_sync(0xffffffffu, rem, owner);
}

// The same by probability mass (fixed point, `unit` per 1.0): the highest bucket at which the mass from the top,
// `above` included, reaches the share p_cut of total_mass; bucket 0 if none does.  *above_out: the mass above it.
__device__ __forceinline__ void warp_bucket_by_mass(const unsigned long long* hist, unsigned long long above, double unit,
                                                    double total_mass, double p_cut, int* digit_out, unsigned long long* above_out) {
    const int lane = threadIdx.x & 31;
    unsigned long long c[8], sum = 0ull;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        c[j] = hist[255 - 8 * lane - j];
        sum += c[j];
    }
    unsigned long long inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += up;
    }
    unsigned long long before = above + (inc - sum);          // mass above this lane's first bucket
    int digit = -1;
    unsigned long long before_hit = 0ull;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = 255 - 8 * lane - j;
        if (digit < 0 && d > 0 && ((double)(before + c[j]) / unit) / total_mass >= p_cut) {
            digit = d;
            before_hit = before;
        }
        before += c[j];
    }
    const unsigned hit = __ballot_sync(0xffffffffu, digit >= 0);
    if (hit != 0u) {
        const int owner = __ffs(hit) - 1;
        *digit_out = __shfl_sync(0xffffffffu, digit, owner);
        *above_out = __shfl_sync(0xffffffffu, before_hit, owner);
    } else {
        // No bucket reaches the share: the lowest takes what is left (the last lane's `before` stops short of bucket 0).
        const unsigned long long all = __shfl_sync(0xffffffffu, inc, 31);
        const unsigned long long lowest = __shfl_sync(0xffffffffu, c[7], 31);
        *digit_out = 0;
        *above_out = above + all - lowest;
    }
}

// The n-th largest of the block's keys (one per thread, n >= 1 and at most the block's size), to its upper 24 bits:
// a value that at least n of the keys reach.  Radix selection, eight bits a pass; a pass is a histogram in shared
// memory (lanes with the same bucket add once, together) and one warp that finds the bucket of the n-th largest.
__device__ uint32_t nth_largest_floor(uint32_t key, int n, int* hist /* 256 */, uint32_t* sh_prefix, int* sh_remaining) {
    const int tid = threadIdx.x, lane = tid & 31;
    uint32_t prefix = 0;
    int remaining = n;
    for (int shift = 24; shift >= 8; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        const int bucket = (key & mask) == prefix ? (int)((key >> shift) & 255u) : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, bucket);
        if (bucket >= 0 && lane == __ffs(peers) - 1) atomicAdd(&hist[bucket], __popc(peers));
        __syncthreads();
        if (tid < 32) {
            int digit, rem;
            warp_bucket_by_count(hist, remaining, &digit, &rem);
            if (tid == 0) {
                *sh_prefix = prefix | ((uint32_t)digit << shift);
                *sh_remaining = rem;
            }
        }
        __syncthreads();
        prefix = *sh_prefix;
        remaining = *sh_remaining;
    }
    return prefix;
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int64_t row_stride, int vocab, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const float* __restrict__ top_p, const double* __restrict__ uniform,
              int32_t* __restrict__ out_ids, float* __restrict__ out_probs) {
    __shared__ ArgMax am_scratch[33];
    __shared__ int i_scratch[33];
    __shared__ double d_scratch[33];
    __shared__ int hist_count[256];
    __shared__ unsigned long long hist_mass[256];      // masses in fixed point (kMassUnit), so that their sums do not depend on the order
    __shared__ uint32_t sh_prefix;
    __shared__ int sh_int;
    __shared__ double sh_double;
    __shared__ int sh_choice;

    lb_wait_for_predecessor();
    lb_dependents_may_launch();
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * row_stride;
    float* probs = out_probs != nullptr ? out_probs + (size_t)row * vocab : nullptr;
    const float temp = temperature[row];

    // Contiguous range of this thread: sums and ranks in index order need one scan.  The first thread takes the
    // (up to three) logits before the row's first 16-byte boundary, the others a multiple of four from there on, so
    // that they read with 16-byte loads (the lanes of a warp read 32 different lines whatever the width of a load:
    // four times fewer loads, four times fewer trips through the first-level cache).
    const int peel = (int)((4 - ((reinterpret_cast<uintptr_t>(x) >> 2) & 3)) & 3);
    const int per = ((vocab + kThreads - 2) / (kThreads - 1) + 3) & ~3;
    const int lo = min(vocab, max(0, (tid - 1) * per + peel)), hi = min(vocab, max(0, tid * per + peel));
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x + lo) & 15) == 0;
    auto for_range = [&](auto&& body) {          // body(i, x[i]) for this thread's i, in order
        int i = lo;
        if (vec_ok) {
            for (; i + 4 <= hi; i += 4) {
                const float4 q = *reinterpret_cast<const float4*>(x + i);
                body(i, q.x);
                body(i + 1, q.y);
                body(i + 2, q.z);
                body(i + 3, q.w);
            }
        }
        for (; i < hi; ++i) body(i, x[i]);
    };

    // A logit that is no number counts as the lowest: every row, even one of nothing else, gets an id inside the
    // vocabulary (the next step reads the embedding table with it).
    ArgMax best{-CUDART_INF_F, 0x7fffffff};
    for (int i = tid; i < vocab; i += kThreads) {
        const float v = x[i];
        best = better(best, ArgMax{v == v ? v : -CUDART_INF_F, i});
    }
    const uint32_t my_max_key = best.i != 0x7fffffff ? order_key(best.v) : 0u;      // largest key among this thread's logits
    best = block_argmax(best, am_scratch);
    if (temp <= 0.0f) {
        if (probs != nullptr)
            for (int i = tid; i < vocab; i += kThreads) probs[i] = i == best.i ? 1.0f : 0.0f;
        if (tid == 0) out_ids[row] = best.i;
        return;
    }
    const float max_logit = best.v;
    const float inv_t = 1.0f / temp;
    const int mass_bits = min(47, 62 - (31 - __clz(vocab)));
    const double kMassUnit = (double)(1ull << mass_bits);

    int k = top_k[row];
    // ---- the short way for the usual top-k of some dozens: two more walks over the vocabulary instead of a dozen.
    // A threshold that at least k logits reach and few more do is found from the threads' own maxima; the logits
    // that reach it go to a list in shared memory, and everything else (exact top-k with
    // ties to the lower index, the softmax, the top-p cut, the draw) happens among them, with the same
    // distribution and tie rules as the general path below.  A list that would be too long takes the general path.
    // The same way serves top-p without top-k while the kSmallK largest logits hold the asked share of the whole
    // vocabulary's mass (they do for any distribution peaked enough to sample from): they are then the candidates.
    const bool topk_on = k > 0 && k < vocab;
    const bool nucleus_only = !topk_on && top_p[row] < 1.0f;
    if ((topk_on && k <= kSmallK) || nucleus_only) {
        const int ke = topk_on ? k : min(kSmallK, vocab);          // members: the ke largest
        double vocab_mass = 0.0;
        if (nucleus_only) {
            double mine = 0.0;
            for (int i = tid; i < vocab; i += kThreads) mine += (double)expf((x[i] - max_logit) * inv_t);
            block_exclusive_scan<double>(mine, d_scratch, &vocab_mass);
        }
        __shared__ int list_idx[kMaxList];
        __shared__ uint32_t list_key[kMaxList];
        __shared__ int list_rank[kMaxList];
        __shared__ int cand_idx[kSmallK];
        __shared__ float cand_e[kSmallK];          // exp((logit - max) / T), in index order
        __shared__ int cand_rank[kSmallK];         // place by (logit descending, index ascending)
        __shared__ float sorted_e[kSmallK];        // cand_e in that order
        __shared__ int sh_list_n, sh_cut;
        // The k-th largest of the 1,024 threads' own maxima is a lower bound of the k-th largest logit (k logits
        // are at least that large), and few other logits are: it is the threshold of the list (taken to its upper
        // 24 bits, which lets a few more in).  The logits that reach it are listed in one walk; a list that would
        // not fit is counted to its end and left to the general path.
        if (tid == 0) sh_list_n = 0;
        const uint32_t threshold = nth_largest_floor(my_max_key, ke, hist_count, &sh_prefix, &sh_int);
        for (int i = tid; i < vocab; i += kThreads) {
            const uint32_t key = order_key(x[i]);
            if (key >= threshold) {
                const int at = atomicAdd(&sh_list_n, 1);
                if (at < kMaxList) {
                    list_idx[at] = i;
                    list_key[at] = key;
                }
            }
        }
        __syncthreads();
        const int n_list = sh_list_n;
        if (n_list <= kMaxList) {
            // Place of every listed logit by (key descending, index ascending): the first k are the members; then the
            // members' places in index order.  Both are counts over the list; the block's threads share an entry's
            // count (threads / entries of them per entry, each over a part of the list, added up in shared memory).
            __shared__ int list_pos[kMaxList];
            for (int c = tid; c < n_list; c += kThreads) {
                list_rank[c] = 0;
                list_pos[c] = 0;
            }
            __syncthreads();
            const int sharers = max(1, kThreads / max(1, n_list)), part_len = (n_list + sharers - 1) / sharers;
            for (int w = tid; w < n_list * sharers; w += kThreads) {
                const int c = w % n_list, j0 = (w / n_list) * part_len, j1 = min(n_list, j0 + part_len);
                const uint32_t key = list_key[c];
                const int idx = list_idx[c];
                int before = 0;
                for (int j = j0; j < j1; ++j) before += (list_key[j] > key || (list_key[j] == key && list_idx[j] < idx)) ? 1 : 0;
                if (before != 0) atomicAdd(&list_rank[c], before);
            }
            __syncthreads();
            for (int w = tid; w < n_list * sharers; w += kThreads) {
                const int c = w % n_list, j0 = (w / n_list) * part_len, j1 = min(n_list, j0 + part_len);
                if (list_rank[c] >= ke) continue;
                const int idx = list_idx[c];
                int at = 0;
                for (int j = j0; j < j1; ++j) at += (list_rank[j] < ke && list_idx[j] < idx) ? 1 : 0;
                if (at != 0) atomicAdd(&list_pos[c], at);
            }
            __syncthreads();
            // Members in index order.
            for (int c = tid; c < n_list; c += kThreads) {
                if (list_rank[c] >= ke) continue;
                const int idx = list_idx[c], at = list_pos[c];
                const float e = expf((x[idx] - max_logit) * inv_t);
                cand_idx[at] = idx;
                cand_e[at] = e;
                cand_rank[at] = list_rank[c];
                sorted_e[list_rank[c]] = e;
            }
            __syncthreads();
            const int n = ke;
            // The sums run in a fixed order on one thread (they are a few dozen additions); the divisions, which
            // are slow in double precision, run one per thread.
            __shared__ double acc_s[kSmallK];
            __shared__ float cand_p[kSmallK];
            __shared__ double sh_total_mass;
            const float p_cut = top_p[row];
            if (tid < 32) {
                double mine, total_mass, run;
                int a, b;
                warp_ordered_offsets(n, [&](int c) { return (double)cand_e[c]; }, &mine, &total_mass, &a, &b);
                if (nucleus_only) total_mass = vocab_mass;          // the share is of the whole vocabulary's mass
                double before_me = warp_ordered_offsets(n, [&](int r) { return (double)sorted_e[r]; }, &mine, &run, &a, &b);
                for (int r = a; r < b; ++r) {
                    before_me += (double)sorted_e[r];
                    acc_s[r] = before_me;
                }
                if (tid == 0) {
                    sh_total_mass = total_mass;
                    sh_cut = n;
                }
            }
            __syncthreads();
            if (tid < n && p_cut < 1.0f && acc_s[tid] / sh_total_mass >= (double)p_cut) atomicMin(&sh_cut, tid + 1);
            __syncthreads();
            const int cut = sh_cut;
            // Top-p alone, and the candidates do not hold the asked share: the general path takes the row.
            const bool inside = !nucleus_only || n == vocab || acc_s[n - 1] / sh_total_mass >= (double)top_p[row];
            if (inside) {
            if (tid < 32) {
                double mine, kept;
                int a, b;
                warp_ordered_offsets(n, [&](int c) { return cand_rank[c] < cut ? (double)cand_e[c] : 0.0; }, &mine, &kept, &a, &b);
                if (tid == 0) sh_double = kept;
            }
            __syncthreads();
            const double kept_mass = sh_double;
            if (tid < n) cand_p[tid] = cand_rank[tid] < cut ? (float)((double)cand_e[tid] / kept_mass) : 0.0f;
            __syncthreads();
            if (tid < 32) {
                // The walk in index order: the lane whose run of candidates holds the draw walks it.
                double mine, total;
                int a, b;
                const double before_me = warp_ordered_offsets(n, [&](int c) { return cand_rank[c] < cut ? (double)cand_p[c] : 0.0; },
                                                              &mine, &total, &a, &b);
                const double r = uniform[row] * total;
                int choice = 0x7fffffff;
                if (before_me <= r && r < before_me + mine) {
                    double left = r - before_me;
                    for (int c = a; c < b && choice == 0x7fffffff; ++c) {
                        if (cand_rank[c] >= cut) continue;
                        left -= (double)cand_p[c];
                        if (left < 0.0) choice = cand_idx[c];
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) choice = min(choice, __shfl_xor_sync(0xffffffffu, choice, o));
                if (choice == 0x7fffffff) {           // rounding left the draw at or past the last kept id: the last id with mass
                    int last = -1;
                    for (int c = a; c < b; ++c)
                        if (cand_rank[c] < cut && cand_e[c] > 0.0f) last = cand_idx[c];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
                    choice = last >= 0 ? last : best.i;
                }
                if (tid == 0) out_ids[row] = choice;
            }
            if (probs != nullptr) {
                for (int i = tid; i < vocab; i += kThreads) probs[i] = 0.0f;
                __syncthreads();
                for (int c = tid; c < n; c += kThreads)
                    if (cand_rank[c] < cut) probs[cand_idx[c]] = cand_p[c];
            }
            return;
            }
        }
        __syncthreads();
    }

    // ---- top-k by count: key of the k-th largest, and how many ties at it are kept.

    uint32_t kth_key = 0;          // every key >= 0 is a member when top-k is off
    int kth_need = 0x7fffffff;     // ties at kth_key that are members (by index order)
    if (k > 0 && k < vocab) {
        uint32_t prefix = 0;
        int remaining = k;         // rank still to find inside the current bucket
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += kThreads) hist_count[b] = 0;
            __syncthreads();
            const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            // Thousands of keys share a few buckets (sign and exponent): lanes with the same bucket add once, together.
            for (int i0 = 0; i0 < vocab; i0 += kThreads) {
                const int i = i0 + tid;
                int bucket = -1;
                if (i < vocab) {
                    const uint32_t key = order_key(x[i]);
                    if ((key & mask) == prefix) bucket = (int)((key >> shift) & 255u);
                }
                const unsigned peers = __match_any_sync(0xffffffffu, bucket);
                if (bucket >= 0 && (int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist_count[bucket], __popc(peers));
            }
            __syncthreads();
            if (tid < 32) {
                int digit, rem;
                warp_bucket_by_count(hist_count, remaining, &digit, &rem);
                if (tid == 0) {
                    sh_int = rem;
                    sh_prefix = prefix | ((uint32_t)digit << shift);
                }
            }
            __syncthreads();
            remaining = sh_int;
            prefix = sh_prefix;
            __syncthreads();
        }
        kth_key = prefix;
        kth_need = remaining;      // >= 1
    }

    // ---- rank of each tie at kth_key in index order (only if some ties are cut).
    int tie_rank_base = 0;
    if (k > 0 && k < vocab) {          // without top-k every logit is a member, whatever its rank among equals
        int mine = 0;
        for_range([&](int, float xi) { mine += order_key(xi) == kth_key ? 1 : 0; });
        int total;
        tie_rank_base = block_exclusive_scan<int>(mine, i_scratch, &total);
    }
    // member(i): key > kth_key, or key == kth_key and its rank among such ties < kth_need.

    // ---- total mass of the members.
    double total_mass;
    {
        double mine = 0.0;
        int rank = tie_rank_base;
        for_range([&](int, float xi) {
            const uint32_t key = order_key(xi);
            bool member = key > kth_key;
            if (key == kth_key) member = rank++ < kth_need;
            if (member) mine += (double)expf((xi - max_logit) * inv_t);
        });
        block_exclusive_scan<double>(mine, d_scratch, &total_mass);
    }

    // ---- top-p by mass over the members: cut key, mass above it, ties kept at it.
    const float p_cut = top_p[row];
    uint32_t cut_key = 0;
    int cut_need = 0x7fffffff;
    double kept_mass = total_mass;
    if (p_cut < 1.0f) {
        uint32_t prefix = 0;
        unsigned long long above_fixed = 0ull;        // mass of members with a key above the current bucket, in fixed point
        __shared__ unsigned long long sh_above;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += kThreads) hist_mass[b] = 0ull;
            __syncthreads();
            const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            int rank = tie_rank_base;
            float four[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
            for (int it = 0; it < per; ++it) {                  // the same number of trips for every lane
                const int i = lo + it;
                if ((it & 3) == 0) {
                    if (vec_ok && i + 4 <= hi) {
                        const float4 q = *reinterpret_cast<const float4*>(x + i);
                        four[0] = q.x; four[1] = q.y; four[2] = q.z; four[3] = q.w;
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) four[e] = i + e < hi ? x[i + e] : 0.0f;
                    }
                }
                int bucket = -1;
                unsigned long long term = 0ull;
                if (i < hi) {
                    const float xi = four[it & 3];
                    const uint32_t key = order_key(xi);
                    bool member = key > kth_key;
                    if (key == kth_key) member = rank++ < kth_need;
                    if (member && (key & mask) == prefix) {
                        bucket = (int)((key >> shift) & 255u);
                        term = (unsigned long long)((double)expf((xi - max_logit) * inv_t) * kMassUnit);      // < 2^48
                    }
                }
                if (!__any_sync(0xffffffffu, bucket >= 0)) continue;          // no lane of the warp has a term (the later passes, mostly)
                const unsigned peers = __match_any_sync(0xffffffffu, bucket);
                const unsigned s0 = __reduce_add_sync(peers, (unsigned)(term & 0xffffu));
                const unsigned s1 = __reduce_add_sync(peers, (unsigned)((term >> 16) & 0xffffu));
                const unsigned s2 = __reduce_add_sync(peers, (unsigned)(term >> 32));
                if (bucket >= 0 && (int)(threadIdx.x & 31) == __ffs(peers) - 1)
                    atomicAdd(&hist_mass[bucket], (unsigned long long)s0 + ((unsigned long long)s1 << 16) + ((unsigned long long)s2 << 32));
            }
            __syncthreads();
            if (tid < 32) {
                int digit;
                unsigned long long above_digit;
                warp_bucket_by_mass(hist_mass, above_fixed, kMassUnit, total_mass, (double)p_cut, &digit, &above_digit);
                if (tid == 0) {
                    sh_above = above_digit;
                    sh_prefix = prefix | ((uint32_t)digit << shift);
                }
            }
            __syncthreads();
            above_fixed = sh_above;
            prefix = sh_prefix;
            __syncthreads();
        }
        cut_key = prefix;
        const double above = (double)above_fixed / kMassUnit;
        // Members at cut_key all have the same p; keep as many (in index order) as the prefix needs.
        if (tid == 0) {
            const uint32_t b = (cut_key & 0x80000000u) ? (cut_key & 0x7fffffffu) : ~cut_key;
            const float pv = expf((__uint_as_float(b) - max_logit) * inv_t);
            // At least one tie is kept (the bucket was chosen because it reaches p_cut or is the last).
            const double unit = (double)pv / total_mass, start = above / total_mass;
            long long need = unit > 0.0 ? (long long)ceil(((double)p_cut - start) / unit) : 1;
            if (need < 1) need = 1;
            if (need > vocab) need = vocab;
            while (need > 1 && start + (double)(need - 1) * unit >= (double)p_cut) --need;
            while (need < vocab && start + (double)need * unit < (double)p_cut) ++need;
            sh_int = (int)need;
        }
        __syncthreads();
        cut_need = sh_int;
        __syncthreads();
    }

    // ---- final pass in index order: kept mass, probabilities, and the draw.
    // kept(i): member(i) and (key > cut_key, or key == cut_key with rank among member ties at cut_key < cut_need).
    int cut_rank_base = 0;
    {
        int mine = 0, rank = tie_rank_base;
        for_range([&](int, float xi) {
            const uint32_t key = order_key(xi);
            bool member = key > kth_key;
            if (key == kth_key) member = rank++ < kth_need;
            mine += (member && key == cut_key) ? 1 : 0;
        });
        int total;
        cut_rank_base = block_exclusive_scan<int>(mine, i_scratch, &total);
    }
    {
        double mine = 0.0;
        int rank = tie_rank_base, crank = cut_rank_base;
        for_range([&](int, float xi) {
            const uint32_t key = order_key(xi);
            bool member = key > kth_key;
            if (key == kth_key) member = rank++ < kth_need;
            bool kept = member && key > cut_key;
            if (member && key == cut_key) kept = crank++ < cut_need;
            if (kept) mine += (double)expf((xi - max_logit) * inv_t);
        });
        block_exclusive_scan<double>(mine, d_scratch, &kept_mass);
    }
    // Normalised float probabilities, their double sum in index order, and the walk.
    double my_sum = 0.0;
    {
        int rank = tie_rank_base, crank = cut_rank_base;
        for_range([&](int i, float xi) {
            const uint32_t key = order_key(xi);
            bool member = key > kth_key;
            if (key == kth_key) member = rank++ < kth_need;
            bool kept = member && key > cut_key;
            if (member && key == cut_key) kept = crank++ < cut_need;
            const float p = kept ? (float)((double)expf((xi - max_logit) * inv_t) / kept_mass) : 0.0f;
            if (probs != nullptr) probs[i] = p;
            my_sum += (double)p;
        });
    }
    double total;
    const double before = block_exclusive_scan<double>(my_sum, d_scratch, &total);
    if (tid == 0) sh_choice = 0x7fffffff;
    __syncthreads();
    const double r = uniform[row] * total;
    if (before <= r && r < before + my_sum) {
        // The draw falls inside this thread's range: walk it as the reference walks the whole vocabulary.
        double left = r - before;
        int rank = tie_rank_base, crank = cut_rank_base, choice = -1;
        for_range([&](int i, float xi) {
            if (choice >= 0) return;
            const uint32_t key = order_key(xi);
            bool member = key > kth_key;
            if (key == kth_key) member = rank++ < kth_need;
            bool kept = member && key > cut_key;
            if (member && key == cut_key) kept = crank++ < cut_need;
            if (!kept) return;
            left -= (double)(float)((double)expf((xi - max_logit) * inv_t) / kept_mass);
            if (left < 0.0) choice = i;
        });
        if (choice >= 0) atomicMin(&sh_choice, choice);
    }
    __syncthreads();
    if (sh_choice == 0x7fffffff) {
        // Rounding left r at or past the last kept id: take the last id with mass.
        int last = -1, rank = tie_rank_base, crank = cut_rank_base;
        for_range([&](int i, float xi) {
            const uint32_t key = order_key(xi);
            bool member = key > kth_key;
            if (key == kth_key) member = rank++ < kth_need;
            bool kept = member && key > cut_key;
            if (member && key == cut_key) kept = crank++ < cut_need;
            if (kept && expf((xi - max_logit) * inv_t) > 0.0f) last = i;
        });
        __shared__ int sh_last;
        if (tid == 0) sh_last = -1;
        __syncthreads();
        if (last >= 0) atomicMax(&sh_last, last);
        __syncthreads();
        if (tid == 0) out_ids[row] = sh_last >= 0 ? sh_last : best.i;
    } else if (tid == 0) {
        out_ids[row] = sh_choice;
    }
}

}  // namespace

extern "C" int lb_sample(const float* logits, int64_t row_stride, int n_rows, int vocab, const float* temperature,
                         const int32_t* top_k, const float* top_p, const double* uniform, int32_t* out_ids,
                         float* out_probs, void* stream) {
    LB_CHECK_ARG(n_rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d vocab=%d", n_rows, vocab);
    if (n_rows == 0) return LB_OK;
    LB_CHECK_CUDA(lb_launch_overlapped(sample_kernel, dim3(n_rows), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), 
        logits, row_stride, vocab, temperature, top_k, top_p, uniform, out_ids, out_probs));
    LB_CHECK_LAUNCH();
    return LB_OK;
}
