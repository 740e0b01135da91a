// Kernels of the toy parts that the tests register from outside the framework.  Plain, slow, one thread per
// element: they only have to be right.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__device__ float load(const void* p, int bf16, int64_t i) {
    return bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]) : static_cast<const float*>(p)[i];
}
__device__ void store(void* p, int bf16, int64_t i, float v) {
    if (bf16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    else static_cast<float*>(p)[i] = v;
}

// means[t] = (sum before the step + h[first .. t]) / (count before + t - first + 1) for every token of request
// blockIdx.x; the request's state [hidden sums | count] is advanced when `write`.
__global__ void running_mean_kernel(const void* h, int bf16, int64_t h_stride, void* means, int64_t m_stride, float* state,
                                    const int32_t* q_start, const int32_t* slots, int hidden, int write, int only_seq) {
    const int s = only_seq >= 0 ? only_seq : blockIdx.x;
    float* st = state + (int64_t)slots[s] * (hidden + 1);
    const int lo = q_start[s], hi = q_start[s + 1];
    const float count0 = st[hidden];
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float sum = st[c];
        for (int t = lo; t < hi; ++t) {
            sum += load(h, bf16, (int64_t)t * h_stride + c);
            store(means, bf16, (int64_t)t * m_stride + c, sum / (count0 + (float)(t - lo + 1)));
        }
        if (write) st[c] = sum;
    }
    __syncthreads();
    if (write && threadIdx.x == 0) st[hidden] = count0 + (float)(hi - lo);
}

__global__ void rms_kernel(const float* x, const int32_t* rows, const float* weight, void* out, int bf16, int width, float eps) {
    const int r = blockIdx.x;
    const float* src = x + (int64_t)(rows ? rows[r] : r) * width;
    __shared__ float total;
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int c = 0; c < width; ++c) s += src[c] * src[c];
        total = rsqrtf(s / width + eps);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < width; c += blockDim.x) store(out, bf16, (int64_t)r * width + c, src[c] * total * weight[c]);
}

__global__ void sinusoid_kernel(float* x, const int32_t* positions, int width, float base) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float freq = powf(base, -(float)(c & ~1) / width);
        const float angle = (float)positions[t] * freq;
        x[(int64_t)t * width + c] += (c & 1) ? cosf(angle) : sinf(angle);
    }
}

// Every token goes to its best `top` of `experts` small ungated experts (relu); router softmax in 32-bit.
// One block per token; weights are float32 or bfloat16.
__global__ void routed_ff_kernel(const void* h, int bf16, int64_t h_stride, float* x, int64_t x_stride, const void* router, const void* up,
                                 const void* down, int experts, int inner, int hidden, int top) {
    extern __shared__ float sh[];        // gate[experts] | mid[inner]
    float* gate = sh;
    float* mid = sh + experts;
    const int t = blockIdx.x;
    if (threadIdx.x == 0) {
        float mx = -1e30f;
        for (int e = 0; e < experts; ++e) {
            float s = 0.0f;
            for (int c = 0; c < hidden; ++c) s += load(h, bf16, (int64_t)t * h_stride + c) * load(router, bf16, (int64_t)e * hidden + c);
            gate[e] = s;
            mx = fmaxf(mx, s);
        }
        float sum = 0.0f;
        for (int e = 0; e < experts; ++e) { gate[e] = expf(gate[e] - mx); sum += gate[e]; }
        for (int e = 0; e < experts; ++e) gate[e] /= sum;
    }
    __syncthreads();
    // the `top` largest gates, earlier index first among equals; their shares renormalised
    __shared__ int chosen[8];
    __shared__ float share[8];
    if (threadIdx.x == 0) {
        float kept = 0.0f;
        for (int k = 0; k < top; ++k) {
            int best = -1;
            for (int e = 0; e < experts; ++e) {
                bool taken = false;
                for (int j = 0; j < k; ++j) taken = taken || chosen[j] == e;
                if (!taken && (best < 0 || gate[e] > gate[best])) best = e;
            }
            chosen[k] = best;
            kept += gate[best];
        }
        for (int k = 0; k < top; ++k) share[k] = gate[chosen[k]] / kept;
    }
    __syncthreads();
    for (int k = 0; k < top; ++k) {
        const int e = chosen[k];
        for (int i = threadIdx.x; i < inner; i += blockDim.x) {
            float s = 0.0f;
            for (int c = 0; c < hidden; ++c) s += load(h, bf16, (int64_t)t * h_stride + c) * load(up, bf16, ((int64_t)e * inner + i) * hidden + c);
            mid[i] = fmaxf(s, 0.0f);
        }
        __syncthreads();
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            float s = 0.0f;
            for (int i = 0; i < inner; ++i) s += mid[i] * load(down, bf16, ((int64_t)e * hidden + c) * inner + i);
            x[(int64_t)t * x_stride + c] += share[k] * s;
        }
        __syncthreads();
    }
}

}  // namespace

extern "C" {

void toy_running_mean(const void* h, int bf16, int64_t h_stride, void* means, int64_t m_stride, float* state, const int32_t* q_start,
                      const int32_t* slots, int n_seq, int hidden, int write, int only_seq, cudaStream_t s) {
    running_mean_kernel<<<only_seq >= 0 ? 1 : n_seq, 64, 0, s>>>(h, bf16, h_stride, means, m_stride, state, q_start, slots, hidden, write, only_seq);
}

void toy_rms(const float* x, const int32_t* rows, const float* weight, void* out, int bf16, int n_rows, int width, float eps, cudaStream_t s) {
    rms_kernel<<<n_rows, 64, 0, s>>>(x, rows, weight, out, bf16, width, eps);
}

void toy_sinusoid(float* x, const int32_t* positions, int n_tokens, int width, float base, cudaStream_t s) {
    sinusoid_kernel<<<n_tokens, 64, 0, s>>>(x, positions, width, base);
}

void toy_routed_ff(const void* h, int bf16, int64_t h_stride, float* x, int64_t x_stride, const void* router, const void* up, const void* down,
                   int n_tokens, int experts, int inner, int hidden, int top, cudaStream_t s) {
    routed_ff_kernel<<<n_tokens, 64, (experts + inner) * sizeof(float), s>>>(h, bf16, h_stride, x, x_stride, router, up, down, experts, inner, hidden, top);
}

}
