// Several small tensors per launch: the sum of squares of their gradients and
// their RangerLite update.  The trainer holds ten parameter groups
// (model/nnue.py:117-182 of the reference project); nine of them are small
// (biases, the layer-stack weights), and one launch per tensor costs more in
// launch overhead than in work.  The tensor descriptors travel by value in
// the kernel parameters; blockIdx.y selects the tensor.
#include <algorithm>

#include "ranger.cuh"

namespace nnue {

struct SumsqJob {
    const float* g[NNUE_MULTI_MAX];
    int64_t n[NNUE_MULTI_MAX];
};

// Reproducible: every CTA leaves its partial sum in a slot of its own; the CTA that arrives last adds
// all slots in a fixed order (whichever CTA that is) and adds the total to *out.  The slots are a
// file-scope array: calls that overlap on the GPU (different streams) would share it and must not.
constexpr int kSumsqMaxGridX = 1024;
__device__ float g_sumsq_partial[NNUE_MULTI_MAX * kSumsqMaxGridX];
__device__ unsigned int g_sumsq_arrived;

__device__ __forceinline__ void sumsq_finish(float mine, float* __restrict__ out) {
    __shared__ float s_w[kWarpsPerCta];
    __shared__ bool s_last;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mine += __shfl_xor_sync(kFullMask, mine, d);
    if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = mine;
    __syncthreads();
    const unsigned n_ctas = gridDim.x * gridDim.y;
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < kWarpsPerCta; ++w) t += s_w[w];
        g_sumsq_partial[blockIdx.y * gridDim.x + blockIdx.x] = t;
        __threadfence();
        s_last = atomicAdd(&g_sumsq_arrived, 1u) == n_ctas - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float acc = 0.f;
    for (unsigned i = threadIdx.x; i < n_ctas; i += kThreads) acc += __ldcg(&g_sumsq_partial[i]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(kFullMask, acc, d);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < kWarpsPerCta; ++w) t += s_w[w];
        *out += t;
        g_sumsq_arrived = 0;  // ready for the next launch
    }
}

__global__ void __launch_bounds__(kThreads) k_sumsq_multi(SumsqJob job, float* __restrict__ out) {
    const float* g = job.g[blockIdx.y];
    const int64_t n = job.n[blockIdx.y];
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    float acc = 0.f;
    int64_t done = 0;
    if ((reinterpret_cast<uintptr_t>(g) & 15u) == 0) {
        const int64_t n4 = n >> 2;
        const float4* g4 = reinterpret_cast<const float4*>(g);
        for (int64_t i = t0; i < n4; i += stride) {
            const float4 v = __ldg(g4 + i);
            acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        done = n4 << 2;
    }
    for (int64_t i = done + t0; i < n; i += stride) acc += g[i] * g[i];
    sumsq_finish(acc, out);
}

struct RangerJob {
    nnue_ranger_tensor t[NNUE_MULTI_MAX];
};

__global__ void __launch_bounds__(kThreads)
    k_ranger_multi(const __grid_constant__ RangerJob job, const float* __restrict__ d_scale) {
    const nnue_ranger_tensor& t = job.t[blockIdx.y];
    const int64_t n = t.n;
    if ((int64_t)blockIdx.x * blockDim.x >= n) return;
    const RangerConst& c = t.hp;
    const float scale = d_scale ? __ldg(d_scale) : 1.f;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t done = 0;
    const uintptr_t all = reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.grad) |
                          reinterpret_cast<uintptr_t>(t.grad_ma) | reinterpret_cast<uintptr_t>(t.neg_grad_ma) |
                          reinterpret_cast<uintptr_t>(t.variance_ma) | reinterpret_cast<uintptr_t>(t.slow);
    if ((all & 15u) == 0) {
        const int64_t n4 = n >> 2;
        const float4* g4 = reinterpret_cast<const float4*>(t.grad);
        for (int64_t i = t0; i < n4; i += stride)
            ranger_vec4(c, scale, i, g4, reinterpret_cast<float4*>(t.p), reinterpret_cast<float4*>(t.grad_ma),
                        reinterpret_cast<float4*>(t.neg_grad_ma), reinterpret_cast<float4*>(t.variance_ma),
                        reinterpret_cast<float4*>(t.slow), __ldg(g4 + i));
        done = n4 << 2;
    }
    for (int64_t i = done + t0; i < n; i += stride) {
        float pv = t.p[i], gmv = t.grad_ma[i], vmv = t.variance_ma[i];
        float ngv = c.use_pnm ? t.neg_grad_ma[i] : 0.f, sv = c.do_merge ? t.slow[i] : 0.f;
        ranger_elem(c, scale, t.grad[i], pv, gmv, ngv, vmv, sv);
        if (c.phase != 2) t.variance_ma[i] = vmv;
        if (c.phase == 1) continue;
        t.p[i] = pv;
        if (!c.use_pnm || c.step_is_odd) t.grad_ma[i] = gmv;
        if (c.use_pnm && !c.step_is_odd) t.neg_grad_ma[i] = ngv;
        if (c.do_merge) t.slow[i] = sv;
    }
}

static unsigned grid_x_for(int64_t max_n) {
    const int64_t want = (max_n / 4 + kThreads - 1) / kThreads + 1;
    return (unsigned)std::min<int64_t>(want, std::min<int64_t>((int64_t)sm_count() * 4, kSumsqMaxGridX));
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_grad_sumsq_multi(const float* const* h_grads, const int64_t* h_n, int32_t count,
                                     float* d_out_sumsq, void* stream) {
    NNUE_REQUIRE(count >= 0 && (count == 0 || (h_grads && h_n && d_out_sumsq)), NNUE_ERR_ARG,
                 "nnue_grad_sumsq_multi: null pointer or negative count");
    for (int32_t base = 0; base < count; base += NNUE_MULTI_MAX) {
        const int m = std::min<int32_t>(NNUE_MULTI_MAX, count - base);
        SumsqJob job;
        int64_t max_n = 0;
        for (int i = 0; i < NNUE_MULTI_MAX; ++i) {
            job.g[i] = i < m ? h_grads[base + i] : nullptr;
            job.n[i] = i < m ? h_n[base + i] : 0;
            NNUE_REQUIRE(job.n[i] >= 0 && (job.n[i] == 0 || job.g[i]), NNUE_ERR_ARG,
                         "nnue_grad_sumsq_multi: tensor %d is null or has a negative size", base + i);
            max_n = std::max(max_n, job.n[i]);
        }
        if (max_n == 0) continue;
        k_sumsq_multi<<<dim3(grid_x_for(max_n), (unsigned)m), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            job, d_out_sumsq);
        NNUE_CUDA_TRY(cudaGetLastError());
        note_launches(1);
    }
    return NNUE_OK;
}

extern "C" int nnue_rangerlite_update_multi(const nnue_ranger_tensor* h_tensors, int32_t count,
                                            const float* d_grad_scale, void* stream) {
    NNUE_REQUIRE(count >= 0 && (count == 0 || h_tensors), NNUE_ERR_ARG,
                 "nnue_rangerlite_update_multi: null descriptors or negative count");
    for (int32_t base = 0; base < count; base += NNUE_MULTI_MAX) {
        const int m = std::min<int32_t>(NNUE_MULTI_MAX, count - base);
        RangerJob job;
        memset(&job, 0, sizeof(job));
        int64_t max_n = 0;
        for (int i = 0; i < m; ++i) {
            const nnue_ranger_tensor& t = h_tensors[base + i];
            NNUE_REQUIRE(t.n >= 0, NNUE_ERR_ARG, "nnue_rangerlite_update_multi: tensor %d has a negative size", base + i);
            if (t.n > 0) {
                NNUE_REQUIRE(t.p && t.grad && t.grad_ma && t.variance_ma, NNUE_ERR_ARG,
                             "nnue_rangerlite_update_multi: tensor %d has a null buffer", base + i);
                NNUE_REQUIRE(!t.hp.use_pnm || t.neg_grad_ma, NNUE_ERR_ARG,
                             "nnue_rangerlite_update_multi: tensor %d uses PNM without neg_grad_ma", base + i);
                NNUE_REQUIRE(!t.hp.do_merge || t.slow, NNUE_ERR_ARG,
                             "nnue_rangerlite_update_multi: tensor %d merges without a lookahead copy", base + i);
            }
            job.t[i] = t;
            max_n = std::max(max_n, t.n);
        }
        if (max_n == 0) continue;
        k_ranger_multi<<<dim3(grid_x_for(max_n), (unsigned)m), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            job, d_grad_scale);
        NNUE_CUDA_TRY(cudaGetLastError());
        note_launches(1);
    }
    return NNUE_OK;
}
