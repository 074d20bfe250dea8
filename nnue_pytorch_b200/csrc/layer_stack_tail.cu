// Everything of the layer stack after the first layer, per position:
// squared / linear clipped activations, layer 2 (64 -> 32), output layer
// (128 -> 1), the skip connection and the output fake quantization, and the
// gradient of all of it (model/modules/layer_stacks.py:33-84 and
// model/quantize.py:36-45,133-147 of the reference project; every fake
// quantization is straight-through in the backward).
// A CTA takes one tile (<= 64 positions of one bucket, see layer_stack.cu) so
// the bucket's weights sit in shared memory; a warp takes one position at a
// time with one lane per hidden unit.
#include <algorithm>

#include "layer_stack.cuh"

namespace nnue {

constexpr int kIn2 = 2 * kLsOut;            // 64 inputs of layer 2
constexpr int kIn3 = 4 * kLsOut;            // 128 inputs of the output layer
constexpr int kW2Pad = kIn2 + 1;            // row stride of the shared copy: conflict-free columns
constexpr int kPartW2 = kLsOut * kIn2;      // 2048
constexpr int kPartStride = kPartW2 + kLsOut + kIn3 + 4;  // dW2 | db2 | dW3 | db3 (+pad) = 2212

struct TailAct {
    float a, b;  // the two activations of one unit: clipped fq(v*v)*corr and clipped fq(v)
    bool ma, mb; // gradient masks of the two clamps (closed interval)
};

__device__ __forceinline__ TailAct tail_act(float v, const LsAct& c) {
    TailAct r;
    const float sq = __fmul_rn(ls_fq(__fmul_rn(v, v), c), c.sqr_corr);
    const float li = ls_fq(v, c);
    r.ma = sq >= 0.f && sq <= c.max_hidden;
    r.mb = li >= 0.f && li <= c.max_hidden;
    r.a = fminf(fmaxf(sq, 0.f), c.max_hidden);
    r.b = fminf(fmaxf(li, 0.f), c.max_hidden);
    return r;
}

__device__ __forceinline__ void load_bucket_weights(const float* __restrict__ W2, const float* __restrict__ b2,
                                                    const float* __restrict__ W3, int bk, float (*W2s)[kW2Pad],
                                                    float* b2s, float* W3s) {
    for (int i = threadIdx.x; i < kPartW2; i += blockDim.x)
        W2s[i / kIn2][i % kIn2] = __ldg(W2 + (int64_t)bk * kPartW2 + i);
    for (int i = threadIdx.x; i < kIn3; i += blockDim.x) W3s[i] = __ldg(W3 + (int64_t)bk * kIn3 + i);
    if (b2s)
        for (int i = threadIdx.x; i < kLsOut; i += blockDim.x) b2s[i] = __ldg(b2 + bk * kLsOut + i);
}

// lane o: b2[o] + sum_i W2[o][i] * x1[i], i ascending (x1 = [xa (32), xb (32)] spread over the lanes)
__device__ __forceinline__ float layer2_row(const float (*W2s)[kW2Pad], float bias, float xa, float xb, int lane) {
    float acc = bias;
#pragma unroll
    for (int i = 0; i < kLsOut; ++i) acc = __fmaf_rn(W2s[lane][i], __shfl_sync(kFullMask, xa, i), acc);
#pragma unroll
    for (int i = 0; i < kLsOut; ++i) acc = __fmaf_rn(W2s[lane][kLsOut + i], __shfl_sync(kFullMask, xb, i), acc);
    return acc;
}

__global__ void __launch_bounds__(256)
    k_ls_tail_fwd(const float* __restrict__ o1, LsPlanView plan, const float* __restrict__ W2,
                  const float* __restrict__ b2, const float* __restrict__ W3, const float* __restrict__ b3,
                  LsAct c, float* __restrict__ o2, float* __restrict__ y) {
    __shared__ float W2s[kLsOut][kW2Pad];
    __shared__ float b2s[kLsOut], W3s[kIn3];
    const int t = blockIdx.x;
    if (t >= *plan.n_tiles) return;
    const int cnt = plan.tile_count[t], bk = plan.tile_bucket[t];
    const int32_t* perm = plan.perm + plan.tile_start[t];
    load_bucket_weights(W2, b2, W3, bk, W2s, b2s, W3s);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float bias3 = __ldg(b3 + bk);
    for (int i = warp; i < cnt; i += 8) {
        const int64_t p = perm[i];
        const float v1 = __ldg(o1 + p * kLsOut + lane);
        const float skip = __fadd_rn(__shfl_sync(kFullMask, v1, kLsOut - 2), -__shfl_sync(kFullMask, v1, kLsOut - 1));
        const TailAct x1 = tail_act(v1, c);
        const float v2 = layer2_row(W2s, b2s[lane], x1.a, x1.b, lane);
        const TailAct x2 = tail_act(v2, c);
        float part = __fmul_rn(W3s[lane], x1.a);
        part = __fmaf_rn(W3s[kLsOut + lane], x1.b, part);
        part = __fmaf_rn(W3s[2 * kLsOut + lane], x2.a, part);
        part = __fmaf_rn(W3s[3 * kLsOut + lane], x2.b, part);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) part = __fadd_rn(part, __shfl_xor_sync(kFullMask, part, d));
        float out = __fadd_rn(__fadd_rn(part, bias3), skip);
        if (c.quantize_out) {
            const long long as_int = llrintf(__fmul_rn(out, c.out_den));
            const long long q = (as_int * (long long)c.out_mul) / (long long)c.out_den;  // truncates toward zero
            out = __fdiv_rn((float)q, c.out_mul);
        }
        o2[p * kLsOut + lane] = v2;
        if (lane == 0) y[p] = out;
    }
}

__global__ void __launch_bounds__(256)
    k_ls_tail_bwd(const float* __restrict__ o1, const float* __restrict__ o2, LsPlanView plan,
                  const float* __restrict__ W2, const float* __restrict__ W3, const float* __restrict__ grad_y,
                  LsAct c, float* __restrict__ d_o1, float* __restrict__ part) {
    __shared__ float W2s[kLsOut][kW2Pad];
    __shared__ float W3s[kIn3];
    __shared__ float red[kPartStride];
    const int t = blockIdx.x;
    if (t >= *plan.n_tiles) return;
    const int cnt = plan.tile_count[t], bk = plan.tile_bucket[t];
    const int32_t* perm = plan.perm + plan.tile_start[t];
    load_bucket_weights(W2, nullptr, W3, bk, W2s, nullptr, W3s);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float aW2[kIn2];  // row `lane` of dW2, this warp's positions
#pragma unroll
    for (int i = 0; i < kIn2; ++i) aW2[i] = 0.f;
    float ab2 = 0.f, aW3[4] = {0.f, 0.f, 0.f, 0.f}, ab3 = 0.f;
    for (int i = warp; i < cnt; i += 8) {
        const int64_t p = perm[i];
        const float v1 = __ldg(o1 + p * kLsOut + lane), v2 = __ldg(o2 + p * kLsOut + lane);
        const float gy = __ldg(grad_y + p);
        const TailAct x1 = tail_act(v1, c), x2 = tail_act(v2, c);
        // output layer
        aW3[0] = __fmaf_rn(gy, x1.a, aW3[0]);
        aW3[1] = __fmaf_rn(gy, x1.b, aW3[1]);
        aW3[2] = __fmaf_rn(gy, x2.a, aW3[2]);
        aW3[3] = __fmaf_rn(gy, x2.b, aW3[3]);
        ab3 = __fadd_rn(ab3, gy);
        const float g2a = __fmul_rn(gy, W3s[2 * kLsOut + lane]), g2b = __fmul_rn(gy, W3s[3 * kLsOut + lane]);
        float g1a = __fmul_rn(gy, W3s[lane]), g1b = __fmul_rn(gy, W3s[kLsOut + lane]);
        // through the activations of layer 2: d(v*v) = 2 v, fake quantization is straight-through
        float d2 = x2.ma ? __fmul_rn(__fmul_rn(g2a, c.sqr_corr), __fmul_rn(2.f, v2)) : 0.f;
        d2 = __fadd_rn(d2, x2.mb ? g2b : 0.f);
        ab2 = __fadd_rn(ab2, d2);
        // dW2[lane][i] += d2 * x1[i];  g_x1[i] += sum_o d2[o] * W2[o][i] (lane i owns columns i, 32 + i)
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int j = 0; j < kLsOut; ++j) {
            aW2[j] = __fmaf_rn(d2, __shfl_sync(kFullMask, x1.a, j), aW2[j]);
            aW2[kLsOut + j] = __fmaf_rn(d2, __shfl_sync(kFullMask, x1.b, j), aW2[kLsOut + j]);
            const float dj = __shfl_sync(kFullMask, d2, j);
            sa = __fmaf_rn(dj, W2s[j][lane], sa);
            sb = __fmaf_rn(dj, W2s[j][kLsOut + lane], sb);
        }
        g1a = __fadd_rn(g1a, sa);
        g1b = __fadd_rn(g1b, sb);
        float d1 = x1.ma ? __fmul_rn(__fmul_rn(g1a, c.sqr_corr), __fmul_rn(2.f, v1)) : 0.f;
        d1 = __fadd_rn(d1, x1.mb ? g1b : 0.f);
        if (lane == kLsOut - 2) d1 = __fadd_rn(d1, gy);   // skip = o1[30] - o1[31]
        if (lane == kLsOut - 1) d1 = __fadd_rn(d1, -gy);
        d_o1[p * kLsOut + lane] = d1;
    }
    // combine the 8 warps in warp order through one shared buffer
    for (int w = 0; w < 8; ++w) {
        if (warp == w) {
#pragma unroll
            for (int i = 0; i < kIn2; ++i) {
                const int j = i * kLsOut + lane;  // transposed in shared memory: no bank conflicts
                red[j] = w ? __fadd_rn(red[j], aW2[i]) : aW2[i];
            }
            const int jb = kPartW2 + lane;
            red[jb] = w ? __fadd_rn(red[jb], ab2) : ab2;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j3 = kPartW2 + kLsOut + q * kLsOut + lane;
                red[j3] = w ? __fadd_rn(red[j3], aW3[q]) : aW3[q];
            }
            if (lane == 0) {
                const int jz = kPartW2 + kLsOut + kIn3;
                red[jz] = w ? __fadd_rn(red[jz], ab3) : ab3;
            }
        }
        __syncthreads();
    }
    float* dst = part + (int64_t)t * kPartStride;
    for (int i = threadIdx.x; i <= kPartW2 + kLsOut + kIn3; i += blockDim.x)
        dst[i] = i < kPartW2 ? red[(i % kIn2) * kLsOut + i / kIn2] : red[i];  // dW2 back to [unit][input]
}

// out[bucket][j] = sum over the bucket's tiles (tile order) of part[tile][j]
__global__ void __launch_bounds__(256)
    k_ls_tail_wsum(const float* __restrict__ part, LsPlanView plan, float* __restrict__ dW2,
                   float* __restrict__ db2, float* __restrict__ dW3, float* __restrict__ db3) {
    const int bk = blockIdx.y;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j > kPartW2 + kLsOut + kIn3) return;
    float s = 0.f;
    for (int t = plan.bucket_tile[bk]; t < plan.bucket_tile[bk + 1]; ++t)
        s = __fadd_rn(s, part[(int64_t)t * kPartStride + j]);
    if (j < kPartW2) dW2[(int64_t)bk * kPartW2 + j] = s;
    else if (j < kPartW2 + kLsOut) db2[bk * kLsOut + (j - kPartW2)] = s;
    else if (j < kPartW2 + kLsOut + kIn3) dW3[bk * kIn3 + (j - kPartW2 - kLsOut)] = s;
    else db3[bk] = s;
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_ls_tail_fwd(const float* o1, const void* plan, const float* W2, const float* b2,
                                const float* W3, const float* b3, const nnue_ls_params* params, float* o2,
                                float* y, int64_t B, int32_t C, void* stream) {
    NNUE_REQUIRE(params != nullptr && plan != nullptr, NNUE_ERR_ARG, "nnue_ls_tail_fwd: null params or plan");
    NNUE_REQUIRE(B >= 0 && C > 0 && C <= 16, NNUE_ERR_UNSUPPORTED, "nnue_ls_tail_fwd: bad batch or bucket count");
    if (B == 0) return NNUE_OK;
    NNUE_REQUIRE(o1 && W2 && b2 && W3 && b3 && o2 && y, NNUE_ERR_ARG, "nnue_ls_tail_fwd: null tensor");
    k_ls_tail_fwd<<<(unsigned)ls_max_tiles(B, C), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        o1, ls_view(plan, B, C), W2, b2, W3, b3, *params, o2, y);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

extern "C" size_t nnue_ls_tail_bwd_workspace_bytes(int64_t B, int32_t C) {
    if (B < 0 || C <= 0) return 0;
    return (size_t)ls_max_tiles(B, C) * kPartStride * sizeof(float) + 256;
}

extern "C" int nnue_ls_tail_bwd(const float* o1, const float* o2, const void* plan, const float* W2,
                                const float* W3, const float* grad_y, const nnue_ls_params* params,
                                float* d_o1, float* dW2, float* db2, float* dW3, float* db3, void* workspace,
                                size_t workspace_bytes, int64_t B, int32_t C, void* stream) {
    NNUE_REQUIRE(params != nullptr && plan != nullptr, NNUE_ERR_ARG, "nnue_ls_tail_bwd: null params or plan");
    NNUE_REQUIRE(B >= 0 && C > 0 && C <= 16, NNUE_ERR_UNSUPPORTED, "nnue_ls_tail_bwd: bad batch or bucket count");
    NNUE_REQUIRE(dW2 && db2 && dW3 && db3, NNUE_ERR_ARG, "nnue_ls_tail_bwd: null output");
    NNUE_REQUIRE(workspace && workspace_bytes >= nnue_ls_tail_bwd_workspace_bytes(B, C), NNUE_ERR_WORKSPACE,
                 "nnue_ls_tail_bwd: workspace too small");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const LsPlanView v = ls_view(plan, B, C);
    float* part = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t)255);
    if (B > 0) {
        NNUE_REQUIRE(o1 && o2 && W2 && W3 && grad_y && d_o1, NNUE_ERR_ARG, "nnue_ls_tail_bwd: null tensor");
        k_ls_tail_bwd<<<(unsigned)ls_max_tiles(B, C), 256, 0, s>>>(o1, o2, v, W2, W3, grad_y, *params, d_o1, part);
        note_launches(1);
    }
    // with B == 0 the plan has no tiles and the sums below write zeros
    const dim3 grid((kPartW2 + kLsOut + kIn3 + 1 + 255) / 256, (unsigned)C);
    k_ls_tail_wsum<<<grid, 256, 0, s>>>(part, v, dW2, db2, dW3, db3);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
