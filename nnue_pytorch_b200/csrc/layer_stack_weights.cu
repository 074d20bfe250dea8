// Effective weights of the bucketed layer stack for one training step.
//
// The reference builds them with elementwise torch ops before every forward
// (model/modules/stacked_linear.py:96-127: `linear.weight +
// factorized_linear.weight.repeat(count, 1)`, same for the bias; then
// model/quantize.py:49-50 `round(w * scale) / scale` with a straight-through
// gradient on each of the six tensors): about forty launches over small
// tensors.  Here: one launch writes all six effective tensors, and one launch
// folds the gradient of the first layer back onto the shared factor layer
// (sum over buckets, bucket order).  Every other gradient passes through
// unchanged, so it needs no kernel.
#include <algorithm>

#include "layer_stack.cuh"

namespace nnue {

struct LsWeightJob {
    const float* l1_w;   // [C*32, L1]
    const float* l1_b;   // [C*32]
    const float* l1f_w;  // [32, L1] or null
    const float* l1f_b;  // [32] or null
    const float* l2_w;   // [C*32, 64]
    const float* l2_b;   // [C*32]
    const float* out_w;  // [C, 128]
    const float* out_b;  // [C]
    float *w1, *b1, *w2, *b2, *w3, *b3;
    int64_t n_w1, n_b1, n_w2, n_b2, n_w3, n_b3;
    int64_t f_w, f_b;  // elements of the factor tensors (period of the repeat)
    nnue_ls_weight_scales sc;
};

__device__ __forceinline__ float fq_weight(float v, float scale, int on) {
    return on ? __fdiv_rn(rintf(__fmul_rn(v, scale)), scale) : v;  // rintf: half to even, as torch.round
}

__global__ void __launch_bounds__(256) k_ls_effective_weights(LsWeightJob j) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int q = j.sc.quantize;
    for (int64_t i = t0; i < j.n_w1; i += stride) {
        float v = j.l1_w[i];
        if (j.l1f_w) v = __fadd_rn(v, __ldg(j.l1f_w + i % j.f_w));
        j.w1[i] = fq_weight(v, j.sc.w1, q);
    }
    for (int64_t i = t0; i < j.n_b1; i += stride) {
        float v = j.l1_b[i];
        if (j.l1f_b) v = __fadd_rn(v, __ldg(j.l1f_b + i % j.f_b));
        j.b1[i] = fq_weight(v, j.sc.b1, q);
    }
    for (int64_t i = t0; i < j.n_w2; i += stride) j.w2[i] = fq_weight(j.l2_w[i], j.sc.w2, q);
    for (int64_t i = t0; i < j.n_b2; i += stride) j.b2[i] = fq_weight(j.l2_b[i], j.sc.b2, q);
    for (int64_t i = t0; i < j.n_w3; i += stride) j.w3[i] = fq_weight(j.out_w[i], j.sc.w3, q);
    for (int64_t i = t0; i < j.n_b3; i += stride) j.b3[i] = fq_weight(j.out_b[i], j.sc.b3, q);
}

// d_l1f_w[r, c] = sum over buckets of dW1[bucket*32 + r, c]; the bias likewise.
__global__ void __launch_bounds__(256)
    k_ls_fold_grads(const float* __restrict__ dW1, const float* __restrict__ db1, float* __restrict__ d_f_w,
                    float* __restrict__ d_f_b, int64_t f_w, int64_t f_b, int C) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < f_w) {
        float s = dW1[i];
        for (int c = 1; c < C; ++c) s = __fadd_rn(s, dW1[(int64_t)c * f_w + i]);
        d_f_w[i] = s;
    } else if (i < f_w + f_b) {
        const int64_t k = i - f_w;
        float s = db1[k];
        for (int c = 1; c < C; ++c) s = __fadd_rn(s, db1[(int64_t)c * f_b + k]);
        d_f_b[k] = s;
    }
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_ls_effective_weights(const float* l1_w, const float* l1_b, const float* l1f_w,
                                         const float* l1f_b, const float* l2_w, const float* l2_b,
                                         const float* out_w, const float* out_b,
                                         const nnue_ls_weight_scales* h_scales, float* w1, float* b1, float* w2,
                                         float* b2, float* w3, float* b3, int32_t L1, int32_t C, void* stream) {
    NNUE_REQUIRE(h_scales != nullptr && L1 > 0 && C > 0 && C <= 16, NNUE_ERR_ARG,
                 "nnue_ls_effective_weights: bad shape (L1=%d C=%d) or null scales", L1, C);
    NNUE_REQUIRE(l1_w && l1_b && l2_w && l2_b && out_w && out_b && w1 && b1 && w2 && b2 && w3 && b3, NNUE_ERR_ARG,
                 "nnue_ls_effective_weights: null tensor");
    NNUE_REQUIRE((l1f_w == nullptr) == (l1f_b == nullptr), NNUE_ERR_ARG,
                 "nnue_ls_effective_weights: factor weight and bias come together");
    if (h_scales->quantize) {
        NNUE_REQUIRE(h_scales->w1 > 0 && h_scales->b1 > 0 && h_scales->w2 > 0 && h_scales->b2 > 0 &&
                         h_scales->w3 > 0 && h_scales->b3 > 0,
                     NNUE_ERR_ARG, "nnue_ls_effective_weights: scales must be positive");
    }
    LsWeightJob j;
    j.l1_w = l1_w, j.l1_b = l1_b, j.l1f_w = l1f_w, j.l1f_b = l1f_b;
    j.l2_w = l2_w, j.l2_b = l2_b, j.out_w = out_w, j.out_b = out_b;
    j.w1 = w1, j.b1 = b1, j.w2 = w2, j.b2 = b2, j.w3 = w3, j.b3 = b3;
    j.f_w = (int64_t)kLsOut * L1, j.f_b = kLsOut;
    j.n_w1 = (int64_t)C * j.f_w, j.n_b1 = (int64_t)C * kLsOut;
    j.n_w2 = (int64_t)C * kLsOut * 2 * kLsOut, j.n_b2 = (int64_t)C * kLsOut;
    j.n_w3 = (int64_t)C * 4 * kLsOut, j.n_b3 = C;
    j.sc = *h_scales;
    const unsigned grid = (unsigned)std::min<int64_t>((j.n_w1 + 255) / 256, 4 * (int64_t)sm_count());
    k_ls_effective_weights<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(j);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

extern "C" int nnue_ls_fold_grads(const float* dW1, const float* db1, float* d_l1f_w, float* d_l1f_b, int32_t L1,
                                  int32_t C, void* stream) {
    NNUE_REQUIRE(dW1 && db1 && d_l1f_w && d_l1f_b && L1 > 0 && C > 0 && C <= 16, NNUE_ERR_ARG,
                 "nnue_ls_fold_grads: null tensor or bad shape (L1=%d C=%d)", L1, C);
    const int64_t f_w = (int64_t)kLsOut * L1, f_b = kLsOut;
    const unsigned grid = (unsigned)((f_w + f_b + 255) / 256);
    k_ls_fold_grads<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(dW1, db1, d_l1f_w, d_l1f_b, f_w, f_b, C);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
