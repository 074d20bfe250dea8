// Training loss and its gradient in one launch.
//
// Restates `calculate_sf_loss` and `remap_tablebase_score` (model/nnue.py:18-69
// of the reference project) together with the two elementwise steps that sit
// in front of it in the training step: the PSQT term of `NNUEModel.forward`
// (model/model.py:107-133: y + (wpsqt - bpsqt) * (us - 0.5)) and the scaling to
// centipawns (scorenet = y * nnue2score).  In the reference these are about
// forty elementwise kernels over [B, 1] tensors, forward and backward.
//
// Up to 64 CTAs compute every position's loss term, weight and the derivative
// of the term (written to d_y), with per-thread sums in double and a
// fixed-shape block reduction into one partial per CTA.  The CTA that
// finishes last (a counter in the workspace) adds the partials in CTA order,
// writes the loss and scales the derivatives by net_scale / sum(weights).
// The result does not depend on which CTA is last.
#include <algorithm>

#include "common.cuh"

namespace nnue {

constexpr int kLossThreads = 1024;
constexpr int kLossMaxCtas = 64;

struct LossWorkspace {
    unsigned int arrived;  // zero between launches
    unsigned int pad;
    double part_l[kLossMaxCtas], part_w[kLossMaxCtas];
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

__global__ void __launch_bounds__(kLossThreads)
    k_sf_loss(const float* __restrict__ y, const float* __restrict__ wpsqt, const float* __restrict__ bpsqt,
              const float* __restrict__ us, const float* __restrict__ score, const float* __restrict__ outcome,
              nnue_loss_params lp, float* __restrict__ loss, float* d_y, float* __restrict__ d_wpsqt,
              float* __restrict__ d_bpsqt, int64_t B, LossWorkspace* ws) {
    __shared__ double red_l[kLossThreads / 32], red_w[kLossThreads / 32];
    __shared__ double tot_w;
    __shared__ bool last;
    const int tid = threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * kLossThreads;
    const float w_gain = exp2f(lp.w1) - 1.f;
    double sum_l = 0.0, sum_w = 0.0;
    for (int64_t i = (int64_t)blockIdx.x * kLossThreads + tid; i < B; i += stride) {
        float net = y[i];
        if (wpsqt) net += (wpsqt[i] - bpsqt[i]) * (us[i] - 0.5f);
        const float sn = net * lp.net_scale;
        float sc = score[i];
        const float a = fabsf(sc);
        if (a >= 32000.f - 245.f) {  // tablebase / mate range: remapped by distance to mate
            const float r = lp.tb_remap_base + powf(lp.tb_remap_decay, fmaxf(32000.f - a, 0.f)) * lp.tb_remap_scale;
            sc = sc < 0.f ? -r : r;
        }
        const float sq = sigmoidf_((sn - lp.in_offset) / lp.in_scaling);
        const float sqm = sigmoidf_((-sn - lp.in_offset) / lp.in_scaling);
        const float qf = 0.5f * (1.f + sq - sqm);
        const float ss = sigmoidf_((sc - lp.out_offset) / lp.out_scaling);
        const float ssm = sigmoidf_((-sc - lp.out_offset) / lp.out_scaling);
        const float pf = 0.5f * (1.f + ss - ssm);
        const float pt = pf * lp.lambda + outcome[i] * (1.f - lp.lambda);
        const float d = pt - qf, ad = fabsf(d);
        float term = powf(ad, lp.pow_exp);
        float asym = 1.f;
        if (lp.qp_asymmetry != 0.f && qf > pt) asym = lp.qp_asymmetry + 1.f;
        term *= asym;
        const float h = pf - 0.5f;
        const float w = 1.f + w_gain * powf(h * h * pf * (1.f - pf), lp.w2);
        sum_l += (double)(term * w);
        sum_w += (double)w;
        if (d_y) {
            // d term / d qf = -p |d|^(p-1) sign(d) asym;  d qf / d sn = (sq(1-sq) + sqm(1-sqm)) / (2 in_scaling)
            const float sgn = d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
            const float dterm = ad > 0.f ? -lp.pow_exp * powf(ad, lp.pow_exp - 1.f) * sgn * asym : 0.f;
            const float dqf = 0.5f * (sq * (1.f - sq) + sqm * (1.f - sqm)) / lp.in_scaling;
            d_y[i] = w * dterm * dqf;
        }
    }
    __threadfence();  // this thread's d_y entries are visible device-wide before its CTA arrives
    // fixed-shape reduction: lanes by shuffle, then the 32 warp sums by warp 0
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sum_l += __shfl_down_sync(kFullMask, sum_l, o);
        sum_w += __shfl_down_sync(kFullMask, sum_w, o);
    }
    if ((tid & 31) == 0) {
        red_l[tid >> 5] = sum_l;
        red_w[tid >> 5] = sum_w;
    }
    __syncthreads();
    if (tid < 32) {
        sum_l = red_l[tid];
        sum_w = red_w[tid];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sum_l += __shfl_down_sync(kFullMask, sum_l, o);
            sum_w += __shfl_down_sync(kFullMask, sum_w, o);
        }
        if (tid == 0) {
            ws->part_l[blockIdx.x] = sum_l;
            ws->part_w[blockIdx.x] = sum_w;
            __threadfence();  // partials and this CTA's d_y before the arrival
            last = atomicAdd(&ws->arrived, 1u) == gridDim.x - 1;
        }
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (tid == 0) {
        double l = 0.0, w = 0.0;
        for (unsigned c = 0; c < gridDim.x; ++c) {  // CTA order, whichever CTA runs this
            l += __ldcg(&ws->part_l[c]);
            w += __ldcg(&ws->part_w[c]);
        }
        tot_w = w;
        *loss = (float)(l / w);
        ws->arrived = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!d_y) return;
    const float k = (float)((double)lp.net_scale / tot_w);
    for (int64_t i = tid; i < B; i += kLossThreads) {
        const float g = __ldcg(d_y + i) * k;
        d_y[i] = g;
        if (d_wpsqt) {
            const float gp = g * (us[i] - 0.5f);
            d_wpsqt[i] = gp;
            d_bpsqt[i] = -gp;
        }
    }
}

}  // namespace nnue

using namespace nnue;

extern "C" size_t nnue_sf_loss_workspace_bytes(void) { return sizeof(LossWorkspace); }

extern "C" int nnue_sf_loss(const float* y, const float* wpsqt, const float* bpsqt, const float* us,
                            const float* score, const float* outcome, const nnue_loss_params* h_params,
                            float* loss, float* d_y, float* d_wpsqt, float* d_bpsqt, void* workspace,
                            int64_t B, void* stream) {
    NNUE_REQUIRE(workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 7u) == 0, NNUE_ERR_ARG,
                 "nnue_sf_loss: null or misaligned workspace");
    NNUE_REQUIRE(h_params != nullptr && loss != nullptr && B > 0, NNUE_ERR_ARG,
                 "nnue_sf_loss: null parameters/loss or empty batch (B=%lld)", (long long)B);
    NNUE_REQUIRE(y && score && outcome, NNUE_ERR_ARG, "nnue_sf_loss: null input");
    NNUE_REQUIRE((wpsqt == nullptr) == (bpsqt == nullptr) && (wpsqt == nullptr || us != nullptr), NNUE_ERR_ARG,
                 "nnue_sf_loss: the PSQT term needs wpsqt, bpsqt and us together");
    NNUE_REQUIRE((d_wpsqt == nullptr) == (d_bpsqt == nullptr) && (d_wpsqt == nullptr || (d_y && wpsqt)),
                 NNUE_ERR_ARG, "nnue_sf_loss: PSQT gradients need d_y and the PSQT inputs");
    NNUE_REQUIRE(h_params->in_scaling != 0.f && h_params->out_scaling != 0.f, NNUE_ERR_ARG,
                 "nnue_sf_loss: zero scaling");
    const unsigned grid = (unsigned)std::min<int64_t>((B + kLossThreads - 1) / kLossThreads, kLossMaxCtas);
    k_sf_loss<<<grid, kLossThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        y, wpsqt, bpsqt, us, score, outcome, *h_params, loss, d_y, d_wpsqt, d_bpsqt, B,
        static_cast<LossWorkspace*>(workspace));
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
