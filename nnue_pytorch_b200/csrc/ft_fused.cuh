// Device helpers shared by the forward kernels of the fused double feature
// transformer (fp32 table: ft_fused.cu; int16 table: ft_fused_q16.cu).
#pragma once

#include <math.h>

#include "gather.cuh"

namespace nnue {

// Activation constants of one call: clamp bound, optional fake quantization of
// the pairwise product (floor(x * act_scale + act_eps) / act_scale, the
// reference's `fake_quantize_ft_act`, model/quantize.py:36-45) and the
// correction factor applied after it (composed_feature_transformer.py:143-149).
struct FtAct {
    float max_act;
    float act_scale;  // 0 = no fake quantization
    float act_eps;
    float out_scale;  // 1 = none
    float act_inv;    // 1 / act_scale when that is exact (power of two), else 0
};

__device__ __forceinline__ float finish_l0(float x, const FtAct& a) {
    if (a.act_scale > 0.f) {
        const float q = floorf(__fadd_rn(__fmul_rn(x, a.act_scale), a.act_eps));
        x = a.act_inv != 0.f ? __fmul_rn(q, a.act_inv) : __fdiv_rn(q, a.act_scale);
    }
    if (a.out_scale != 1.f) x = __fmul_rn(x, a.out_scale);
    return x;
}

// ---------------------------------------------------------------------------
// index staging: the K-entry lists of the 8 positions of a CTA are contiguous
// in global memory (8*K*4 bytes per perspective); one elected thread pulls
// both blocks into shared memory with two 1-D bulk copies on one mbarrier.
// ---------------------------------------------------------------------------
struct StagedLists {
    const int32_t* w;  // this warp's white list
    const int32_t* b;  // this warp's black list
};

__device__ __forceinline__ StagedLists stage_lists(const int32_t* __restrict__ wi,
                                                   const int32_t* __restrict__ bi, int64_t p0,
                                                   int64_t B, int K, bool want_stage,
                                                   int32_t* s_idx, uint64_t* bar, int warp,
                                                   unsigned long long* status) {
    StagedLists out;
    const int64_t p = p0 + warp;
    out.w = wi + p * K;
    out.b = bi + p * K;
    // Full CTAs only: the block is 8*K*4 bytes = a multiple of 32; the host
    // already checked the 16-byte alignment of the base pointers.
    const bool stage = want_stage && (p0 + kWarpsPerCta <= B);
    if (!stage) return out;  // uniform across the CTA

    const unsigned bytes = (unsigned)(kWarpsPerCta * K * sizeof(int32_t));
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, 2 * bytes);
        bulk_g2s(s_idx, wi + p0 * K, bytes, bar);
        bulk_g2s(s_idx + kWarpsPerCta * K, bi + p0 * K, bytes, bar);
    }
    const bool landed = mbar_wait_bounded(bar, 0);
    if (landed) {
        out.w = s_idx + warp * K;
        out.b = s_idx + (kWarpsPerCta + warp) * K;
    } else if ((threadIdx.x & 31) == 0) {
        note_timeout(status);  // keep going on the global-memory lists
    }
    return out;
}

// Sequential (bias first, k ascending) sum of one scalar column over the
// listed rows; loads are spread over the lanes, the adds are ordered.
__device__ __forceinline__ float psqt_sum(const float* __restrict__ weight, int64_t W,
                                          int64_t n_rows, const int32_t* list, int n, int colidx,
                                          float init, int lane) {
    float s = init;
    for (int k0 = 0; k0 < n; k0 += 32) {
        const int m = min(32, n - k0);
        float v = 0.f;
        bool live = false;
        if (lane < m) {
            const int r = list[k0 + lane];
            live = (unsigned)r < (unsigned long long)n_rows;
            if (live) v = __ldg(weight + (int64_t)r * W + colidx);
        }
        const unsigned lives = __ballot_sync(kFullMask, live);
        for (int j = 0; j < m; ++j) {
            const float x = __shfl_sync(kFullMask, v, j);
            if ((lives >> j) & 1u) s = __fadd_rn(s, x);
        }
    }
    return s;
}

// One float4 column `c` of the first half with its partner column h4 + c of the second half:
// mix the two perspectives by side to move, keep the pre-clamp values for the backward, write
// the clipped pairwise products (optionally fake-quantized and scaled).
__device__ __forceinline__ void ft_store_columns(float u_, float t_, float4 w_lo, float4 w_hi, float4 b_lo,
                                                 float4 b_hi, int c, int h4, float4* sv, float4* l0p,
                                                 const FtAct& act) {
    const float4 x0 = f4_mix(u_, w_lo, t_, b_lo);
    const float4 x1 = f4_mix(u_, w_hi, t_, b_hi);
    const float4 x2 = f4_mix(u_, b_lo, t_, w_lo);
    const float4 x3 = f4_mix(u_, b_hi, t_, w_hi);
    st_stream4(sv + 0 * h4 + c, x0);
    st_stream4(sv + 1 * h4 + c, x1);
    st_stream4(sv + 2 * h4 + c, x2);
    st_stream4(sv + 3 * h4 + c, x3);
    const float max_act = act.max_act;
    auto cl = [max_act](float x) { return fminf(fmaxf(x, 0.f), max_act); };
    auto pr = [&](float p, float q) { return finish_l0(__fmul_rn(cl(p), cl(q)), act); };
    const float4 a = make_float4(pr(x0.x, x1.x), pr(x0.y, x1.y), pr(x0.z, x1.z), pr(x0.w, x1.w));
    const float4 b = make_float4(pr(x2.x, x3.x), pr(x2.y, x3.y), pr(x2.z, x3.z), pr(x2.w, x3.w));
    st_stream4(l0p + c, a);
    st_stream4(l0p + h4 + c, b);
}

}  // namespace nnue
