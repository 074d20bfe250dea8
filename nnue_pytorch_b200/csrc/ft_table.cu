// One-pass preparation of the table the feature-transformer kernels read:
// fold the factor ("virtual") rows into the real rows and fake-quantize, and
// the matching backward for the factor rows.  Replaces the chain of dense
// elementwise passes the reference runs every step
// (model/modules/features/halfka_v2_hm.py:68-69 `weight + virtual.repeat(32, 1)`,
// model/modules/feature_transformer/composed_feature_transformer.py:61-76 with
// model/quantize.py:47-56: round(x * scale) / scale, two scales, a concat).
#include <math.h>

#include <algorithm>

#include "common.cuh"

namespace nnue {

__device__ __forceinline__ float fq1(float x, float scale) {
    return __fdiv_rn(rintf(__fmul_rn(x, scale)), scale);  // rintf: half to even, like torch.round
}
// Same value when `scale` is a power of two: dividing by it and multiplying by
// its reciprocal are both exact.
__device__ __forceinline__ float fq1_pow2(float x, float scale, float inv_scale) {
    return __fmul_rn(rintf(__fmul_rn(x, scale)), inv_scale);
}

// out[r, c] = fq(weight[r, c] + virtual[r % n_virtual, c]); thread = float4 (VEC) or float.
// IDX = unsigned when the element count fits 32 bits (cheap index division), else int64_t.
// inv_main > 0 marks a power-of-two main scale.
template <bool VEC, typename IDX>
__global__ void __launch_bounds__(kThreads)
    k_prepare_table(const float* __restrict__ weight, const float* __restrict__ virt,
                    float* __restrict__ out, int64_t N, int64_t n_virtual, int W, int L1,
                    float scale_main, float scale_psqt, float inv_main) {
    const IDX stride = (IDX)gridDim.x * blockDim.x;
    const IDX t0 = (IDX)blockIdx.x * blockDim.x + threadIdx.x;
    if (VEC) {
        const IDX W4 = (IDX)(W >> 2), L4 = (IDX)(L1 >> 2);  // a float4 never straddles the L1 | PSQT border
        const IDX n4 = (IDX)N * W4, nv = (IDX)n_virtual;
        const float4* w4 = reinterpret_cast<const float4*>(weight);
        const float4* v4 = reinterpret_cast<const float4*>(virt);
        float4* o4 = reinterpret_cast<float4*>(out);
        for (IDX i = t0; i < n4; i += stride) {
            const IDX r = i / W4;
            const IDX c4 = i - r * W4;
            float4 x = __ldcs(w4 + i);
            if (virt) x = f4_add(x, __ldg(v4 + (int64_t)(r % nv) * W4 + c4));
            if (scale_main > 0.f) {
                if (c4 >= L4) {
                    x = make_float4(fq1(x.x, scale_psqt), fq1(x.y, scale_psqt), fq1(x.z, scale_psqt),
                                    fq1(x.w, scale_psqt));
                } else if (inv_main > 0.f) {
                    x = make_float4(fq1_pow2(x.x, scale_main, inv_main), fq1_pow2(x.y, scale_main, inv_main),
                                    fq1_pow2(x.z, scale_main, inv_main), fq1_pow2(x.w, scale_main, inv_main));
                } else {
                    x = make_float4(fq1(x.x, scale_main), fq1(x.y, scale_main), fq1(x.z, scale_main),
                                    fq1(x.w, scale_main));
                }
            }
            o4[i] = x;
        }
    } else {
        const IDX n = (IDX)N * (IDX)W, nv = (IDX)n_virtual;
        for (IDX i = t0; i < n; i += stride) {
            const IDX r = i / (IDX)W;
            const int c = (int)(i - r * (IDX)W);
            float x = weight[i];
            if (virt) x = __fadd_rn(x, virt[(int64_t)(r % nv) * W + c]);
            if (scale_main > 0.f) x = fq1(x, c < L1 ? scale_main : scale_psqt);
            out[i] = x;
        }
    }
}

// The same table as integers: k[r, c] = rint((weight + virtual)[r, c] * scale_main) for the L1 columns,
// psqt[r, j] = fq(.., scale_psqt) for the PSQT columns (fp32, their scale is not a power of two).
// Neighbouring columns (c, c + 1), c even, are stored as the int32 NUMBER k[c + 1] * 65536 + k[c]: its
// low half is k[c] in two's complement, its high half k[c + 1] minus one when k[c] is negative, so that
// 32-bit adds of such words sum both columns (see ft_fused_q16.cu).  A value outside the int16 range is
// stored saturated and tallied in stats[0] (the reader then takes its fp32 route); stats[1] collects
// max |k|.  Thread = 8 consecutive columns (two float4 in, one 16-byte store out).
template <typename IDX>
__global__ void __launch_bounds__(kThreads)
    k_quantize_table(const float* __restrict__ weight, const float* __restrict__ virt,
                     int16_t* __restrict__ q16, int64_t pitch8, float* __restrict__ psqt, int64_t N,
                     int64_t n_virtual, int W, int L1, int P, float scale_main, float scale_psqt,
                     int* __restrict__ stats) {
    const IDX stride = (IDX)gridDim.x * blockDim.x;
    const IDX t0 = (IDX)blockIdx.x * blockDim.x + threadIdx.x;
    const IDX L8 = (IDX)(L1 >> 3), P4 = (IDX)(P >> 2);
    const IDX per_row = L8 + P4;                  // work items per row: 8-column groups, then PSQT float4
    const IDX total = (IDX)N * per_row, nv = (IDX)n_virtual;
    const int64_t W4 = W >> 2;
    const float4* w4 = reinterpret_cast<const float4*>(weight);
    const float4* v4 = reinterpret_cast<const float4*>(virt);
    int bad = 0, max_abs = 0;
    for (IDX i = t0; i < total; i += stride) {
        const IDX r = i / per_row;
        const IDX j = i - r * per_row;
        const float4* wrow = w4 + (int64_t)r * W4;
        const float4* vrow = virt ? v4 + (int64_t)(r % nv) * W4 : nullptr;
        if (j < L8) {
            float4 a = __ldcs(wrow + 2 * j), b = __ldcs(wrow + 2 * j + 1);
            if (virt) {
                a = f4_add(a, __ldg(vrow + 2 * j));
                b = f4_add(b, __ldg(vrow + 2 * j + 1));
            }
            const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            unsigned packed[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float lo = rintf(__fmul_rn(x[2 * k], scale_main)), hi = rintf(__fmul_rn(x[2 * k + 1], scale_main));
                if (!(fabsf(lo) <= 32767.f)) { ++bad; lo = fminf(fmaxf(lo, -32767.f), 32767.f); if (lo != lo) lo = 0.f; }
                if (!(fabsf(hi) <= 32767.f)) { ++bad; hi = fminf(fmaxf(hi, -32767.f), 32767.f); if (hi != hi) hi = 0.f; }
                packed[k] = (unsigned)((int)hi * 65536 + (int)lo);
                max_abs = max(max_abs, max(abs((int)lo), abs((int)hi)));
            }
            reinterpret_cast<uint4*>(q16)[(int64_t)r * pitch8 + j] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        } else {
            const IDX q = j - L8;
            float4 x = __ldcs(wrow + 2 * L8 + q);
            if (virt) x = f4_add(x, __ldg(vrow + 2 * L8 + q));
            x = make_float4(fq1(x.x, scale_psqt), fq1(x.y, scale_psqt), fq1(x.z, scale_psqt), fq1(x.w, scale_psqt));
            reinterpret_cast<float4*>(psqt)[(int64_t)r * P4 + q] = x;
        }
    }
    if (bad) atomicAdd(stats, bad);
    max_abs = __reduce_max_sync(kFullMask, max_abs);
    if ((threadIdx.x & 31) == 0 && max_abs > 0) atomicMax(stats + 1, max_abs);
}

// out[v, c] = sum over b of grad[b * n_virtual + v, c], b ascending.
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
    k_virtual_grad(const float* __restrict__ grad, float* __restrict__ out, int64_t repeats,
                   int64_t n_virtual, int W) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (VEC) {
        const int64_t per = n_virtual * (W >> 2);
        const float4* g4 = reinterpret_cast<const float4*>(grad);
        float4* o4 = reinterpret_cast<float4*>(out);
        for (int64_t i = t0; i < per; i += stride) {
            float4 s = __ldg(g4 + i);
            for (int64_t b = 1; b < repeats; ++b) s = f4_add(s, __ldg(g4 + b * per + i));
            o4[i] = s;
        }
    } else {
        const int64_t per = n_virtual * W;
        for (int64_t i = t0; i < per; i += stride) {
            float s = grad[i];
            for (int64_t b = 1; b < repeats; ++b) s = __fadd_rn(s, grad[b * per + i]);
            out[i] = s;
        }
    }
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_ft_prepare_table(const float* weight, const float* virtual_weight, float* out,
                                     int64_t N, int64_t n_virtual, int32_t L1, int32_t P,
                                     float scale_main, float scale_psqt, void* stream) {
    NNUE_REQUIRE(N >= 0 && L1 > 0 && P >= 0 && n_virtual >= 0, NNUE_ERR_ARG,
                 "nnue_ft_prepare_table: bad size");
    if (N == 0) return NNUE_OK;
    NNUE_REQUIRE(weight && out, NNUE_ERR_ARG, "nnue_ft_prepare_table: null pointer");
    NNUE_REQUIRE(!virtual_weight || (n_virtual > 0 && N % n_virtual == 0), NNUE_ERR_ARG,
                 "nnue_ft_prepare_table: N (%lld) is not a multiple of the factor rows (%lld)",
                 (long long)N, (long long)n_virtual);
    NNUE_REQUIRE(scale_main <= 0.f || scale_psqt > 0.f, NNUE_ERR_ARG,
                 "nnue_ft_prepare_table: both scales must be positive when quantizing");
    const int W = L1 + P;
    const bool vec = (W % 4 == 0) && (L1 % 4 == 0) && aligned16(weight) && aligned16(out) &&
                     (!virtual_weight || aligned16(virtual_weight));
    // power-of-two main scale (the usual 256): the division becomes an exact multiplication
    int exp2 = 0;
    const float inv_main = (scale_main > 0.f && frexpf(scale_main, &exp2) == 0.5f) ? 1.0f / scale_main : 0.f;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t work = vec ? N * (W / 4) : N * (int64_t)W;
    const unsigned grid = (unsigned)std::min<int64_t>((work + kThreads - 1) / kThreads, (int64_t)sm_count() * 16);
    const bool narrow = work + (int64_t)grid * kThreads < 0x7fffffffLL;  // index + stride stays below 2^31
    const int64_t nv = n_virtual ? n_virtual : 1;
#define LAUNCH_PREP(VV, II)                                                                              \
    k_prepare_table<VV, II><<<grid, kThreads, 0, s>>>(weight, virtual_weight, out, N, nv, W, L1, scale_main, \
                                                      scale_psqt, inv_main)
    ProfScope prof("k_prepare_table", s);
    if (vec && narrow) LAUNCH_PREP(true, unsigned);
    else if (vec) LAUNCH_PREP(true, int64_t);
    else if (narrow) LAUNCH_PREP(false, unsigned);
    else LAUNCH_PREP(false, int64_t);
#undef LAUNCH_PREP
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

extern "C" int nnue_ft_virtual_grad(const float* grad, float* out, int64_t N, int64_t n_virtual,
                                    int32_t W, void* stream) {
    NNUE_REQUIRE(N >= 0 && n_virtual > 0 && W > 0 && N % n_virtual == 0, NNUE_ERR_ARG,
                 "nnue_ft_virtual_grad: bad size");
    NNUE_REQUIRE(grad && out, NNUE_ERR_ARG, "nnue_ft_virtual_grad: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (N == 0) {
        NNUE_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)n_virtual * W * sizeof(float), s));
        return NNUE_OK;
    }
    const bool vec = (W % 4 == 0) && aligned16(grad) && aligned16(out);
    const int64_t work = vec ? n_virtual * (W / 4) : n_virtual * (int64_t)W;
    const unsigned grid = (unsigned)((work + kThreads - 1) / kThreads);
    if (vec) k_virtual_grad<true><<<grid, kThreads, 0, s>>>(grad, out, N / n_virtual, n_virtual, W);
    else k_virtual_grad<false><<<grid, kThreads, 0, s>>>(grad, out, N / n_virtual, n_virtual, W);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

// The bias of the int16 forward in one launch of one CTA: bias_fq[c] = round(bias[c] * scale) / scale for the L1
// columns (the bits of nnue_ft_prepare_table), zeros for the PSQT columns (that part of the bias never trains and
// the operator adds zeros), and the range statistics of the L1 part into stats (added to what is there, or
// written over it).
__global__ void __launch_bounds__(kThreads)
    k_bias_q16(const float* __restrict__ bias, float* __restrict__ out, int L1, int P, float scale, float inv_scale,
               int* __restrict__ stats, int overwrite) {
    __shared__ int s_bad[kWarpsPerCta], s_max[kWarpsPerCta];
    int bad = 0, mx = 0;
    for (int c = threadIdx.x; c < L1 + P; c += kThreads) {
        float v = 0.f;
        if (c < L1) {
            float r = rintf(__fmul_rn(__ldg(bias + c), scale));
            v = __fmul_rn(r, inv_scale);
            if (!(fabsf(r) <= 32767.f)) {
                ++bad;
                r = fminf(fmaxf(r, -32767.f), 32767.f);
                if (r != r) r = 0.f;
            }
            mx = max(mx, abs((int)r));
        }
        out[c] = v;
    }
    bad = __reduce_add_sync(kFullMask, bad);
    mx = __reduce_max_sync(kFullMask, mx);
    if ((threadIdx.x & 31) == 0) {
        s_bad[threadIdx.x >> 5] = bad;
        s_max[threadIdx.x >> 5] = mx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kWarpsPerCta; ++w) {
            bad += s_bad[w];
            mx = max(mx, s_max[w]);
        }
        if (overwrite) {
            stats[0] = bad;
            stats[1] = mx;
        } else {
            if (bad) atomicAdd(stats, bad);
            if (mx > 0) atomicMax(stats + 1, mx);
        }
    }
}

extern "C" int nnue_ft_prepare_bias_q16(const float* bias, float* bias_fq, int32_t L1, int32_t P, float scale_main,
                                        int32_t* d_stats, int32_t overwrite_stats, void* stream) {
    NNUE_REQUIRE(L1 > 0 && P >= 0 && bias && bias_fq && d_stats, NNUE_ERR_ARG, "nnue_ft_prepare_bias_q16: bad argument");
    int exp2 = 0;
    NNUE_REQUIRE(scale_main > 0.f && frexpf(scale_main, &exp2) == 0.5f, NNUE_ERR_UNSUPPORTED,
                 "nnue_ft_prepare_bias_q16: the scale must be a power of two (got %g)", (double)scale_main);
    k_bias_q16<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(bias, bias_fq, L1, P, scale_main, 1.0f / scale_main,
                                                                     d_stats, overwrite_stats);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

extern "C" int nnue_ft_quantize_table(const float* weight, const float* virtual_weight, int16_t* q16,
                                      int64_t q16_pitch, float* psqt, int64_t N, int64_t n_virtual, int32_t L1,
                                      int32_t P, float scale_main, float scale_psqt, int32_t* d_overflow,
                                      void* stream) {
    NNUE_REQUIRE(N >= 0 && L1 > 0 && P >= 0 && n_virtual >= 0, NNUE_ERR_ARG, "nnue_ft_quantize_table: bad size");
    NNUE_REQUIRE(L1 % 8 == 0 && P % 4 == 0, NNUE_ERR_UNSUPPORTED,
                 "nnue_ft_quantize_table: needs L1 %% 8 == 0 and P %% 4 == 0 (L1=%d P=%d)", L1, P);
    NNUE_REQUIRE(q16_pitch >= L1 && q16_pitch % 8 == 0, NNUE_ERR_ARG,
                 "nnue_ft_quantize_table: the row pitch (%lld) must be a multiple of 8 not below L1", (long long)q16_pitch);
    int exp2 = 0;
    NNUE_REQUIRE(scale_main > 0.f && frexpf(scale_main, &exp2) == 0.5f && scale_psqt > 0.f, NNUE_ERR_UNSUPPORTED,
                 "nnue_ft_quantize_table: the main scale must be a power of two (got %g)", (double)scale_main);
    if (N == 0) return NNUE_OK;
    NNUE_REQUIRE(weight && q16 && d_overflow && (psqt || P == 0), NNUE_ERR_ARG, "nnue_ft_quantize_table: null pointer");
    NNUE_REQUIRE(!virtual_weight || (n_virtual > 0 && N % n_virtual == 0), NNUE_ERR_ARG,
                 "nnue_ft_quantize_table: N (%lld) is not a multiple of the factor rows (%lld)", (long long)N,
                 (long long)n_virtual);
    NNUE_REQUIRE(aligned16(weight) && aligned16(q16) && aligned16(psqt) && (!virtual_weight || aligned16(virtual_weight)),
                 NNUE_ERR_ALIGN, "nnue_ft_quantize_table: 16-byte aligned buffers");
    const int W = L1 + P;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t work = N * (int64_t)(L1 / 8 + P / 4);
    const unsigned grid = (unsigned)std::min<int64_t>((work + kThreads - 1) / kThreads, (int64_t)sm_count() * 16);
    const bool narrow = work + (int64_t)grid * kThreads < 0x7fffffffLL;
    const int64_t nv = n_virtual ? n_virtual : 1;
    ProfScope prof("k_quantize_table", s);
    if (narrow)
        k_quantize_table<unsigned><<<grid, kThreads, 0, s>>>(weight, virtual_weight, q16, q16_pitch / 8, psqt, N, nv, W,
                                                            L1, P, scale_main, scale_psqt, d_overflow);
    else
        k_quantize_table<int64_t><<<grid, kThreads, 0, s>>>(weight, virtual_weight, q16, q16_pitch / 8, psqt, N, nv, W,
                                                           L1, P, scale_main, scale_psqt, d_overflow);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
