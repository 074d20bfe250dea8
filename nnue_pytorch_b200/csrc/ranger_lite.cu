// Fused RangerLite update: Adam second moment, positive-negative momentum,
// optional stable weight decay, parameter step and lookahead merge in one
// pass over the tensor (5 reads + 3 writes of 4 bytes per element, +2/+1 on a
// merge step).  Arithmetic follows model/optimizers/ranger_lite.py:592-742 of
// the reference project (its Python path); replaces its CuPy kernels (:46-201)
// and the separate lookahead pass (:746-768).
#include <algorithm>

#include "ranger.cuh"

namespace nnue {

// Flat tensor: grid-stride over float4 (VEC) or scalars.
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
    k_ranger_flat(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ gm,
                  float* __restrict__ ngm, float* __restrict__ vm, float* __restrict__ slow,
                  const float* __restrict__ d_scale, int64_t n, RangerConst c) {
    const float scale = d_scale ? __ldg(d_scale) : 1.f;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t done = 0;
    if (VEC) {
        const int64_t n4 = n >> 2;
        const float4* g4 = reinterpret_cast<const float4*>(g);
        for (int64_t i = t0; i < n4; i += stride)
            ranger_vec4(c, scale, i, g4, reinterpret_cast<float4*>(p), reinterpret_cast<float4*>(gm),
                        reinterpret_cast<float4*>(ngm), reinterpret_cast<float4*>(vm),
                        reinterpret_cast<float4*>(slow), __ldg(g4 + i));
        done = n4 << 2;
    }
    for (int64_t i = done + t0; i < n; i += stride) {
        float pv = p[i], gmv = gm[i], vmv = vm[i];
        float ngv = c.use_pnm ? ngm[i] : 0.f, sv = c.do_merge ? slow[i] : 0.f;
        ranger_elem(c, scale, g[i], pv, gmv, ngv, vmv, sv);
        if (c.phase != 2) vm[i] = vmv;
        if (c.phase == 1) continue;
        p[i] = pv;
        if (!c.use_pnm || c.step_is_odd) gm[i] = gmv;
        if (c.use_pnm && !c.step_is_odd) ngm[i] = ngv;
        if (c.do_merge) slow[i] = sv;
    }
}

// Touched-rows-only rule, in two kernels.  A row whose flag is clear and whose
// gradient row is all zero is left alone: all of its moments are zero, so the
// full update would rewrite the same bits.
//   k_rows_activate  one warp per row that is still inactive: any non-zero
//                    gradient element sets the flag for good;
//   k_ranger_rows    the flat update, skipping float4 of inactive rows.
__global__ void __launch_bounds__(kThreads)
    k_rows_activate(const float* __restrict__ g, uint8_t* __restrict__ row_active, int64_t rows,
                    int64_t width4) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (row >= rows || row_active[row]) return;  // warp-uniform
    // rows that never get a gradient (features no legal position has) stay inactive for good and are scanned in
    // full every step: eight independent loads per trip, so that a scan costs three load latencies, not 24
    const float4* g4 = reinterpret_cast<const float4*>(g) + row * width4;
    int nz = 0;
    for (int64_t c0 = 0; c0 < width4 && !nz; c0 += 8 * 32) {
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int64_t c = c0 + 32 * i + lane;
            v[i] = c < width4 ? __ldg(g4 + c) : f4_zero();
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) nz |= (v[i].x != 0.f) | (v[i].y != 0.f) | (v[i].z != 0.f) | (v[i].w != 0.f);
        nz = __any_sync(kFullMask, nz);
    }
    if (nz && lane == 0) row_active[row] = 1;
}

// IDX = unsigned when the float4 count (plus one grid stride) fits 32 bits: cheap row lookup.
// EMIT: the new parameter values also leave the kernel as the integer table the next forward gathers
// (nnue_ft_quantize_table's format), which saves that pass its read of the whole table; rows the update
// skips are emitted from the values they hold.
template <typename IDX, bool EMIT>
__global__ void __launch_bounds__(kThreads)
    k_ranger_rows(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ gm,
                  float* __restrict__ ngm, float* __restrict__ vm, float* __restrict__ slow,
                  const uint8_t* __restrict__ row_active, const float* __restrict__ d_scale, int64_t rows,
                  int64_t width4, RangerConst c, TableEmit emit) {
    const float scale = d_scale ? __ldg(d_scale) : 1.f;
    const float4* g4 = reinterpret_cast<const float4*>(g);
    const IDX w4 = (IDX)width4;
    const IDX n4 = (IDX)rows * w4;
    const IDX stride = (IDX)gridDim.x * blockDim.x;
    int bad = 0, max_abs = 0;
    for (IDX i = (IDX)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const IDX row = i / w4;
        float4 pv;
        if (__ldg(row_active + row)) {
            pv = ranger_vec4(c, scale, (int64_t)i, g4, reinterpret_cast<float4*>(p), reinterpret_cast<float4*>(gm),
                             reinterpret_cast<float4*>(ngm), reinterpret_cast<float4*>(vm),
                             reinterpret_cast<float4*>(slow), __ldg(g4 + i));
        } else {
            if (!EMIT) continue;
            pv = reinterpret_cast<const float4*>(p)[i];
        }
        if (EMIT) emit_group(emit, (long long)row, (int)(i - row * w4), pv, bad, max_abs);
    }
    if (EMIT) {
        if (bad) atomicAdd(emit.stats, bad);
        max_abs = __reduce_max_sync(kFullMask, max_abs);
        if ((threadIdx.x & 31) == 0 && max_abs > 0) atomicMax(emit.stats + 1, max_abs);
    }
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
    k_lookahead(float* __restrict__ p, float* __restrict__ slow, int64_t n, float alpha,
                float one_minus_alpha) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t done = 0;
    auto f = [alpha, one_minus_alpha](float a, float b) {
        return __fadd_rn(__fmul_rn(a, alpha), __fmul_rn(one_minus_alpha, b));
    };
    if (VEC) {
        const int64_t n4 = n >> 2;
        float4* p4 = reinterpret_cast<float4*>(p);
        float4* s4 = reinterpret_cast<float4*>(slow);
        for (int64_t i = t0; i < n4; i += stride) {
            const float4 a = p4[i], b = s4[i];
            const float4 r = make_float4(f(a.x, b.x), f(a.y, b.y), f(a.z, b.z), f(a.w, b.w));
            p4[i] = r;
            s4[i] = r;
        }
        done = n4 << 2;
    }
    for (int64_t i = done + t0; i < n; i += stride) {
        const float r = f(p[i], slow[i]);
        p[i] = r;
        slow[i] = r;
    }
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_rangerlite_update(float* p, const float* grad, float* grad_ma,
                                      float* neg_grad_ma, float* variance_ma, float* slow,
                                      uint8_t* row_active, const float* d_grad_scale, int64_t rows,
                                      int64_t width, const nnue_ranger_hparams* hp, void* stream) {
    return nnue_rangerlite_update_emit(p, grad, grad_ma, neg_grad_ma, variance_ma, slow, row_active, d_grad_scale,
                                       rows, width, hp, nullptr, stream);
}

extern "C" int nnue_rangerlite_update_emit(float* p, const float* grad, float* grad_ma,
                                           float* neg_grad_ma, float* variance_ma, float* slow,
                                           uint8_t* row_active, const float* d_grad_scale, int64_t rows,
                                           int64_t width, const nnue_ranger_hparams* hp,
                                           const nnue_table_emit* h_emit, void* stream) {
    NNUE_REQUIRE(hp != nullptr, NNUE_ERR_ARG, "nnue_rangerlite_update: null hyper-parameters");
    if (h_emit) {
        int e2 = 0;
        NNUE_REQUIRE(h_emit->q16 && h_emit->d_stats && (h_emit->psqt || h_emit->P == 0), NNUE_ERR_ARG,
                     "nnue_rangerlite_update_emit: null table pointer");
        NNUE_REQUIRE(h_emit->L1 > 0 && h_emit->L1 % 8 == 0 && h_emit->P >= 0 && h_emit->P % 4 == 0 &&
                         (int64_t)h_emit->L1 + h_emit->P == width,
                     NNUE_ERR_ARG, "nnue_rangerlite_update_emit: L1 + P must be the tensor's width (L1 %% 8, P %% 4)");
        NNUE_REQUIRE(h_emit->q16_pitch >= h_emit->L1 && h_emit->q16_pitch % 8 == 0, NNUE_ERR_ARG,
                     "nnue_rangerlite_update_emit: bad row pitch");
        NNUE_REQUIRE(h_emit->scale_main > 0.f && frexpf(h_emit->scale_main, &e2) == 0.5f && h_emit->scale_psqt > 0.f,
                     NNUE_ERR_UNSUPPORTED, "nnue_rangerlite_update_emit: the main scale must be a power of two");
        NNUE_REQUIRE(aligned16(h_emit->q16) && aligned16(h_emit->psqt), NNUE_ERR_ALIGN,
                     "nnue_rangerlite_update_emit: 16-byte aligned table buffers");
    }
    NNUE_REQUIRE(rows >= 0 && width >= 0, NNUE_ERR_ARG, "nnue_rangerlite_update: negative size");
    const int64_t n = rows * width;
    if (n == 0) return NNUE_OK;
    NNUE_REQUIRE(p && grad && grad_ma && variance_ma, NNUE_ERR_ARG, "nnue_rangerlite_update: null tensor");
    NNUE_REQUIRE(!hp->use_pnm || neg_grad_ma, NNUE_ERR_ARG, "nnue_rangerlite_update: PNM needs neg_grad_ma");
    NNUE_REQUIRE(!hp->do_merge || slow, NNUE_ERR_ARG, "nnue_rangerlite_update: merge needs the slow copy");
    NNUE_REQUIRE(hp->phase >= 0 && hp->phase <= 2, NNUE_ERR_ARG, "nnue_rangerlite_update: bad phase");
    RangerConst c = *hp;
    if (c.phase == 1) c.do_merge = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool al = aligned16(p) && aligned16(grad) && aligned16(grad_ma) && aligned16(variance_ma) &&
                    (!neg_grad_ma || aligned16(neg_grad_ma)) && (!slow || aligned16(slow));
    const int sms = sm_count();
    bool emitted = false;
    if (row_active && al && width % 4 == 0 && hp->phase != 1) {
        k_rows_activate<<<(unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta), kThreads, 0, s>>>(
            grad, row_active, rows, width / 4);
        const unsigned grid = (unsigned)std::min<int64_t>((n / 4 + kThreads - 1) / kThreads, (int64_t)sms * 8);
        TableEmit te{};
        if (h_emit) {
            te = TableEmit{h_emit->q16, h_emit->psqt, h_emit->d_stats, h_emit->q16_pitch / 4, h_emit->L1 / 4,
                           h_emit->P / 4, h_emit->scale_main, h_emit->scale_psqt};
            NNUE_CUDA_TRY(cudaMemsetAsync(h_emit->d_stats, 0, 2 * sizeof(int32_t), s));
            emitted = true;
        }
        const bool narrow = n / 4 + (int64_t)grid * kThreads < 0x7fffffffLL;
        ProfScope prof("k_ranger_rows", s);
#define LAUNCH_ROWS(II, EE)                                                                                       \
    k_ranger_rows<II, EE><<<grid, kThreads, 0, s>>>(p, grad, grad_ma, neg_grad_ma, variance_ma, slow, row_active, \
                                                    d_grad_scale, rows, width / 4, c, te)
        if (narrow && h_emit) LAUNCH_ROWS(unsigned, true);
        else if (narrow) LAUNCH_ROWS(unsigned, false);
        else if (h_emit) LAUNCH_ROWS(int64_t, true);
        else LAUNCH_ROWS(int64_t, false);
#undef LAUNCH_ROWS
        note_launches(1);
    } else {
        const int64_t work = al ? (n / 4 + 1) : n;
        const unsigned grid = (unsigned)std::min<int64_t>((work + kThreads - 1) / kThreads, (int64_t)sms * 8);
        if (al)
            k_ranger_flat<true><<<grid, kThreads, 0, s>>>(p, grad, grad_ma, neg_grad_ma, variance_ma, slow,
                                                         d_grad_scale, n, c);
        else
            k_ranger_flat<false><<<grid, kThreads, 0, s>>>(p, grad, grad_ma, neg_grad_ma, variance_ma,
                                                          slow, d_grad_scale, n, c);
    }
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    if (h_emit && !emitted) {  // shapes the row kernel does not take: the table in a pass of its own
        NNUE_CUDA_TRY(cudaMemsetAsync(h_emit->d_stats, 0, 2 * sizeof(int32_t), s));
        return nnue_ft_quantize_table(p, nullptr, h_emit->q16, h_emit->q16_pitch, h_emit->psqt, rows, 0, h_emit->L1,
                                      h_emit->P, h_emit->scale_main, h_emit->scale_psqt, h_emit->d_stats, stream);
    }
    return NNUE_OK;
}

extern "C" int nnue_lookahead_merge(float* p, float* slow, int64_t n, float alpha, void* stream) {
    NNUE_REQUIRE(n >= 0, NNUE_ERR_ARG, "nnue_lookahead_merge: negative size");
    if (n == 0) return NNUE_OK;
    NNUE_REQUIRE(p && slow, NNUE_ERR_ARG, "nnue_lookahead_merge: null tensor");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool al = aligned16(p) && aligned16(slow);
    const int64_t work = al ? (n / 4 + 1) : n;
    const unsigned grid = (unsigned)std::min<int64_t>((work + kThreads - 1) / kThreads, (int64_t)sm_count() * 8);
    if (al) k_lookahead<true><<<grid, kThreads, 0, s>>>(p, slow, n, alpha, 1.0f - alpha);
    else k_lookahead<false><<<grid, kThreads, 0, s>>>(p, slow, n, alpha, 1.0f - alpha);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
