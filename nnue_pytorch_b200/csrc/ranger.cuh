// Per-element RangerLite arithmetic shared by the single-GPU update kernels
// and the data-parallel shard update.  Follows the Python path of
// model/optimizers/ranger_lite.py:592-742 in the reference project.
#pragma once

#include "common.cuh"

namespace nnue {

using RangerConst = nnue_ranger_hparams;

__device__ __forceinline__ void ranger_elem(const RangerConst& c, float scale, float g, float& p,
                                            float& gm, float& ngm, float& vm, float& slow) {
    g = __fmul_rn(g, scale);
    if (c.phase != 2) vm = __fadd_rn(__fmul_rn(vm, c.beta2), __fmul_rn(c.one_minus_beta2, __fmul_rn(g, g)));
    if (c.phase == 1) return;
    const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(vm), c.bc2_sqrt), c.eps);
    float upd;
    if (c.use_pnm) {
        float pos = c.step_is_odd ? gm : ngm;
        const float neg = c.step_is_odd ? ngm : gm;
        pos = __fadd_rn(__fmul_rn(pos, c.mom), __fmul_rn(c.one_minus_mom, g));
        upd = __fmul_rn(__fadd_rn(__fmul_rn(pos, c.one_plus_f), __fmul_rn(-c.f, neg)), c.noise_norm_inv);
        if (c.step_is_odd) gm = pos; else ngm = pos;
    } else {
        gm = __fadd_rn(__fmul_rn(gm, c.mom), __fmul_rn(c.one_minus_mom, g));
        upd = gm;
    }
    float q = p;
    if (c.wd_keep != 1.f) q = __fmul_rn(q, c.wd_keep);
    q = __fadd_rn(q, __fmul_rn(-c.step_size, __fdiv_rn(upd, denom)));
    if (c.do_merge) {
        q = __fadd_rn(__fmul_rn(q, c.alpha), __fmul_rn(c.one_minus_alpha, slow));
        slow = q;
    }
    p = q;
}

// Returns the parameter values the element holds after the call.
__device__ __forceinline__ float4 ranger_vec4(const RangerConst& c, float scale, int64_t i,
                                              const float4* g4, float4* p4, float4* gm4, float4* ngm4,
                                              float4* vm4, float4* slow4, float4 gv) {
    float4 pv = p4[i], gmv = gm4[i], vmv = vm4[i];
    float4 ngv = c.use_pnm ? ngm4[i] : f4_zero();
    float4 sv = c.do_merge ? slow4[i] : f4_zero();
    ranger_elem(c, scale, gv.x, pv.x, gmv.x, ngv.x, vmv.x, sv.x);
    ranger_elem(c, scale, gv.y, pv.y, gmv.y, ngv.y, vmv.y, sv.y);
    ranger_elem(c, scale, gv.z, pv.z, gmv.z, ngv.z, vmv.z, sv.z);
    ranger_elem(c, scale, gv.w, pv.w, gmv.w, ngv.w, vmv.w, sv.w);
    if (c.phase != 2) vm4[i] = vmv;
    if (c.phase == 1) return p4[i];
    p4[i] = pv;
    if (!c.use_pnm || c.step_is_odd) gm4[i] = gmv;
    if (c.use_pnm && !c.step_is_odd) ngm4[i] = ngv;
    if (c.do_merge) slow4[i] = sv;
    (void)g4;
    return pv;
}

// The integer form of a table row group as nnue_ft_quantize_table writes it, from values already in
// registers: four L1 columns -> two packed int32 words, or four PSQT columns -> one fake-quantized float4.
struct TableEmit {
    int16_t* q16;
    float* psqt;
    int* stats;
    long long pitch4;   // q16 row pitch in groups of four int16
    int l4, p4;         // float4 per row: L1 part, PSQT part
    float scale_main, scale_psqt;
};

__device__ __forceinline__ void emit_group(const TableEmit& e, long long row, int c4, float4 v, int& bad, int& max_abs) {
    if (c4 < e.l4) {
        const float x[4] = {v.x, v.y, v.z, v.w};
        int k[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float r = rintf(__fmul_rn(x[j], e.scale_main));
            if (!(fabsf(r) <= 32767.f)) {
                ++bad;
                r = fminf(fmaxf(r, -32767.f), 32767.f);
                if (r != r) r = 0.f;
            }
            k[j] = (int)r;
            max_abs = max(max_abs, abs(k[j]));
        }
        reinterpret_cast<int2*>(e.q16)[row * e.pitch4 + c4] = make_int2(k[1] * 65536 + k[0], k[3] * 65536 + k[2]);
    } else {
        auto fq = [&](float a) { return __fdiv_rn(rintf(__fmul_rn(a, e.scale_psqt)), e.scale_psqt); };
        reinterpret_cast<float4*>(e.psqt)[row * e.p4 + (c4 - e.l4)] = make_float4(fq(v.x), fq(v.y), fq(v.z), fq(v.w));
    }
}

}  // namespace nnue
