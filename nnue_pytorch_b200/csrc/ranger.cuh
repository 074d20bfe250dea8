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

__device__ __forceinline__ void ranger_vec4(const RangerConst& c, float scale, int64_t i,
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
    if (c.phase == 1) return;
    p4[i] = pv;
    if (!c.use_pnm || c.step_is_odd) gm4[i] = gmv;
    if (c.use_pnm && !c.step_is_odd) ngm4[i] = ngv;
    if (c.do_merge) slow4[i] = sv;
    (void)g4;
}

}  // namespace nnue
