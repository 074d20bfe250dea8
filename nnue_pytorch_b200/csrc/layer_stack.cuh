// Shared declarations of the bucketed layer-stack kernels: the batch plan
// (positions grouped by bucket into tiles) and the activation constants.
#pragma once

#include "common.cuh"

namespace nnue {

constexpr int kTP = 64;     // positions per tile
constexpr int kLsOut = 32;  // L2 = L3: one lane per output in the tail kernels

struct LsPlanView {
    const int32_t* n_tiles;      // [1]
    const int32_t* bucket_tile;  // [C + 1] first tile of each bucket
    const int32_t* tile_start;   // [T] offset into perm
    const int32_t* tile_count;   // [T] 1..kTP
    const int32_t* tile_bucket;  // [T]
    const int32_t* perm;         // [B] positions grouped by bucket, ascending inside a bucket
};

__host__ __device__ inline int64_t ls_max_tiles(int64_t B, int C) { return (B + kTP - 1) / kTP + C; }

__host__ __device__ inline int64_t ls_plan_ints(int64_t B, int C) {
    return 4 + (C + 1 + 3) / 4 * 4 + 3 * ls_max_tiles(B, C) + B;
}

__host__ __device__ inline LsPlanView ls_view(const void* plan, int64_t B, int C) {
    const int32_t* p = static_cast<const int32_t*>(plan);
    const int64_t T = ls_max_tiles(B, C);
    LsPlanView v;
    v.n_tiles = p;
    v.bucket_tile = p + 4;
    v.tile_start = v.bucket_tile + (C + 1 + 3) / 4 * 4;
    v.tile_count = v.tile_start + T;
    v.tile_bucket = v.tile_count + T;
    v.perm = v.tile_bucket + T;
    return v;
}

using LsAct = nnue_ls_params;

// floor(x * scale + eps) / scale when fake quantization is on (straight-through in the backward)
__device__ __forceinline__ float ls_fq(float x, const LsAct& a) {
    if (a.act_scale <= 0.f) return x;
    return __fdiv_rn(floorf(__fadd_rn(__fmul_rn(x, a.act_scale), a.act_eps)), a.act_scale);
}

}  // namespace nnue
