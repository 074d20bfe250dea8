// First layer of the bucketed layer stack: o1[p] = W1[bucket(p)] . x[p] + b1,
// its input gradient and its weight gradient, tile by tile over positions of
// one bucket (see layer_stack.cu).  fp32 FMA, shared-memory tiles, float4
// shared loads; every reduction runs in a fixed order.
#include <algorithm>

#include "layer_stack.cuh"

namespace nnue {

constexpr int kKC = 32;       // K chunk of the forward tile product
constexpr int kPadK = kKC + 4;  // row stride in floats: 144 B keeps float4 alignment and spreads banks

__device__ __forceinline__ float dot4(float acc, float4 a, float4 b) {
    acc = __fmaf_rn(a.x, b.x, acc);
    acc = __fmaf_rn(a.y, b.y, acc);
    acc = __fmaf_rn(a.z, b.z, acc);
    return __fmaf_rn(a.w, b.w, acc);
}

// ---- forward: tile = 64 positions x 32 outputs -----------------------------
// Shared-memory bandwidth is the limit of an fp32 FMA tile kernel here (one
// 16-byte shared load per lane costs 4 cycles of the SM's single shared-memory
// pipe, 4 FMA pipes retire 4 warp instructions per cycle), so every thread
// holds an 8 x 8 register tile: 16 shared float4 loads feed 256 FMA.
// A 64 x 32 tile is then ONE warp; the kWarpsL1 warps of a CTA split K between
// them (contiguous ranges, walked in chunks of 16 through a kFwdStages-deep
// cp.async pipeline in buffers private to the warp: warp-level barriers only)
// and their tiles are added in warp order at the end.
constexpr int kWarpsL1 = 4;
constexpr int kStagesL1 = 4;       // pipeline depth of the weight-gradient kernel
constexpr int kFwdStages = 3;      // ... and of the forward
constexpr int kKC8 = 16;           // K chunk of a warp (64 B of every row per stage)
constexpr int kPad8 = kKC8 + 4;    // row stride 80 B: float4 aligned, conflict-free for the access patterns below
constexpr int kFwdStage = (kTP + kLsOut) * kPad8;  // floats per stage: A [64][20] + W [32][20]
constexpr int kFwdSmemFloats = kWarpsL1 * kFwdStages * kFwdStage;  // >= the (kWarpsL1 - 1) partial tiles [64][33]
static_assert(kFwdSmemFloats >= (kWarpsL1 - 1) * kTP * (kLsOut + 1), "partial tiles alias the staging buffers");
__global__ void __launch_bounds__(32 * kWarpsL1, 2)
    k_ls_l1_fwd(const float* __restrict__ x, const float* __restrict__ W1, const float* __restrict__ b1,
                LsPlanView plan, float* __restrict__ o1, int L1) {
    extern __shared__ __align__(16) float smem[];
    const int t = blockIdx.x;
    if (t >= *plan.n_tiles) return;
    const int cnt = plan.tile_count[t], bk = plan.tile_bucket[t];
    const int32_t* perm = plan.perm + plan.tile_start[t];
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    float* stage0 = smem + g * kFwdStages * kFwdStage;
    // this warp's K range, in chunks of 8
    const int nc = L1 / kKC8;
    const int c_beg = (int)((int64_t)nc * g / kWarpsL1), c_end = (int)((int64_t)nc * (g + 1) / kWarpsL1);
    // loader: kF4 lanes per row (one float4 each), kRowsPass rows per pass: A in kTP / kRowsPass passes, W in
    // kLsOut / kRowsPass
    constexpr int kF4 = kKC8 / 4, kRowsPass = 32 / kF4, kPassA = kTP / kRowsPass, kPassW = kLsOut / kRowsPass;
    const int lr = lane / kF4, lc = lane % kF4;
    const float4* xa[kPassA];
    bool live[kPassA];
#pragma unroll
    for (int i = 0; i < kPassA; ++i) {
        live[i] = lr + kRowsPass * i < cnt;
        xa[i] = reinterpret_cast<const float4*>(x + (int64_t)(live[i] ? perm[lr + kRowsPass * i] : 0) * L1) + lc;
    }
    const float4* wr = reinterpret_cast<const float4*>(W1 + ((int64_t)bk * kLsOut + lr) * L1) + lc;
    const int64_t w_pass = (int64_t)kRowsPass * (L1 / 4);  // float4 between the W rows of two passes
    auto issue = [&](int c, int st) {  // chunk c into stage st; chunks past the range copy nothing
        if (c < c_end) {
            float (*As)[kPad8] = reinterpret_cast<float (*)[kPad8]>(stage0 + st * kFwdStage);
            float (*Ws)[kPad8] = As + kTP;
            const int o = c * kF4;
#pragma unroll
            for (int i = 0; i < kPassA; ++i) cp_async16(&As[lr + kRowsPass * i][4 * lc], xa[i] + o, live[i]);
#pragma unroll
            for (int i = 0; i < kPassW; ++i) cp_async16(&Ws[lr + kRowsPass * i][4 * lc], wr + i * w_pass + o, true);
        }
        cp_async_commit();  // one group per call, empty or not: the wait below counts groups
    };
    const int pg = lane >> 2, og = lane & 3;  // positions pg + 8 i, outputs og + 4 j
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
#pragma unroll
    for (int st = 0; st < kFwdStages - 1; ++st) issue(c_beg + st, st);
    int st = 0;
    for (int c = c_beg; c < c_end; ++c) {
        cp_async_wait<kFwdStages - 2>();  // this lane's part of chunk c has landed
        __syncwarp();                    // ... and every other lane's; the stage refilled next was read last iteration
        issue(c + kFwdStages - 1, (st + kFwdStages - 1) % kFwdStages);
        float (*As)[kPad8] = reinterpret_cast<float (*)[kPad8]>(stage0 + st * kFwdStage);
        float (*Ws)[kPad8] = As + kTP;
#pragma unroll
        for (int k4 = 0; k4 < kKC8 / 4; ++k4) {
            float4 a[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = *reinterpret_cast<const float4*>(&As[pg + 8 * i][4 * k4]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 w = *reinterpret_cast<const float4*>(&Ws[og + 4 * j][4 * k4]);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i][j] = dot4(acc[i][j], a[i], w);
            }
        }
        st = (st + 1) % kFwdStages;
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its staging buffers
    float (*red)[kTP][kLsOut + 1] = reinterpret_cast<float (*)[kTP][kLsOut + 1]>(smem);
    if (g > 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) red[g - 1][pg + 8 * i][og + 4 * j] = acc[i][j];
    }
    __syncthreads();
    if (g == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int pos = pg + 8 * i;
            if (pos < cnt) {
                float* dst = o1 + (int64_t)perm[pos] * kLsOut;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float v = acc[i][j];
#pragma unroll
                    for (int q = 0; q < kWarpsL1 - 1; ++q) v = __fadd_rn(v, red[q][pos][og + 4 * j]);
                    dst[og + 4 * j] = __fadd_rn(v, __ldg(b1 + bk * kLsOut + og + 4 * j));
                }
            }
        }
    }
}

// ---- input gradient: dx[p, c] = sum_o d_o1[p, o] * W1[bucket, o, c] --------
// Tile of 64 positions; columns in chunks of 128 (the bucket's weight chunk double
// buffered through cp.async).  Lane = 4 columns, warp = 8 positions: per output
// unit two broadcast float4 of d_o1 (stored transposed) and one float4 of W
// feed 32 FMA.
constexpr int kDxCols = 128;
constexpr int kPadP = kTP + 4;
__global__ void __launch_bounds__(256)
    k_ls_l1_dx(const float* __restrict__ d_o1, const float* __restrict__ W1, LsPlanView plan,
               float* __restrict__ dx, int L1) {
    __shared__ __align__(16) float Dt[kLsOut][kPadP];  // [unit][position]
    __shared__ __align__(16) float Ws[2][kLsOut][kDxCols];  // double buffer: chunk c + 1 lands while c is used
    const int t = blockIdx.x;
    if (t >= *plan.n_tiles) return;
    const int cnt = plan.tile_count[t], bk = plan.tile_bucket[t];
    const int32_t* perm = plan.perm + plan.tile_start[t];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* wbase = W1 + (int64_t)bk * kLsOut * L1;
    auto issue = [&](int c0, int buf) {  // columns [c0, c0 + 128) of the bucket's 32 rows; past L1: zeros
        for (int i = tid; i < kLsOut * (kDxCols / 4); i += 256) {
            const int o = i / (kDxCols / 4), c4 = i % (kDxCols / 4);
            const bool ok = c0 + 4 * c4 < L1;
            cp_async16(&Ws[buf][o][4 * c4], wbase + (int64_t)o * L1 + (ok ? c0 + 4 * c4 : 0), ok);
        }
        cp_async_commit();
    };
    issue(0, 0);
    for (int i = tid; i < kTP * kLsOut; i += 256) {
        const int r = i >> 5, o = i & 31;  // coalesced read of a position's 32 units
        Dt[o][r] = r < cnt ? __ldg(d_o1 + (int64_t)perm[r] * kLsOut + o) : 0.f;
    }
    int64_t prow[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) prow[i] = 8 * warp + i < cnt ? (int64_t)perm[8 * warp + i] * L1 : -1;
    int buf = 0;
    for (int c0 = 0; c0 < L1; c0 += kDxCols, buf ^= 1) {
        cp_async_wait<0>();
        __syncthreads();  // chunk c0 (and, first pass, Dt) visible to all; the other buffer is free again
        if (c0 + kDxCols < L1) issue(c0 + kDxCols, buf ^ 1);
        float4 acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = f4_zero();
#pragma unroll 8
        for (int o = 0; o < kLsOut; ++o) {
            const float4 w = *reinterpret_cast<const float4*>(&Ws[buf][o][4 * lane]);
            const float4 da = *reinterpret_cast<const float4*>(&Dt[o][8 * warp]);
            const float4 db = *reinterpret_cast<const float4*>(&Dt[o][8 * warp + 4]);
            const float d[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                acc[i].x = __fmaf_rn(d[i], w.x, acc[i].x);
                acc[i].y = __fmaf_rn(d[i], w.y, acc[i].y);
                acc[i].z = __fmaf_rn(d[i], w.z, acc[i].z);
                acc[i].w = __fmaf_rn(d[i], w.w, acc[i].w);
            }
        }
        if (c0 + 4 * lane < L1) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (prow[i] >= 0) __stcs(reinterpret_cast<float4*>(dx + prow[i] + c0) + lane, acc[i]);
        }
    }
}

// ---- weight gradient: dW1[bucket, o, c] = sum_p d_o1[p, o] * x[p, c] -------
// CTA = (bucket, 64 columns).  As in the forward, one warp holds the whole
// 32 x 64 output tile as 8 x 8 register tiles (units 4 og + {0..3} and
// 16 + 4 og + {0..3}, columns 4 cg + {0..3} and 32 + 4 cg + {0..3}); the
// kWarpsL1 warps take every kWarpsL1-th block of 8 positions of the bucket
// (kStagesL1-deep cp.async pipeline in buffers private to the warp, warp-level
// barriers only) and their tiles are added in warp order at the end.
constexpr int kDwCols = 64;
constexpr int kPadC = kDwCols + 4;
constexpr int kDwBlock = 8;  // positions per block
constexpr int kDwStage = kDwBlock * (kPadC + kPadK);  // floats per stage: X [8][68] + D [8][36]
constexpr int kDwSmemFloats = kWarpsL1 * kStagesL1 * kDwStage;
static_assert(kDwSmemFloats >= (kWarpsL1 - 1) * kLsOut * (kDwCols + 4), "partial tiles alias the staging buffers");
__global__ void __launch_bounds__(32 * kWarpsL1, 2)
    k_ls_l1_dw(const float* __restrict__ x, const float* __restrict__ d_o1, LsPlanView plan,
               float* __restrict__ dW1, float* __restrict__ db1, int L1, int n_col_chunks) {
    extern __shared__ __align__(16) float smem[];
    const int bk = blockIdx.x / n_col_chunks, cc = blockIdx.x % n_col_chunks;
    const int t0 = plan.bucket_tile[bk], t1 = plan.bucket_tile[bk + 1];
    const int beg = t0 < t1 ? plan.tile_start[t0] : 0;
    const int end = t0 < t1 ? plan.tile_start[t1 - 1] + plan.tile_count[t1 - 1] : 0;
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    float* stage0 = smem + g * kStagesL1 * kDwStage;
    const int c0 = cc * kDwCols;
    const int cg = lane & 7, og = lane >> 3;
    float acc[8][8];  // [unit][column]
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    float bsum = 0.f;
    // loader: X rows (lane >> 4) + 2 i (i < 4), float4 column lane & 15; D rows (lane >> 3) + 4 i (i < 2), float4 lane & 7
    const int xr = lane >> 4, xc = lane & 15, dr = lane >> 3, dc = lane & 7;
    const bool col_ok = c0 + 4 * xc < L1;
    auto issue = [&](int s, int st) {  // the block of positions starting at s into stage st; past the end: nothing
        if (s < end) {
            float (*Xs)[kPadC] = reinterpret_cast<float (*)[kPadC]>(stage0 + st * kDwStage);
            float (*Ds)[kPadK] = reinterpret_cast<float (*)[kPadK]>(stage0 + st * kDwStage + kDwBlock * kPadC);
            const int m = min(kDwBlock, end - s);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = xr + 2 * i;
                const bool ok = r < m && col_ok;
                cp_async16(&Xs[r][4 * xc], x + (int64_t)(ok ? plan.perm[s + r] : 0) * L1 + c0 + (ok ? 4 * xc : 0), ok);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = dr + 4 * i;
                const bool ok = r < m;
                cp_async16(&Ds[r][4 * dc], d_o1 + (int64_t)(ok ? plan.perm[s + r] : 0) * kLsOut + 4 * dc, ok);
            }
        }
        cp_async_commit();  // one group per call, empty or not: the wait below counts groups
    };
    const int step = kDwBlock * kWarpsL1;
    const int s0 = beg + kDwBlock * g;
#pragma unroll
    for (int st = 0; st < kStagesL1 - 1; ++st) issue(s0 + st * step, st);
    int st = 0;
    for (int s = s0; s < end; s += step) {
        const int m = min(kDwBlock, end - s);
        cp_async_wait<kStagesL1 - 2>();  // this lane's part of the block has landed
        __syncwarp();                    // ... and every other lane's; the stage refilled next was read last iteration
        issue(s + (kStagesL1 - 1) * step, (st + kStagesL1 - 1) % kStagesL1);
        float (*Xs)[kPadC] = reinterpret_cast<float (*)[kPadC]>(stage0 + st * kDwStage);
        float (*Ds)[kPadK] = reinterpret_cast<float (*)[kPadK]>(stage0 + st * kDwStage + kDwBlock * kPadC);
#pragma unroll
        for (int pp = 0; pp < kDwBlock; ++pp) {
            const float4 x0 = *reinterpret_cast<const float4*>(&Xs[pp][4 * cg]);
            const float4 x1 = *reinterpret_cast<const float4*>(&Xs[pp][32 + 4 * cg]);
            const float4 d0 = *reinterpret_cast<const float4*>(&Ds[pp][4 * og]);
            const float4 d1 = *reinterpret_cast<const float4*>(&Ds[pp][16 + 4 * og]);
            const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            const float dv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = __fmaf_rn(dv[i], xv[j], acc[i][j]);
        }
        if (cc == 0) {
            for (int pp = 0; pp < m; ++pp) bsum = __fadd_rn(bsum, Ds[pp][lane]);
        }
        st = (st + 1) % kStagesL1;
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its staging buffers
    float (*red)[kLsOut][kDwCols + 4] = reinterpret_cast<float (*)[kLsOut][kDwCols + 4]>(smem);
    if (g > 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int o = (i < 4 ? 4 * og + i : 16 + 4 * og + (i - 4));
            *reinterpret_cast<float4*>(&red[g - 1][o][4 * cg]) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            *reinterpret_cast<float4*>(&red[g - 1][o][32 + 4 * cg]) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
        }
        red[g - 1][lane][kDwCols] = bsum;  // row `lane`, first padding column
    }
    __syncthreads();
    if (g == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int o = (i < 4 ? 4 * og + i : 16 + 4 * og + (i - 4));
            float4 lo = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            float4 hi = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
#pragma unroll
            for (int q = 0; q < kWarpsL1 - 1; ++q) {
                lo = f4_add(lo, *reinterpret_cast<const float4*>(&red[q][o][4 * cg]));
                hi = f4_add(hi, *reinterpret_cast<const float4*>(&red[q][o][32 + 4 * cg]));
            }
            float* row = dW1 + ((int64_t)bk * kLsOut + o) * L1 + c0;
            if (c0 + 4 * cg < L1) *reinterpret_cast<float4*>(row + 4 * cg) = lo;
            if (c0 + 32 + 4 * cg < L1) *reinterpret_cast<float4*>(row + 32 + 4 * cg) = hi;
        }
        if (cc == 0) {
#pragma unroll
            for (int q = 0; q < kWarpsL1 - 1; ++q) bsum = __fadd_rn(bsum, red[q][lane][kDwCols]);
            db1[bk * kLsOut + lane] = bsum;
        }
    }
}

}  // namespace nnue

using namespace nnue;

// More than 48 KB of dynamic shared memory needs an opt-in per kernel and device.
static int ls_l1_opt_in() {
    static bool done[64] = {};
    int dev = 0;
    NNUE_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && done[dev]) return NNUE_OK;
    NNUE_CUDA_TRY(cudaFuncSetAttribute(k_ls_l1_fwd, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(kFwdSmemFloats * sizeof(float))));
    NNUE_CUDA_TRY(cudaFuncSetAttribute(k_ls_l1_dw, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(kDwSmemFloats * sizeof(float))));
    if (dev >= 0 && dev < 64) done[dev] = true;
    return NNUE_OK;
}

static int ls_check(const char* who, int64_t B, int32_t L1, int32_t C, const void* plan) {
    NNUE_REQUIRE(B >= 0 && L1 > 0 && L1 % 32 == 0 && C > 0 && C <= 16, NNUE_ERR_UNSUPPORTED,
                 "%s: needs L1 %% 32 == 0 and 1..16 buckets (B=%lld L1=%d C=%d)", who, (long long)B, L1, C);
    NNUE_REQUIRE(plan != nullptr && aligned16(plan), NNUE_ERR_ARG, "%s: null or unaligned plan", who);
    return ls_l1_opt_in();
}

extern "C" int nnue_ls_l1_fwd(const float* x, const float* W1, const float* b1, const void* plan, float* o1,
                              int64_t B, int32_t L1, int32_t C, void* stream) {
    int rc = ls_check("nnue_ls_l1_fwd", B, L1, C, plan);
    if (rc != NNUE_OK) return rc;
    if (B == 0) return NNUE_OK;
    NNUE_REQUIRE(x && W1 && b1 && o1 && aligned16(x) && aligned16(W1) && aligned16(o1), NNUE_ERR_ARG,
                 "nnue_ls_l1_fwd: null or unaligned tensor");
    k_ls_l1_fwd<<<(unsigned)ls_max_tiles(B, C), 32 * kWarpsL1, kFwdSmemFloats * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
        x, W1, b1, ls_view(plan, B, C), o1, L1);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

extern "C" int nnue_ls_l1_bwd(const float* x, const float* W1, const float* d_o1, const void* plan, float* dx,
                              float* dW1, float* db1, int64_t B, int32_t L1, int32_t C, void* stream) {
    int rc = ls_check("nnue_ls_l1_bwd", B, L1, C, plan);
    if (rc != NNUE_OK) return rc;
    NNUE_REQUIRE(dW1 && db1 && aligned16(dW1), NNUE_ERR_ARG, "nnue_ls_l1_bwd: null or unaligned output");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (B == 0) {
        NNUE_CUDA_TRY(cudaMemsetAsync(dW1, 0, (size_t)C * kLsOut * L1 * sizeof(float), s));
        NNUE_CUDA_TRY(cudaMemsetAsync(db1, 0, (size_t)C * kLsOut * sizeof(float), s));
        return NNUE_OK;
    }
    NNUE_REQUIRE(x && W1 && d_o1 && aligned16(x) && aligned16(W1) && aligned16(d_o1), NNUE_ERR_ARG,
                 "nnue_ls_l1_bwd: null or unaligned tensor");
    const LsPlanView v = ls_view(plan, B, C);
    if (dx) {
        NNUE_REQUIRE(aligned16(dx), NNUE_ERR_ALIGN, "nnue_ls_l1_bwd: dx not 16-byte aligned");
        k_ls_l1_dx<<<(unsigned)ls_max_tiles(B, C), 256, 0, s>>>(d_o1, W1, v, dx, L1);
        note_launches(1);
    }
    const int chunks = (L1 + kDwCols - 1) / kDwCols;
    k_ls_l1_dw<<<(unsigned)(C * chunks), 32 * kWarpsL1, kDwSmemFloats * sizeof(float), s>>>(x, d_o1, v, dW1, db1, L1, chunks);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
