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

// ---- forward: tile = 64 positions x 32 outputs, K = L1 in chunks of 32 -----
// 128 threads, each a 4 x 4 register tile (positions ty + 16 i, outputs tx + 8 j):
// 8 shared float4 loads feed 64 FMA.
__global__ void __launch_bounds__(128)
    k_ls_l1_fwd(const float* __restrict__ x, const float* __restrict__ W1, const float* __restrict__ b1,
                LsPlanView plan, float* __restrict__ o1, int L1) {
    __shared__ __align__(16) float As[kTP][kPadK];
    __shared__ __align__(16) float Ws[kLsOut][kPadK];
    const int t = blockIdx.x;
    if (t >= *plan.n_tiles) return;
    const int cnt = plan.tile_count[t], bk = plan.tile_bucket[t];
    const int32_t* perm = plan.perm + plan.tile_start[t];
    const int tid = threadIdx.x;
    const int lr = tid >> 3, lc = tid & 7;  // loader: rows lr + 16 i of A, rows lr + 16 i of W; float4 column lc
    const float4 z = f4_zero();
    const float4* xa[4];
    bool live[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        live[i] = lr + 16 * i < cnt;
        xa[i] = reinterpret_cast<const float4*>(x + (int64_t)(live[i] ? perm[lr + 16 * i] : 0) * L1) + lc;
    }
    const float4* wr0 = reinterpret_cast<const float4*>(W1 + ((int64_t)bk * kLsOut + lr) * L1) + lc;
    const float4* wr1 = reinterpret_cast<const float4*>(W1 + ((int64_t)bk * kLsOut + lr + 16) * L1) + lc;
    const int ty = tid >> 3, tx = tid & 7;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    float4 ra[4], rw0 = __ldg(wr0), rw1 = __ldg(wr1);
#pragma unroll
    for (int i = 0; i < 4; ++i) ra[i] = live[i] ? __ldg(xa[i]) : z;
    const int nk = L1 / kKC;
    for (int kc = 0; kc < nk; ++kc) {
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(&As[lr + 16 * i][4 * lc]) = ra[i];
        *reinterpret_cast<float4*>(&Ws[lr][4 * lc]) = rw0;
        *reinterpret_cast<float4*>(&Ws[lr + 16][4 * lc]) = rw1;
        __syncthreads();
        if (kc + 1 < nk) {  // next chunk travels while this one is multiplied
            const int o = (kc + 1) * (kKC / 4);
#pragma unroll
            for (int i = 0; i < 4; ++i) ra[i] = live[i] ? __ldg(xa[i] + o) : z;
            rw0 = __ldg(wr0 + o);
            rw1 = __ldg(wr1 + o);
        }
#pragma unroll
        for (int k4 = 0; k4 < kKC / 4; ++k4) {
            float4 a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(&As[ty + 16 * i][4 * k4]);
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = *reinterpret_cast<const float4*>(&Ws[tx + 8 * j][4 * k4]);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = dot4(acc[i][j], a[i], w[j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int pos = ty + 16 * i;
        if (pos < cnt) {
            float* dst = o1 + (int64_t)perm[pos] * kLsOut;
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[tx + 8 * j] = __fadd_rn(acc[i][j], __ldg(b1 + bk * kLsOut + tx + 8 * j));
        }
    }
}

// ---- input gradient: dx[p, c] = sum_o d_o1[p, o] * W1[bucket, o, c] --------
// Tile of 64 positions; columns in chunks of 128.  Lane = 4 columns, warp = 8
// positions: per output unit two broadcast float4 of d_o1 (stored transposed)
// and one float4 of W feed 32 FMA.
constexpr int kDxCols = 128;
constexpr int kPadP = kTP + 4;
__global__ void __launch_bounds__(256)
    k_ls_l1_dx(const float* __restrict__ d_o1, const float* __restrict__ W1, LsPlanView plan,
               float* __restrict__ dx, int L1) {
    __shared__ __align__(16) float Dt[kLsOut][kPadP];  // [unit][position]
    __shared__ __align__(16) float Ws[kLsOut][kDxCols];
    const int t = blockIdx.x;
    if (t >= *plan.n_tiles) return;
    const int cnt = plan.tile_count[t], bk = plan.tile_bucket[t];
    const int32_t* perm = plan.perm + plan.tile_start[t];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < kTP * kLsOut; i += 256) {
        const int r = i >> 5, o = i & 31;  // coalesced read of a position's 32 units
        Dt[o][r] = r < cnt ? __ldg(d_o1 + (int64_t)perm[r] * kLsOut + o) : 0.f;
    }
    int64_t prow[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) prow[i] = 8 * warp + i < cnt ? (int64_t)perm[8 * warp + i] * L1 : -1;
    const float* wbase = W1 + (int64_t)bk * kLsOut * L1;
    for (int c0 = 0; c0 < L1; c0 += kDxCols) {
        __syncthreads();  // Dt ready (first pass) / previous Ws consumed
        for (int i = tid; i < kLsOut * (kDxCols / 4); i += 256) {
            const int o = i / (kDxCols / 4), c4 = i % (kDxCols / 4);
            float4 v = f4_zero();
            if (c0 + 4 * c4 < L1) v = __ldg(reinterpret_cast<const float4*>(wbase + (int64_t)o * L1 + c0) + c4);
            *reinterpret_cast<float4*>(&Ws[o][4 * c4]) = v;
        }
        __syncthreads();
        float4 acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = f4_zero();
#pragma unroll 8
        for (int o = 0; o < kLsOut; ++o) {
            const float4 w = *reinterpret_cast<const float4*>(&Ws[o][4 * lane]);
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
// CTA = (bucket, 64 columns), 128 threads, each a 4 x 4 register tile (units
// 4 ty .. 4 ty + 3, columns 4 tx .. 4 tx + 3); walks the bucket's positions 32
// at a time with the next 32 prefetched into registers.
constexpr int kDwCols = 64;
constexpr int kPadC = kDwCols + 4;
__global__ void __launch_bounds__(128)
    k_ls_l1_dw(const float* __restrict__ x, const float* __restrict__ d_o1, LsPlanView plan,
               float* __restrict__ dW1, float* __restrict__ db1, int L1, int n_col_chunks) {
    __shared__ __align__(16) float Xs[32][kPadC];
    __shared__ __align__(16) float Ds[32][kPadK];
    const int bk = blockIdx.x / n_col_chunks, cc = blockIdx.x % n_col_chunks;
    const int t0 = plan.bucket_tile[bk], t1 = plan.bucket_tile[bk + 1];
    const int beg = t0 < t1 ? plan.tile_start[t0] : 0;
    const int end = t0 < t1 ? plan.tile_start[t1 - 1] + plan.tile_count[t1 - 1] : 0;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;  // ty 0..7
    const int c0 = cc * kDwCols;
    float4 acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = f4_zero();
    float bsum = 0.f;
    // loader roles: X rows xr + 8 i (i < 4), float4 column tx; D rows dr + 16 i (i < 2), float4 column dc
    const int xr = tid >> 4, dr = tid >> 3, dc = tid & 7;
    const bool col_ok = c0 + 4 * tx < L1;
    float4 rx[4], rd[2];
    auto fetch = [&](int s) {
        const int m = min(32, end - s);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = xr + 8 * i;
            rx[i] = (r < m && col_ok)
                        ? __ldg(reinterpret_cast<const float4*>(x + (int64_t)plan.perm[s + r] * L1 + c0) + tx)
                        : f4_zero();
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = dr + 16 * i;
            rd[i] = r < m ? __ldg(reinterpret_cast<const float4*>(d_o1 + (int64_t)plan.perm[s + r] * kLsOut) + dc)
                          : f4_zero();
        }
    };
    if (beg < end) fetch(beg);
    for (int s = beg; s < end; s += 32) {
        const int m = min(32, end - s);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(&Xs[xr + 8 * i][4 * tx]) = rx[i];
#pragma unroll
        for (int i = 0; i < 2; ++i) *reinterpret_cast<float4*>(&Ds[dr + 16 * i][4 * dc]) = rd[i];
        __syncthreads();
        if (s + 32 < end) fetch(s + 32);
#pragma unroll 8
        for (int pp = 0; pp < 32; ++pp) {
            const float4 xv = *reinterpret_cast<const float4*>(&Xs[pp][4 * tx]);
            const float4 dv = *reinterpret_cast<const float4*>(&Ds[pp][4 * ty]);
            const float d[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[j].x = __fmaf_rn(d[j], xv.x, acc[j].x);
                acc[j].y = __fmaf_rn(d[j], xv.y, acc[j].y);
                acc[j].z = __fmaf_rn(d[j], xv.z, acc[j].z);
                acc[j].w = __fmaf_rn(d[j], xv.w, acc[j].w);
            }
        }
        if (cc == 0 && tid < kLsOut) {
            for (int pp = 0; pp < m; ++pp) bsum = __fadd_rn(bsum, Ds[pp][tid]);
        }
    }
    if (col_ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            *reinterpret_cast<float4*>(dW1 + ((int64_t)bk * kLsOut + 4 * ty + j) * L1 + c0 + 4 * tx) = acc[j];
    }
    if (cc == 0 && tid < kLsOut) db1[bk * kLsOut + tid] = bsum;
}

}  // namespace nnue

using namespace nnue;

static int ls_check(const char* who, int64_t B, int32_t L1, int32_t C, const void* plan) {
    NNUE_REQUIRE(B >= 0 && L1 > 0 && L1 % 32 == 0 && C > 0 && C <= 16, NNUE_ERR_UNSUPPORTED,
                 "%s: needs L1 %% 32 == 0 and 1..16 buckets (B=%lld L1=%d C=%d)", who, (long long)B, L1, C);
    NNUE_REQUIRE(plan != nullptr && aligned16(plan), NNUE_ERR_ARG, "%s: null or unaligned plan", who);
    return NNUE_OK;
}

extern "C" int nnue_ls_l1_fwd(const float* x, const float* W1, const float* b1, const void* plan, float* o1,
                              int64_t B, int32_t L1, int32_t C, void* stream) {
    int rc = ls_check("nnue_ls_l1_fwd", B, L1, C, plan);
    if (rc != NNUE_OK) return rc;
    if (B == 0) return NNUE_OK;
    NNUE_REQUIRE(x && W1 && b1 && o1 && aligned16(x) && aligned16(W1) && aligned16(o1), NNUE_ERR_ARG,
                 "nnue_ls_l1_fwd: null or unaligned tensor");
    k_ls_l1_fwd<<<(unsigned)ls_max_tiles(B, C), 128, 0, static_cast<cudaStream_t>(stream)>>>(
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
    k_ls_l1_dw<<<(unsigned)(C * chunks), 128, 0, s>>>(x, d_o1, v, dW1, db1, L1, chunks);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
