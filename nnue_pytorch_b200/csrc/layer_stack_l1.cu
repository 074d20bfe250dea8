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
__global__ void __launch_bounds__(256)
    k_ls_l1_fwd(const float* __restrict__ x, const float* __restrict__ W1, const float* __restrict__ b1,
                LsPlanView plan, float* __restrict__ o1, int L1) {
    __shared__ __align__(16) float As[kTP][kPadK];
    __shared__ __align__(16) float Ws[kLsOut][kPadK];
    const int t = blockIdx.x;
    if (t >= *plan.n_tiles) return;
    const int cnt = plan.tile_count[t], bk = plan.tile_bucket[t];
    const int32_t* perm = plan.perm + plan.tile_start[t];
    const int tid = threadIdx.x;
    // loader roles: two A float4 and one W float4 per thread per chunk
    const int lr = tid >> 3, lc = tid & 7;  // row 0..31 (+32), float4 column 0..7
    const int64_t pa0 = lr < cnt ? perm[lr] : -1, pa1 = lr + 32 < cnt ? perm[lr + 32] : -1;
    const float4* xa0 = reinterpret_cast<const float4*>(x + (pa0 < 0 ? 0 : pa0) * (int64_t)L1) + lc;
    const float4* xa1 = reinterpret_cast<const float4*>(x + (pa1 < 0 ? 0 : pa1) * (int64_t)L1) + lc;
    const float4* wr = reinterpret_cast<const float4*>(W1 + ((int64_t)bk * kLsOut + lr) * L1) + lc;
    // compute roles: positions ty, ty + 32; outputs tx + 8 j
    const int ty = tid >> 3, tx = tid & 7;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const float4 z = f4_zero();
    float4 ra0 = pa0 < 0 ? z : __ldg(xa0), ra1 = pa1 < 0 ? z : __ldg(xa1), rw = __ldg(wr);
    const int nk = L1 / kKC;
    for (int kc = 0; kc < nk; ++kc) {
        *reinterpret_cast<float4*>(&As[lr][4 * lc]) = ra0;
        *reinterpret_cast<float4*>(&As[lr + 32][4 * lc]) = ra1;
        *reinterpret_cast<float4*>(&Ws[lr][4 * lc]) = rw;
        __syncthreads();
        if (kc + 1 < nk) {  // next chunk travels while this one is multiplied
            const int o = (kc + 1) * (kKC / 4);
            ra0 = pa0 < 0 ? z : __ldg(xa0 + o);
            ra1 = pa1 < 0 ? z : __ldg(xa1 + o);
            rw = __ldg(wr + o);
        }
#pragma unroll
        for (int k4 = 0; k4 < kKC / 4; ++k4) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[ty][4 * k4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[ty + 32][4 * k4]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 w = *reinterpret_cast<const float4*>(&Ws[tx + 8 * j][4 * k4]);
                acc[0][j] = dot4(acc[0][j], a0, w);
                acc[1][j] = dot4(acc[1][j], a1, w);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int pos = ty + 32 * h;
        if (pos < cnt) {
            float* dst = o1 + (int64_t)perm[pos] * kLsOut;
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[tx + 8 * j] = __fadd_rn(acc[h][j], __ldg(b1 + bk * kLsOut + tx + 8 * j));
        }
    }
}

// ---- input gradient: dx[p, c] = sum_o d_o1[p, o] * W1[bucket, o, c] --------
constexpr int kDxCols = 128;
__global__ void __launch_bounds__(256)
    k_ls_l1_dx(const float* __restrict__ d_o1, const float* __restrict__ W1, LsPlanView plan,
               float* __restrict__ dx, int L1) {
    __shared__ __align__(16) float Ds[kTP][kPadK];
    __shared__ __align__(16) float Ws[kLsOut][kDxCols];
    const int t = blockIdx.x;
    if (t >= *plan.n_tiles) return;
    const int cnt = plan.tile_count[t], bk = plan.tile_bucket[t];
    const int32_t* perm = plan.perm + plan.tile_start[t];
    const int tid = threadIdx.x;
    for (int i = tid; i < kTP * (kLsOut / 4); i += 256) {
        const int r = i >> 3, c = i & 7;
        float4 v = f4_zero();
        if (r < cnt) v = __ldg(reinterpret_cast<const float4*>(d_o1 + (int64_t)perm[r] * kLsOut) + c);
        *reinterpret_cast<float4*>(&Ds[r][4 * c]) = v;
    }
    const int col = tid & (kDxCols - 1), half = tid >> 7;  // positions half*32 .. +31
    const float* wbase = W1 + (int64_t)bk * kLsOut * L1;
    for (int c0 = 0; c0 < L1; c0 += kDxCols) {
        __syncthreads();  // Ds ready (first pass) / previous Ws consumed
        for (int i = tid; i < kLsOut * (kDxCols / 4); i += 256) {
            const int o = i / (kDxCols / 4), c4 = i % (kDxCols / 4);
            float4 v = f4_zero();
            if (c0 + 4 * c4 < L1) v = __ldg(reinterpret_cast<const float4*>(wbase + (int64_t)o * L1 + c0) + c4);
            *reinterpret_cast<float4*>(&Ws[o][4 * c4]) = v;
        }
        __syncthreads();
        float acc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.f;
#pragma unroll
        for (int o4 = 0; o4 < kLsOut / 4; ++o4) {
            const float4 w = make_float4(Ws[4 * o4][col], Ws[4 * o4 + 1][col], Ws[4 * o4 + 2][col], Ws[4 * o4 + 3][col]);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float4 d = *reinterpret_cast<const float4*>(&Ds[half * 32 + i][4 * o4]);
                acc[i] = dot4(acc[i], d, w);
            }
        }
        if (c0 + col < L1) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int pos = half * 32 + i;
                if (pos < cnt) dx[(int64_t)perm[pos] * L1 + c0 + col] = acc[i];
            }
        }
    }
}

// ---- weight gradient: dW1[bucket, o, c] = sum_p d_o1[p, o] * x[p, c] -------
// CTA = (bucket, 64 columns); walks the bucket's positions 32 at a time.
constexpr int kDwCols = 64;
constexpr int kPadC = kDwCols + 4;
__global__ void __launch_bounds__(256)
    k_ls_l1_dw(const float* __restrict__ x, const float* __restrict__ d_o1, LsPlanView plan,
               float* __restrict__ dW1, float* __restrict__ db1, int L1, int n_col_chunks) {
    __shared__ __align__(16) float Xs[32][kPadC];
    __shared__ __align__(16) float Ds[32][kPadK];
    const int bk = blockIdx.x / n_col_chunks, cc = blockIdx.x % n_col_chunks;
    const int t0 = plan.bucket_tile[bk], t1 = plan.bucket_tile[bk + 1];
    const int beg = t0 < t1 ? plan.tile_start[t0] : 0;
    const int end = t0 < t1 ? plan.tile_start[t1 - 1] + plan.tile_count[t1 - 1] : 0;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;  // columns 4 tx .. 4 tx + 3, outputs ty and ty + 16
    float4 acc0 = f4_zero(), acc1 = f4_zero();
    float bsum = 0.f;
    const int c0 = cc * kDwCols;
    for (int s = beg; s < end; s += 32) {
        const int m = min(32, end - s);
        __syncthreads();
        for (int i = tid; i < 32 * (kDwCols / 4); i += 256) {
            const int r = i >> 4, c4 = i & 15;
            float4 v = f4_zero();
            if (r < m && c0 + 4 * c4 < L1)
                v = __ldg(reinterpret_cast<const float4*>(x + (int64_t)plan.perm[s + r] * L1 + c0) + c4);
            *reinterpret_cast<float4*>(&Xs[r][4 * c4]) = v;
        }
        {
            const int r = tid >> 3, c4 = tid & 7;
            float4 v = f4_zero();
            if (r < m) v = __ldg(reinterpret_cast<const float4*>(d_o1 + (int64_t)plan.perm[s + r] * kLsOut) + c4);
            *reinterpret_cast<float4*>(&Ds[r][4 * c4]) = v;
        }
        __syncthreads();
#pragma unroll 8
        for (int pp = 0; pp < 32; ++pp) {
            const float4 xv = *reinterpret_cast<const float4*>(&Xs[pp][4 * tx]);
            const float d0 = Ds[pp][ty], d1 = Ds[pp][ty + 16];
            acc0.x = __fmaf_rn(d0, xv.x, acc0.x); acc0.y = __fmaf_rn(d0, xv.y, acc0.y);
            acc0.z = __fmaf_rn(d0, xv.z, acc0.z); acc0.w = __fmaf_rn(d0, xv.w, acc0.w);
            acc1.x = __fmaf_rn(d1, xv.x, acc1.x); acc1.y = __fmaf_rn(d1, xv.y, acc1.y);
            acc1.z = __fmaf_rn(d1, xv.z, acc1.z); acc1.w = __fmaf_rn(d1, xv.w, acc1.w);
        }
        if (cc == 0 && tid < kLsOut) {
            for (int pp = 0; pp < m; ++pp) bsum = __fadd_rn(bsum, Ds[pp][tid]);
        }
    }
    if (c0 + 4 * tx < L1) {
        *reinterpret_cast<float4*>(dW1 + ((int64_t)bk * kLsOut + ty) * L1 + c0 + 4 * tx) = acc0;
        *reinterpret_cast<float4*>(dW1 + ((int64_t)bk * kLsOut + ty + 16) * L1 + c0 + 4 * tx) = acc1;
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
    k_ls_l1_fwd<<<(unsigned)ls_max_tiles(B, C), 256, 0, static_cast<cudaStream_t>(stream)>>>(
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
    k_ls_l1_dw<<<(unsigned)(C * chunks), 256, 0, s>>>(x, d_o1, v, dW1, db1, L1, chunks);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
