// Fused double feature transformer: forward, backward prologue and the
// atomic-scatter backward.  Semantics follow the torch composition of
// model/modules/feature_transformer/double_ft_functions.py:62-80 (reference
// project paths); the kernels replace fused_ft_kernel.py:27-117 and :147-272.
//
// Work decomposition (forward and atomic backward): one warp per
// (position, column tile).  A tile is 32*U float4 of the first half of the
// L1 columns plus the same columns of the second half, because the pairwise
// product needs column i and column i + L1/2 of both perspectives.  Tiles are
// the SLOW grid dimension: all positions of tile 0 run before tile 1, so the
// slice of the weight table a tile touches (N * U KiB) stays resident in the
// 126 MB L2 while every position re-reads it.
#include <math.h>

#include "ft_fused.cuh"
#include "segment.cuh"

namespace nnue {

template <int U, int R, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
    k_fused_fwd(const float* __restrict__ us, const float* __restrict__ them,
                const int32_t* __restrict__ wi, const int32_t* __restrict__ bi,
                const int64_t* __restrict__ psqt_idx, const float* __restrict__ weight,
                const float* __restrict__ bias, FtAct act, float* __restrict__ l0,
                float* __restrict__ wpsqt, float* __restrict__ bpsqt, float* __restrict__ saved,
                int64_t B, int K, int64_t N, int L1, int P, int n_pos_groups, int want_stage,
                unsigned long long* status) {
    extern __shared__ __align__(16) int32_t s_idx[];
    __shared__ __align__(8) uint64_t bar;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / n_pos_groups;
    const int64_t p0 = (int64_t)(blockIdx.x % n_pos_groups) * kWarpsPerCta;
    const int64_t p = p0 + warp;

    const StagedLists lists = stage_lists(wi, bi, p0, B, K, want_stage != 0, s_idx, &bar, warp, status);
    if (p >= B) return;

    const int W = L1 + P;
    const int h4 = L1 >> 3;          // float4 per half
    const int64_t W4 = W >> 2;       // float4 per row
    const float4* table = reinterpret_cast<const float4*>(weight);
    const float4* bias4 = reinterpret_cast<const float4*>(bias);

    int col[2 * U];
    bool ok[2 * U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int c = tile * (32 * U) + u * 32 + lane;
        ok[u] = ok[U + u] = c < h4;
        col[u] = c;
        col[U + u] = h4 + c;
    }

    const int nw = count_active(lists.w, K, lane);
    const int nb = count_active(lists.b, K, lane);

    float4 accw[2 * U], accb[2 * U];
#pragma unroll
    for (int c = 0; c < 2 * U; ++c) accw[c] = ok[c] ? ldg4(bias4 + col[c]) : f4_zero();
    gather_sum<2 * U, R>(table, W4, N, lists.w, nw, col, ok, accw, lane, status);
#pragma unroll
    for (int c = 0; c < 2 * U; ++c) accb[c] = ok[c] ? ldg4(bias4 + col[c]) : f4_zero();
    gather_sum<2 * U, R>(table, W4, N, lists.b, nb, col, ok, accb, lane, status);

    const float u_ = __ldg(us + p), t_ = __ldg(them + p);
    const int h = L1 >> 1;
    float4* l0p = reinterpret_cast<float4*>(l0 + p * L1);
    float4* sv = reinterpret_cast<float4*>(saved + p * 2 * (int64_t)L1);
#pragma unroll
    for (int u = 0; u < U; ++u) {
        if (!ok[u]) continue;
        ft_store_columns(u_, t_, accw[u], accw[U + u], accb[u], accb[U + u], col[u], h4, sv, l0p, act);
    }
    (void)h;

    if (tile == 0) {
        const int64_t pi = __ldg(psqt_idx + p);
        if (pi >= 0 && pi < P) {
            const float b0 = __ldg(bias + L1 + pi);
            const float sw = psqt_sum(weight, W, N, lists.w, nw, L1 + (int)pi, b0, lane);
            const float sb = psqt_sum(weight, W, N, lists.b, nb, L1 + (int)pi, b0, lane);
            if (lane == 0) {
                wpsqt[p] = sw;
                bpsqt[p] = sb;
            }
        } else if (lane == 0) {
            note_bad_index(status);
            wpsqt[p] = 0.f;
            bpsqt[p] = 0.f;
        }
    }
}

// Scalar fallback for shapes the float4 kernels cannot take (W % 4 != 0,
// L1 % 8 != 0 or unaligned pointers): one CTA per position, one thread per
// column pair.  Same arithmetic order.
__global__ void k_fused_fwd_scalar(const float* __restrict__ us, const float* __restrict__ them,
                                   const int32_t* __restrict__ wi, const int32_t* __restrict__ bi,
                                   const int64_t* __restrict__ psqt_idx,
                                   const float* __restrict__ weight, const float* __restrict__ bias,
                                   FtAct act, float* __restrict__ l0, float* __restrict__ wpsqt,
                                   float* __restrict__ bpsqt, float* __restrict__ saved, int64_t B,
                                   int K, int64_t N, int L1, int P, unsigned long long* status) {
    const int64_t p = blockIdx.x;
    if (p >= B) return;
    const int h = L1 >> 1, W = L1 + P;
    const int32_t* lw = wi + p * K;
    const int32_t* lb = bi + p * K;
    const float u_ = us[p], t_ = them[p];
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        float w0 = bias[i], w1 = bias[i + h], b0 = w0, b1 = w1;
        for (int k = 0; k < K; ++k) {
            const int r = lw[k];
            if (r < 0) break;
            if (r >= N) { if (i == 0) note_bad_index(status); continue; }
            w0 = __fadd_rn(w0, weight[(int64_t)r * W + i]);
            w1 = __fadd_rn(w1, weight[(int64_t)r * W + i + h]);
        }
        for (int k = 0; k < K; ++k) {
            const int r = lb[k];
            if (r < 0) break;
            if (r >= N) { if (i == 0) note_bad_index(status); continue; }
            b0 = __fadd_rn(b0, weight[(int64_t)r * W + i]);
            b1 = __fadd_rn(b1, weight[(int64_t)r * W + i + h]);
        }
        const float x0 = mix(u_, w0, t_, b0), x1 = mix(u_, w1, t_, b1);
        const float x2 = mix(u_, b0, t_, w0), x3 = mix(u_, b1, t_, w1);
        float* sv = saved + p * 2 * (int64_t)L1;
        sv[i] = x0; sv[h + i] = x1; sv[2 * h + i] = x2; sv[3 * h + i] = x3;
        const float max_act = act.max_act;
        auto cl = [max_act](float x) { return fminf(fmaxf(x, 0.f), max_act); };
        l0[p * L1 + i] = finish_l0(__fmul_rn(cl(x0), cl(x1)), act);
        l0[p * L1 + h + i] = finish_l0(__fmul_rn(cl(x2), cl(x3)), act);
    }
    if (threadIdx.x == 0) {
        const int64_t pi = psqt_idx[p];
        float sw = 0.f, sb = 0.f;
        if (pi >= 0 && pi < P) {
            sw = sb = bias[L1 + pi];
            for (int k = 0; k < K; ++k) {
                const int r = lw[k];
                if (r < 0) break;
                if (r < N) sw = __fadd_rn(sw, weight[(int64_t)r * W + L1 + pi]);
            }
            for (int k = 0; k < K; ++k) {
                const int r = lb[k];
                if (r < 0) break;
                if (r < N) sb = __fadd_rn(sb, weight[(int64_t)r * W + L1 + pi]);
            }
        } else {
            note_bad_index(status);
        }
        wpsqt[p] = sw;
        bpsqt[p] = sb;
    }
}

// ---------------------------------------------------------------------------
// Backward prologue: per position build the two rows the table gradient is a
// scatter of,
//   G[2p]   = [ g_w (L1) | onehot(psqt_idx[p]) * grad_wpsqt[p] (P) ]
//   G[2p+1] = [ g_b (L1) | onehot(psqt_idx[p]) * grad_bpsqt[p] (P) ]
// so that grad_weight[r] = sum of G rows whose list names r, and
// grad_bias = column sum of G.  Also emits per-CTA column sums (bias partials)
// so G is not read a second time for the bias.
// Thread = one float4 column of the first half (+ its partner in the second
// half); a CTA walks `pb` consecutive positions.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float4 f4_mul(float4 a, float4 b) {
    return make_float4(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y), __fmul_rn(a.z, b.z),
                       __fmul_rn(a.w, b.w));
}
__device__ __forceinline__ float4 f4_clamp(float4 x, float m) {
    return make_float4(fminf(fmaxf(x.x, 0.f), m), fminf(fmaxf(x.y, 0.f), m),
                       fminf(fmaxf(x.z, 0.f), m), fminf(fmaxf(x.w, 0.f), m));
}
// gradient mask of torch.clamp: passes on the closed interval [0, m]
__device__ __forceinline__ float4 f4_mask(float4 g, float4 x, float m) {
    return make_float4((x.x >= 0.f && x.x <= m) ? g.x : 0.f, (x.y >= 0.f && x.y <= m) ? g.y : 0.f,
                       (x.z >= 0.f && x.z <= m) ? g.z : 0.f, (x.w >= 0.f && x.w <= m) ? g.w : 0.f);
}

__global__ void __launch_bounds__(kThreads)
    k_bwd_prologue(const float* __restrict__ us, const float* __restrict__ them,
                   const int64_t* __restrict__ psqt_idx, FtAct act,
                   const float* __restrict__ grad_l0, const float* __restrict__ grad_wpsqt,
                   const float* __restrict__ grad_bpsqt, const float* __restrict__ saved,
                   float* __restrict__ G, float* __restrict__ bias_part, int64_t B, int L1, int P,
                   int pb, int n_col_chunks) {
    const float max_act = act.max_act;
    const int chunk = blockIdx.x % n_col_chunks;
    const int64_t blk = blockIdx.x / n_col_chunks;
    const int64_t p_beg = blk * pb;
    const int64_t p_end = min(B, p_beg + (int64_t)pb);
    const int h4 = L1 >> 3;
    const int W = L1 + P;
    const int64_t W4 = W >> 2;
    const int P4 = P >> 2;
    const int c = chunk * kThreads + threadIdx.x;  // float4 column in [0, h4 + P4)

    float4 s0 = f4_zero(), s1 = f4_zero();
    if (c < h4) {
        for (int64_t p = p_beg; p < p_end; ++p) {
            const float u_ = __ldg(us + p), t_ = __ldg(them + p);
            const float4* sv = reinterpret_cast<const float4*>(saved + p * 2 * (int64_t)L1);
            const float4* gl = reinterpret_cast<const float4*>(grad_l0 + p * (int64_t)L1);
            const float4 x0 = __ldcs(sv + c), x1 = __ldcs(sv + h4 + c);
            const float4 x2 = __ldcs(sv + 2 * h4 + c), x3 = __ldcs(sv + 3 * h4 + c);
            float4 ga = __ldcs(gl + c), gb = __ldcs(gl + h4 + c);
            if (act.out_scale != 1.f) {  // gradient of `l0 * out_scale`; the fake quantization is straight-through
                const float4 k = make_float4(act.out_scale, act.out_scale, act.out_scale, act.out_scale);
                ga = f4_mul(ga, k);
                gb = f4_mul(gb, k);
            }
            const float4 d0 = f4_mask(f4_mul(ga, f4_clamp(x1, max_act)), x0, max_act);
            const float4 d1 = f4_mask(f4_mul(ga, f4_clamp(x0, max_act)), x1, max_act);
            const float4 d2 = f4_mask(f4_mul(gb, f4_clamp(x3, max_act)), x2, max_act);
            const float4 d3 = f4_mask(f4_mul(gb, f4_clamp(x2, max_act)), x3, max_act);
            const float4 gw0 = f4_mix(u_, d0, t_, d2), gw1 = f4_mix(u_, d1, t_, d3);
            const float4 gb0 = f4_mix(t_, d0, u_, d2), gb1 = f4_mix(t_, d1, u_, d3);
            float4* gwr = reinterpret_cast<float4*>(G) + (2 * p) * W4;
            float4* gbr = gwr + W4;
            gwr[c] = gw0;
            gwr[h4 + c] = gw1;
            gbr[c] = gb0;
            gbr[h4 + c] = gb1;
            s0 = f4_add(s0, f4_add(gw0, gb0));
            s1 = f4_add(s1, f4_add(gw1, gb1));
        }
        float4* part = reinterpret_cast<float4*>(bias_part) + blk * W4;
        part[c] = s0;
        part[h4 + c] = s1;
    } else if (c < h4 + P4) {
        const int q = c - h4;  // float4 slot inside the PSQT columns
        for (int64_t p = p_beg; p < p_end; ++p) {
            const int64_t pi = __ldg(psqt_idx + p);
            const float gw = __ldg(grad_wpsqt + p), gb = __ldg(grad_bpsqt + p);
            float w[4], b[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool hit = (pi == (int64_t)(q * 4 + j));
                w[j] = hit ? gw : 0.f;
                b[j] = hit ? gb : 0.f;
            }
            float4* gwr = reinterpret_cast<float4*>(G) + (2 * p) * W4;
            float4* gbr = gwr + W4;
            const float4 vw = make_float4(w[0], w[1], w[2], w[3]);
            const float4 vb = make_float4(b[0], b[1], b[2], b[3]);
            gwr[2 * h4 + q] = vw;
            gbr[2 * h4 + q] = vb;
            s0 = f4_add(s0, f4_add(vw, vb));
        }
        float4* part = reinterpret_cast<float4*>(bias_part) + blk * W4;
        part[2 * h4 + q] = s0;
    }
}

// Scalar prologue for unaligned shapes: same outputs, one thread per column.
__global__ void k_bwd_prologue_scalar(const float* __restrict__ us, const float* __restrict__ them,
                                      const int64_t* __restrict__ psqt_idx, FtAct act,
                                      const float* __restrict__ grad_l0,
                                      const float* __restrict__ grad_wpsqt,
                                      const float* __restrict__ grad_bpsqt,
                                      const float* __restrict__ saved, float* __restrict__ G,
                                      int64_t B, int L1, int P) {
    const float max_act = act.max_act;
    const int64_t p = blockIdx.x;
    if (p >= B) return;
    const int h = L1 >> 1, W = L1 + P;
    const float u_ = us[p], t_ = them[p];
    const float* sv = saved + p * 2 * (int64_t)L1;
    const float* gl = grad_l0 + p * (int64_t)L1;
    float* gwr = G + (2 * p) * (int64_t)W;
    float* gbr = gwr + W;
    auto cl = [max_act](float x) { return fminf(fmaxf(x, 0.f), max_act); };
    auto in = [max_act](float x) { return x >= 0.f && x <= max_act; };
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        const float x0 = sv[i], x1 = sv[h + i], x2 = sv[2 * h + i], x3 = sv[3 * h + i];
        float ga = gl[i], gb = gl[h + i];
        if (act.out_scale != 1.f) { ga = __fmul_rn(ga, act.out_scale); gb = __fmul_rn(gb, act.out_scale); }
        const float d0 = in(x0) ? __fmul_rn(ga, cl(x1)) : 0.f;
        const float d1 = in(x1) ? __fmul_rn(ga, cl(x0)) : 0.f;
        const float d2 = in(x2) ? __fmul_rn(gb, cl(x3)) : 0.f;
        const float d3 = in(x3) ? __fmul_rn(gb, cl(x2)) : 0.f;
        gwr[i] = mix(u_, d0, t_, d2);
        gwr[h + i] = mix(u_, d1, t_, d3);
        gbr[i] = mix(t_, d0, u_, d2);
        gbr[h + i] = mix(t_, d1, u_, d3);
    }
    const int64_t pi = psqt_idx[p];
    for (int j = threadIdx.x; j < P; j += blockDim.x) {
        gwr[L1 + j] = (pi == j) ? grad_wpsqt[p] : 0.f;
        gbr[L1 + j] = (pi == j) ? grad_bpsqt[p] : 0.f;
    }
}

// ---------------------------------------------------------------------------
// Atomic-scatter backward: same warp/tile decomposition as the forward, the
// per-position gradient stays in registers and goes out as 16-byte vector
// reductions (red.global.add.v4.f32) into a gradient the host zeroed first.
// All-zero float4 are skipped (clamped-out neurons make most of them zero).
// Bias: per-CTA shared-memory sums, then one vector reduction per column.
// ---------------------------------------------------------------------------
template <int U>
__global__ void __launch_bounds__(kThreads)
    k_fused_bwd_atomic(const float* __restrict__ us, const float* __restrict__ them,
                       const int32_t* __restrict__ wi, const int32_t* __restrict__ bi,
                       const int64_t* __restrict__ psqt_idx, FtAct act,
                       const float* __restrict__ grad_l0, const float* __restrict__ grad_wpsqt,
                       const float* __restrict__ grad_bpsqt, const float* __restrict__ saved,
                       float* __restrict__ grad_weight, float* __restrict__ grad_bias, int64_t B,
                       int K, int64_t N, int L1, int P, int n_pos_groups, int pos_per_cta,
                       unsigned long long* status) {
    const float max_act = act.max_act;
    __shared__ float4 s_bias[kWarpsPerCta][2 * U][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / n_pos_groups;
    const int64_t pbase = (int64_t)(blockIdx.x % n_pos_groups) * pos_per_cta;
    const int W = L1 + P;
    const int h4 = L1 >> 3;
    const int64_t W4 = W >> 2;

    int col[2 * U];
    bool ok[2 * U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int c = tile * (32 * U) + u * 32 + lane;
        ok[u] = ok[U + u] = c < h4;
        col[u] = c;
        col[U + u] = h4 + c;
    }
    float4 bsum[2 * U];
#pragma unroll
    for (int c = 0; c < 2 * U; ++c) bsum[c] = f4_zero();

    for (int64_t p = pbase + warp; p < min(B, pbase + (int64_t)pos_per_cta); p += kWarpsPerCta) {
        const float u_ = __ldg(us + p), t_ = __ldg(them + p);
        const float4* sv = reinterpret_cast<const float4*>(saved + p * 2 * (int64_t)L1);
        const float4* gl = reinterpret_cast<const float4*>(grad_l0 + p * (int64_t)L1);
        float4 gw[2 * U], gb[2 * U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (ok[u]) {
                const int c = col[u];
                const float4 x0 = __ldcs(sv + c), x1 = __ldcs(sv + h4 + c);
                const float4 x2 = __ldcs(sv + 2 * h4 + c), x3 = __ldcs(sv + 3 * h4 + c);
                float4 ga = __ldcs(gl + c), gbv = __ldcs(gl + h4 + c);
                if (act.out_scale != 1.f) {
                    const float4 k = make_float4(act.out_scale, act.out_scale, act.out_scale, act.out_scale);
                    ga = f4_mul(ga, k);
                    gbv = f4_mul(gbv, k);
                }
                const float4 d0 = f4_mask(f4_mul(ga, f4_clamp(x1, max_act)), x0, max_act);
                const float4 d1 = f4_mask(f4_mul(ga, f4_clamp(x0, max_act)), x1, max_act);
                const float4 d2 = f4_mask(f4_mul(gbv, f4_clamp(x3, max_act)), x2, max_act);
                const float4 d3 = f4_mask(f4_mul(gbv, f4_clamp(x2, max_act)), x3, max_act);
                gw[u] = f4_mix(u_, d0, t_, d2);
                gw[U + u] = f4_mix(u_, d1, t_, d3);
                gb[u] = f4_mix(t_, d0, u_, d2);
                gb[U + u] = f4_mix(t_, d1, u_, d3);
            } else {
                gw[u] = gw[U + u] = gb[u] = gb[U + u] = f4_zero();
            }
            bsum[u] = f4_add(bsum[u], f4_add(gw[u], gb[u]));
            bsum[U + u] = f4_add(bsum[U + u], f4_add(gw[U + u], gb[U + u]));
        }
        bool nzw[2 * U], nzb[2 * U];
#pragma unroll
        for (int c = 0; c < 2 * U; ++c) {
            nzw[c] = ok[c] && (gw[c].x != 0.f || gw[c].y != 0.f || gw[c].z != 0.f || gw[c].w != 0.f);
            nzb[c] = ok[c] && (gb[c].x != 0.f || gb[c].y != 0.f || gb[c].z != 0.f || gb[c].w != 0.f);
        }
        const int64_t pi = __ldg(psqt_idx + p);
        const bool psq = (tile == 0) && (pi >= 0 && pi < P);
        const float gwp = psq ? __ldg(grad_wpsqt + p) : 0.f;
        const float gbp = psq ? __ldg(grad_bpsqt + p) : 0.f;
        if (psq && lane == 0) atomicAdd(grad_bias + L1 + pi, __fadd_rn(gwp, gbp));

        for (int persp = 0; persp < 2; ++persp) {
            const int32_t* list = (persp ? bi : wi) + p * K;
            const float gp = persp ? gbp : gwp;
            for (int k0 = 0; k0 < K; k0 += 32) {
                const int k = k0 + lane;
                const int mine = (k < K) ? __ldg(list + k) : -1;
                const unsigned neg = __ballot_sync(kFullMask, mine < 0);
                const int m = neg ? (__ffs(neg) - 1) : 32;
                if (psq && lane < m && (int64_t)mine < N && gp != 0.f)
                    atomicAdd(grad_weight + (int64_t)mine * W + L1 + pi, gp);
                for (int j = 0; j < m; ++j) {
                    const int r = __shfl_sync(kFullMask, mine, j);
                    if ((int64_t)r >= N) {
                        if (lane == 0 && tile == 0) note_bad_index(status);
                        continue;
                    }
                    float* row = grad_weight + (int64_t)r * W;
#pragma unroll
                    for (int c = 0; c < 2 * U; ++c) {
                        if (persp ? nzb[c] : nzw[c]) red_add_v4(row + 4 * col[c], persp ? gb[c] : gw[c]);
                    }
                }
                if (neg) break;
            }
        }
    }
    // bias: fixed-order sum over the 8 warps, then one vector reduction per slot
#pragma unroll
    for (int c = 0; c < 2 * U; ++c) s_bias[warp][c][lane] = bsum[c];
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int c = 0; c < 2 * U; ++c) {
            float4 s = s_bias[0][c][lane];
            for (int w = 1; w < kWarpsPerCta; ++w) s = f4_add(s, s_bias[w][c][lane]);
            if (ok[c]) red_add_v4(grad_bias + 4 * col[c], s);
        }
    }
}

}  // namespace nnue

// ===========================================================================
// C ABI
// ===========================================================================
using namespace nnue;

static bool fused_vec_ok(int L1, int P, const void* a, const void* b, const void* c, const void* d,
                         const void* e) {
    return (L1 % 8 == 0) && (P % 4 == 0) && aligned16(a) && aligned16(b) && aligned16(c) &&
           aligned16(d) && aligned16(e);
}

extern "C" int nnue_ft_fused_fwd(const float* us, const float* them, const int32_t* white_idx,
                                 const int32_t* black_idx, const int64_t* psqt_idx,
                                 const float* weight, const float* bias, float max_act,
                                 float act_quant_scale, float act_quant_eps, float out_scale,
                                 float* l0, float* wpsqt, float* bpsqt, float* saved, int64_t B,
                                 int32_t K, int64_t N, int32_t L1, int32_t P, void* stream) {
    int sc_exp = 0;
    const bool pow2 = act_quant_scale > 0.f && frexpf(act_quant_scale, &sc_exp) == 0.5f;
    const FtAct act{max_act, act_quant_scale, act_quant_eps, out_scale, pow2 ? 1.0f / act_quant_scale : 0.f};
    NNUE_REQUIRE(B >= 0 && K >= 0 && N >= 0 && L1 > 0 && P >= 0, NNUE_ERR_ARG,
                 "nnue_ft_fused_fwd: negative size (B=%lld K=%d N=%lld L1=%d P=%d)", (long long)B, K,
                 (long long)N, L1, P);
    NNUE_REQUIRE(L1 % 2 == 0, NNUE_ERR_ARG, "nnue_ft_fused_fwd: l1_size must be even, got %d", L1);
    if (B == 0) return NNUE_OK;
    NNUE_REQUIRE(us && them && white_idx && black_idx && psqt_idx && weight && bias && l0 && wpsqt &&
                     bpsqt && saved,
                 NNUE_ERR_ARG, "nnue_ft_fused_fwd: null pointer");
    NNUE_REQUIRE(B * (int64_t)K < (1LL << 40), NNUE_ERR_UNSUPPORTED, "nnue_ft_fused_fwd: batch too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "nnue_ft_fused_fwd: no device status word");

    if (!fused_vec_ok(L1, P, weight, bias, l0, saved, weight)) {
        const int threads = 128;
        NNUE_REQUIRE(B <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "nnue_ft_fused_fwd: batch too large");
        k_fused_fwd_scalar<<<(unsigned)B, threads, 0, s>>>(us, them, white_idx, black_idx, psqt_idx,
                                                          weight, bias, act, l0, wpsqt, bpsqt,
                                                          saved, B, K, N, L1, P, status);
        NNUE_CUDA_TRY(cudaGetLastError());
        note_launches(1);
        return NNUE_OK;
    }

    const int h4 = L1 / 8;
    int U = tuning().fwd_u;
    if (U != 1 && U != 2 && U != 4) U = 2;
    while (U > 1 && h4 <= 32 * (U / 2)) U /= 2;  // narrow layers: no empty slots
    const int tiles = (h4 + 32 * U - 1) / (32 * U);
    const int64_t groups = (B + kWarpsPerCta - 1) / kWarpsPerCta;
    NNUE_REQUIRE(groups * tiles <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED,
                 "nnue_ft_fused_fwd: grid too large");
    const size_t smem = (size_t)2 * kWarpsPerCta * K * sizeof(int32_t);
    const int stage = tuning().stage_idx && K > 0 && smem <= 48 * 1024 && aligned16(white_idx) &&
                      aligned16(black_idx);
    const unsigned grid = (unsigned)(groups * tiles);
    ProfScope prof("k_fused_fwd", s);
#define LAUNCH_FWD(UU, RR, MB)                                                                  \
    k_fused_fwd<UU, RR, MB><<<grid, kThreads, stage ? smem : 0, s>>>(                           \
        us, them, white_idx, black_idx, psqt_idx, weight, bias, act, l0, wpsqt, bpsqt, saved, B, \
        K, N, L1, P, (int)groups, stage, status)
    // variant = rows in flight per warp (R) and CTAs per SM the register budget must allow
    const int v = tuning().fwd_variant;
    if (U == 1) {
        if (v == 1) LAUNCH_FWD(1, 2, 6); else if (v == 2) LAUNCH_FWD(1, 4, 3);
        else if (v == 3) LAUNCH_FWD(1, 2, 4); else if (v == 4) LAUNCH_FWD(1, 6, 3);
        else LAUNCH_FWD(1, 4, 4);
    } else if (U == 2) {
        if (v == 1) LAUNCH_FWD(2, 4, 2); else if (v == 2) LAUNCH_FWD(2, 1, 4);
        else LAUNCH_FWD(2, 2, 3);
    } else {
        LAUNCH_FWD(4, 2, 2);
    }
#undef LAUNCH_FWD
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

// Workspace layout of the fused backward (segment mode):
//   G [2B, W] f32 | bias partials [ceil(B/pb), W] f32 | CSR scratch
static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static int resolve_mode(int mode) {
    if (mode == NNUE_BWD_AUTO) return NNUE_BWD_SEGMENT;
    return mode;
}

extern "C" int32_t nnue_ft_fused_bwd_column_tile(int32_t L1, int32_t P) {
    if (L1 <= 0 || P < 0) return 0;
    return (L1 % 8 == 0 && P % 4 == 0) ? csr_column_tile(L1 + P) : 0;
}

extern "C" size_t nnue_ft_fused_bwd_workspace_bytes(int64_t B, int32_t K, int64_t N, int32_t L1,
                                                    int32_t P, int32_t mode) {
    if (B < 0 || K < 0 || N < 0 || L1 <= 0 || P < 0) return 0;
    if (resolve_mode(mode) == NNUE_BWD_ATOMIC && L1 % 8 == 0 && P % 4 == 0) return 256;
    const int64_t W = (int64_t)L1 + P;
    const int pb = tuning().prologue_pb;
    const int64_t nblk = (B + pb - 1) / pb;
    size_t bytes = 0;
    bytes += align_up((size_t)(2 * B) * W * sizeof(float), 256);
    bytes += align_up((size_t)nblk * W * sizeof(float), 256);
    bytes += csr_workspace_bytes(2 * B * (int64_t)K, N, (int)W);
    return bytes + 256;
}

static int fused_bwd_impl(const float* us, const float* them, const int32_t* white_idx,
                          const int32_t* black_idx, const int64_t* psqt_idx, float max_act,
                          float out_scale, const float* grad_l0, const float* grad_wpsqt,
                          const float* grad_bpsqt, const float* saved, float* grad_weight,
                          float* grad_bias, int64_t B, int32_t K, int64_t N, int32_t L1,
                          int32_t P, void* workspace, size_t workspace_bytes, int32_t mode,
                          const nnue_bwd_slices* slices, void* stream) {
    const FtAct act{max_act, 0.f, 0.f, out_scale, 0.f};
    const int n_slices = slices ? slices->n_slices : 0;
    // routes that finish the whole gradient at once still owe the consumer its events
    auto record_all = [&](cudaStream_t st) -> int {
        for (int i = 0; i < n_slices; ++i)
            if (slices->events[i]) NNUE_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(slices->events[i]), st));
        return NNUE_OK;
    };
    NNUE_REQUIRE(B >= 0 && K >= 0 && N >= 0 && L1 > 0 && P >= 0, NNUE_ERR_ARG,
                 "nnue_ft_fused_bwd: negative size");
    NNUE_REQUIRE(L1 % 2 == 0, NNUE_ERR_ARG, "nnue_ft_fused_bwd: l1_size must be even, got %d", L1);
    NNUE_REQUIRE(mode >= NNUE_BWD_AUTO && mode <= NNUE_BWD_SEGMENT, NNUE_ERR_ARG,
                 "nnue_ft_fused_bwd: unknown mode %d", mode);
    NNUE_REQUIRE(n_slices >= 0 && n_slices <= NNUE_BWD_MAX_SLICES, NNUE_ERR_ARG,
                 "nnue_ft_fused_bwd_sliced: 0..%d slices, got %d", NNUE_BWD_MAX_SLICES, n_slices);
    const bool by_columns = n_slices > 0 && slices->by_columns != 0;
    if (by_columns) {
        const int tile_w = csr_column_tile(L1 + P);
        NNUE_REQUIRE(slices->row_bounds[0] == 0 && slices->row_bounds[n_slices] == (int64_t)L1 + P, NNUE_ERR_ARG,
                     "nnue_ft_fused_bwd_sliced: column bounds must run from 0 to L1 + P = %d", L1 + P);
        for (int i = 0; i < n_slices; ++i) {
            NNUE_REQUIRE(slices->row_bounds[i] <= slices->row_bounds[i + 1], NNUE_ERR_ARG,
                         "nnue_ft_fused_bwd_sliced: column bounds must not decrease");
            NNUE_REQUIRE(tile_w > 0 && (i == 0 || slices->row_bounds[i] % tile_w == 0 || slices->row_bounds[i] == (int64_t)L1 + P),
                         NNUE_ERR_ARG, "nnue_ft_fused_bwd_sliced: inner column bounds must be multiples of %d floats "
                         "(nnue_ft_fused_bwd_column_tile)", tile_w);
        }
    } else if (n_slices > 0) {
        NNUE_REQUIRE(slices->row_bounds[0] == 0 && slices->row_bounds[n_slices] == N, NNUE_ERR_ARG,
                     "nnue_ft_fused_bwd_sliced: row bounds must run from 0 to N = %lld", (long long)N);
        for (int i = 0; i < n_slices; ++i)
            NNUE_REQUIRE(slices->row_bounds[i] <= slices->row_bounds[i + 1], NNUE_ERR_ARG,
                         "nnue_ft_fused_bwd_sliced: row bounds must not decrease");
    }
    NNUE_REQUIRE(grad_weight && grad_bias, NNUE_ERR_ARG, "nnue_ft_fused_bwd: null output");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t W = (int64_t)L1 + P;
    if (B == 0 || K == 0) {
        if (N > 0) NNUE_CUDA_TRY(cudaMemsetAsync(grad_weight, 0, (size_t)N * W * sizeof(float), s));
        if (B == 0) {
            NNUE_CUDA_TRY(cudaMemsetAsync(grad_bias, 0, (size_t)W * sizeof(float), s));
            return record_all(s);
        }
    }
    NNUE_REQUIRE(us && them && white_idx && black_idx && psqt_idx && grad_l0 && grad_wpsqt &&
                     grad_bpsqt && saved,
                 NNUE_ERR_ARG, "nnue_ft_fused_bwd: null pointer");
    NNUE_REQUIRE(2 * B < 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "nnue_ft_fused_bwd: batch too large");
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "nnue_ft_fused_bwd: no device status word");
    mode = resolve_mode(mode);
    const bool vec = fused_vec_ok(L1, P, grad_l0, saved, grad_weight, grad_bias, grad_weight);
    // unaligned buffers send the atomic mode down the segment route as well
    const size_t need = nnue_ft_fused_bwd_workspace_bytes(
        B, K, N, L1, P, (mode == NNUE_BWD_ATOMIC && vec) ? NNUE_BWD_ATOMIC : NNUE_BWD_SEGMENT);
    NNUE_REQUIRE(workspace && workspace_bytes >= need, NNUE_ERR_WORKSPACE,
                 "nnue_ft_fused_bwd: workspace %zu bytes < required %zu", workspace_bytes, need);

    if (mode == NNUE_BWD_ATOMIC && vec) {
        NNUE_CUDA_TRY(cudaMemsetAsync(grad_weight, 0, (size_t)N * W * sizeof(float), s));
        NNUE_CUDA_TRY(cudaMemsetAsync(grad_bias, 0, (size_t)W * sizeof(float), s));
        const int h4 = L1 / 8;
        int U = tuning().bwd_u;
        if (U != 1 && U != 2) U = 2;
        while (U > 1 && h4 <= 32 * (U / 2)) U /= 2;
        const int tiles = (h4 + 32 * U - 1) / (32 * U);
        const int ppc = 64;
        const int64_t groups = (B + ppc - 1) / ppc;
        const unsigned grid = (unsigned)(groups * tiles);
        ProfScope prof("k_fused_bwd_atomic", s);
        if (U == 1)
            k_fused_bwd_atomic<1><<<grid, kThreads, 0, s>>>(us, them, white_idx, black_idx, psqt_idx,
                                                           act, grad_l0, grad_wpsqt, grad_bpsqt,
                                                           saved, grad_weight, grad_bias, B, K, N, L1,
                                                           P, (int)groups, ppc, status);
        else
            k_fused_bwd_atomic<2><<<grid, kThreads, 0, s>>>(us, them, white_idx, black_idx, psqt_idx,
                                                           act, grad_l0, grad_wpsqt, grad_bpsqt,
                                                           saved, grad_weight, grad_bias, B, K, N, L1,
                                                           P, (int)groups, ppc, status);
        NNUE_CUDA_TRY(cudaGetLastError());
        note_launches(1);
        return record_all(s);
    }

    // segment mode (also the route of the scalar shapes)
    char* ws = static_cast<char*>(workspace);
    ws = reinterpret_cast<char*>(align_up(reinterpret_cast<uintptr_t>(ws), 256));
    float* G = reinterpret_cast<float*>(ws);
    ws += align_up((size_t)(2 * B) * W * sizeof(float), 256);
    const int pb = tuning().prologue_pb;
    const int64_t nblk = (B + pb - 1) / pb;
    float* bias_part = reinterpret_cast<float*>(ws);
    ws += align_up((size_t)nblk * W * sizeof(float), 256);

    // CSR over both perspectives: entry id = 2*p + perspective = row of G.  It depends on the
    // index lists only, so it is built on the helper stream while the prologue streams G.
    CsrPlan plan;
    int rc = csr_plan(plan, 2, B, K, N, (int)W, ws,
                      workspace_bytes - (size_t)(ws - static_cast<char*>(workspace)));
    if (rc != NNUE_OK) return rc;
    const int32_t* lists[2] = {white_idx, black_idx};
    CsrJoin join;
    rc = csr_build_overlapped(plan, lists, s, join);

    int64_t part_rows = 0;
    const float* part_src = nullptr;
    cudaError_t launch_err = cudaSuccess;
    if (rc == NNUE_OK) {
        if (vec) {
            const int cols4 = L1 / 8 + P / 4;
            const int chunks = (cols4 + kThreads - 1) / kThreads;
            ProfScope prof("k_bwd_prologue", s);
            k_bwd_prologue<<<(unsigned)(nblk * chunks), kThreads, 0, s>>>(
                us, them, psqt_idx, act, grad_l0, grad_wpsqt, grad_bpsqt, saved, G, bias_part, B,
                L1, P, pb, chunks);
            part_rows = nblk;
            part_src = bias_part;
        } else {
            k_bwd_prologue_scalar<<<(unsigned)B, 128, 0, s>>>(us, them, psqt_idx, act, grad_l0,
                                                             grad_wpsqt, grad_bpsqt, saved, G, B, L1,
                                                             P);
            part_rows = 2 * B;  // bias = column sum of G itself
            part_src = G;
        }
        launch_err = cudaGetLastError();
        note_launches(1);
        if (launch_err == cudaSuccess) rc = column_sum(part_src, part_rows, (int)W, grad_bias, s);
    }
    const int rj = csr_join(join, s);  // always: the caller's stream must see the helper's work
    if (launch_err != cudaSuccess) return cuda_fail(launch_err, "backward prologue launch");
    if (rc != NNUE_OK) return rc;
    if (rj != NNUE_OK) return rj;
    if (n_slices > 0 && vec && plan.S > 0) {
        // the gradient in row slices, an event after each: a consumer on another stream (the
        // data-parallel reduce) starts on slice i while slice i + 1 is computed
        if (by_columns) {
            // Column slices write disjoint columns, so their launches need no order among themselves: they
            // alternate between the caller's stream and the helper stream, and the CTAs of slice i + 1 fill the
            // SMs that the last wave of slice i leaves idle (each slice is only a few waves long).
            SideStreamView side;
            const bool two = tuning().col_slice_streams != 0 && n_slices > 1 && side_stream_get(side);
            if (two) {
                NNUE_CUDA_TRY(cudaEventRecord(side.fork, s));  // the helper sees G, the CSR and the caller's earlier work
                NNUE_CUDA_TRY(cudaStreamWaitEvent(side.stream, side.fork, 0));
            }
            int rc_all = NNUE_OK;
            for (int i = 0; i < n_slices; ++i) {
                cudaStream_t st = (two && (i & 1)) ? side.stream : s;
                rc = csr_reduce(plan, G, (int)W, grad_weight, st, 0, -1, slices->row_bounds[i], slices->row_bounds[i + 1]);
                if (rc != NNUE_OK) { rc_all = rc; break; }
                if (slices->events[i] && cudaEventRecord(static_cast<cudaEvent_t>(slices->events[i]), st) != cudaSuccess) {
                    rc_all = cuda_fail(cudaGetLastError(), "slice event");
                    break;
                }
            }
            if (two) {  // always: the caller's stream must see the helper's work
                NNUE_CUDA_TRY(cudaEventRecord(side.join, side.stream));
                NNUE_CUDA_TRY(cudaStreamWaitEvent(s, side.join, 0));
            }
            return rc_all;
        }
        for (int i = 0; i < n_slices; ++i) {
            rc = csr_reduce(plan, G, (int)W, grad_weight, s, slices->row_bounds[i], slices->row_bounds[i + 1]);
            if (rc != NNUE_OK) return rc;
            if (slices->events[i])
                NNUE_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(slices->events[i]), s));
        }
        return NNUE_OK;
    }
    rc = csr_reduce(plan, G, (int)W, grad_weight, s);  // shapes the sliced reduction does not cover: all at once
    if (rc != NNUE_OK) return rc;
    return record_all(s);
}

// ---- mode = auto: which scatter strategy ---------------------------------------------------------
// The segment reduction wins as soon as a position activates more than a handful of rows; on nearly
// empty boards its fixed costs (one gradient row per (position, perspective) written and read, the
// CSR) exceed the whole atomic scatter.  Which case applies is a property of the data, known only on
// the device, and the host must not wait for it: every auto call leaves the number of active entries
// of its lists in pinned host memory (a tiny kernel after the real work), and the NEXT auto call of
// the same batch size reads whatever count has arrived by then.  Training data (about 34 rows per
// list) always take the segment route; mode = segment forces it (and its reproducible sums).
struct DensityProbe {
    long long* h = nullptr;        // pinned, mapped: [0] active entries, [1] lists counted (2 B)
    long long* h_dev = nullptr;    // device view of h
    unsigned long long* d = nullptr;  // device: [0] running entry count, [1] CTAs done
    unsigned calls = 0;
};
static DensityProbe* density_probe() {
    static DensityProbe table[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    DensityProbe& t = table[dev];
    if (!t.h) {
        if (cudaHostAlloc(reinterpret_cast<void**>(&t.h), 2 * sizeof(long long), cudaHostAllocMapped) != cudaSuccess) {
            t.h = nullptr;
            cudaGetLastError();
            return nullptr;
        }
        t.h[0] = t.h[1] = 0;
        if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&t.h_dev), t.h, 0) != cudaSuccess ||
            cudaMalloc(reinterpret_cast<void**>(&t.d), 2 * sizeof(unsigned long long)) != cudaSuccess ||
            cudaMemset(t.d, 0, 2 * sizeof(unsigned long long)) != cudaSuccess) {
            cudaGetLastError();
            cudaFreeHost(t.h);
            t.h = nullptr;
            return nullptr;
        }
    }
    return &t;
}

namespace nnue {
// warp per position: active entries of its two lists; the CTA that finishes last publishes the total
__global__ void __launch_bounds__(kThreads)
    k_density_probe(const int32_t* __restrict__ wi, const int32_t* __restrict__ bi, int64_t B, int K,
                    unsigned long long* __restrict__ d, long long* __restrict__ h_out) {
    __shared__ int s_n[kWarpsPerCta];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int n = 0;
    for (int64_t p = (int64_t)blockIdx.x * kWarpsPerCta + warp; p < B; p += (int64_t)gridDim.x * kWarpsPerCta)
        n += count_active(wi + p * K, K, lane) + count_active(bi + p * K, K, lane);
    if (lane == 0) s_n[warp] = n;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int w = 0; w < kWarpsPerCta; ++w) t += s_n[w];
        atomicAdd(d, (unsigned long long)t);
        __threadfence();
        if (atomicAdd(d + 1, 1ULL) == gridDim.x - 1) {
            __threadfence();
            h_out[0] = (long long)atomicExch(d, 0ULL);
            h_out[1] = 2 * B;
            d[1] = 0;
            __threadfence_system();
        }
    }
}
}  // namespace nnue

constexpr long long kAtomicBelowRowsPerList = 6;

extern "C" int nnue_ft_fused_bwd_sliced(const float* us, const float* them, const int32_t* white_idx,
                                        const int32_t* black_idx, const int64_t* psqt_idx, float max_act,
                                        float out_scale, const float* grad_l0, const float* grad_wpsqt,
                                        const float* grad_bpsqt, const float* saved, float* grad_weight,
                                        float* grad_bias, int64_t B, int32_t K, int64_t N, int32_t L1,
                                        int32_t P, void* workspace, size_t workspace_bytes, int32_t mode,
                                        const nnue_bwd_slices* h_slices, void* stream) {
    int run_mode = mode;
    const bool sliced = h_slices != nullptr && h_slices->n_slices > 0;
    DensityProbe* probe = nullptr;
    if (mode == NNUE_BWD_AUTO && B > 0 && K > 0 && white_idx && black_idx && !sliced) {
        probe = density_probe();
        if (probe) {
            const volatile long long* h = probe->h;
            const long long entries = h[0], lists = h[1];
            const bool known = lists == 2 * B;
            if (known && entries < kAtomicBelowRowsPerList * lists) run_mode = NNUE_BWD_ATOMIC;
            // dense data of a known batch size (training): look again only every fourth call
            if (known && run_mode != NNUE_BWD_ATOMIC && (++probe->calls & 3) != 0) probe = nullptr;
        }
    }
    // the count for the next call runs on the helper stream, beside the real work
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    SideStreamView side;
    bool probing = false;
    if (probe && side_stream_get(side)) {
        NNUE_CUDA_TRY(cudaEventRecord(side.fork, s));
        NNUE_CUDA_TRY(cudaStreamWaitEvent(side.stream, side.fork, 0));
        const unsigned grid = (unsigned)((B + kWarpsPerCta - 1) / kWarpsPerCta);  // a warp per position: 4 loads deep
        k_density_probe<<<grid, kThreads, 0, side.stream>>>(white_idx, black_idx, B, K, probe->d, probe->h_dev);
        NNUE_CUDA_TRY(cudaGetLastError());
        note_launches(1);
        probing = true;
    }
    const int rc = fused_bwd_impl(us, them, white_idx, black_idx, psqt_idx, max_act, out_scale, grad_l0,
                                  grad_wpsqt, grad_bpsqt, saved, grad_weight, grad_bias, B, K, N, L1, P,
                                  workspace, workspace_bytes, run_mode, sliced ? h_slices : nullptr, stream);
    if (probing) {  // the caller's stream must not outrun a reader of its index lists
        NNUE_CUDA_TRY(cudaEventRecord(side.join, side.stream));
        NNUE_CUDA_TRY(cudaStreamWaitEvent(s, side.join, 0));
    }
    return rc;
}

extern "C" int nnue_ft_fused_bwd(const float* us, const float* them, const int32_t* white_idx,
                                 const int32_t* black_idx, const int64_t* psqt_idx, float max_act,
                                 float out_scale, const float* grad_l0, const float* grad_wpsqt,
                                 const float* grad_bpsqt, const float* saved, float* grad_weight,
                                 float* grad_bias, int64_t B, int32_t K, int64_t N, int32_t L1,
                                 int32_t P, void* workspace, size_t workspace_bytes, int32_t mode,
                                 void* stream) {
    return nnue_ft_fused_bwd_sliced(us, them, white_idx, black_idx, psqt_idx, max_act, out_scale, grad_l0,
                                    grad_wpsqt, grad_bpsqt, saved, grad_weight, grad_bias, B, K, N, L1, P,
                                    workspace, workspace_bytes, mode, nullptr, stream);
}
