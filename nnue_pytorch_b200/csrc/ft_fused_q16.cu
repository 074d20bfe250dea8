// Fused double feature transformer, forward, gathering an int16 table.
//
// With weight fake quantization on (the reference's default,
// model/modules/feature_transformer/composed_feature_transformer.py:61-76 with
// model/quantize.py:47-56) every entry of the table the operator reads is
// k / scale with integer k and scale = 256.  For |k| <= 32767 and at most 511
// rows per list, the fp32 sum "bias first, rows in list order" never rounds
// (every partial sum is a multiple of 1/scale below 2^24 / scale), so the same
// bits come out of an int32 sum of the k followed by one multiplication by
// 1/scale.  The kernel reads half the bytes of the fp32 form through the
// L2 -> SM path, which is what bounds the fp32 kernel.
//
// Decomposition: warp = (position, perspective, column tile), tiles the slow
// grid dimension as in k_fused_fwd, a tile being 256 columns of each half: one
// 16-byte load of eight int16 per lane and half, summed as four packed pairs
// (see PairAcc).  The two warps of a position swap their sums through shared
// memory and each writes one half of the outputs.
//
// A table that left the int16 range (the emitting kernel tallies that in a
// device word, the host never waits for it) is served from the fp32 parameters
// instead: the same kernel then gathers weight (+ factor rows) and applies
// round(x * scale) / scale per element.  Slower, same results.
#include "ft_fused.cuh"
#include "gather_q16.cuh"

namespace nnue {

constexpr int kMaxBlocks = 8;
struct MasterBlocks {
    int n;
    const float* weight[kMaxBlocks];
    const float* virt[kMaxBlocks];
    long long row0[kMaxBlocks + 1];   // first table row of each block; row0[n] = N
    long long n_virtual[kMaxBlocks];
};

__device__ __forceinline__ float fq_pow2(float x, float scale, float inv_scale) {
    return __fmul_rn(rintf(__fmul_rn(x, scale)), inv_scale);
}

// fp32 route: acc (float4 x 4: columns 2*c8, 2*c8+1 of each half) += fq(weight + virtual) of the listed rows.
// Whole-warp call (it shuffles the row ids); lanes beyond the last column pass ok = false and load nothing.
__device__ __noinline__ void gather_master(const MasterBlocks& mb, int W, int64_t n_rows, const int32_t* list, int n,
                                           int c8, int h4, bool ok, float scale, float inv_scale, float4 (&acc)[4],
                                           int lane, unsigned long long* status) {
    const int64_t W4 = W >> 2;
    for (int k0 = 0; k0 < n; k0 += 32) {
        const int m = min(32, n - k0);
        int mine = (lane < m) ? list[k0 + lane] : 0;
        if ((unsigned)mine >= (unsigned long long)n_rows) {
            if (lane < m) note_bad_index(status);
            mine = -1;
        }
        for (int j = 0; j < m; ++j) {
            const int r = __shfl_sync(kFullMask, mine, j);
            if (r < 0 || !ok) continue;
            int blk = 0;
            while (blk + 1 < mb.n && r >= mb.row0[blk + 1]) ++blk;
            const long long lr = r - mb.row0[blk];
            const float4* wrow = reinterpret_cast<const float4*>(mb.weight[blk]) + lr * W4;
            const float4* vrow = mb.virt[blk]
                                     ? reinterpret_cast<const float4*>(mb.virt[blk]) + (lr % mb.n_virtual[blk]) * W4
                                     : nullptr;
            const int cols[4] = {2 * c8, 2 * c8 + 1, h4 + 2 * c8, h4 + 2 * c8 + 1};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float4 x = ldg4(wrow + cols[q]);
                if (vrow) x = f4_add(x, ldg4(vrow + cols[q]));
                x = make_float4(fq_pow2(x.x, scale, inv_scale), fq_pow2(x.y, scale, inv_scale),
                                fq_pow2(x.z, scale, inv_scale), fq_pow2(x.w, scale, inv_scale));
                acc[q] = f4_add(acc[q], x);
            }
        }
    }
}

// One float4 column group of ONE output half: `mine` are this warp's perspective sums (columns c of the
// first half and of the second half), `other` the partner perspective's.  The white warp of a
// position produces the first half of l0 and the saved chunks 0, 1; the black warp, with the
// roles of the two perspectives swapped, the second half and chunks 2, 3
// (double_ft_functions.py:62-80: x = us * [w, b] + them * [b, w]).
__device__ __forceinline__ void store_half(float u_, float t_, float4 mine_lo, float4 mine_hi, float4 other_lo,
                                           float4 other_hi, int c, int h4, int side, float4* sv, float4* l0p,
                                           const FtAct& act) {
    const float4 xa = f4_mix(u_, mine_lo, t_, other_lo);
    const float4 xb = f4_mix(u_, mine_hi, t_, other_hi);
    st_stream4(sv + (2 * side) * h4 + c, xa);
    st_stream4(sv + (2 * side + 1) * h4 + c, xb);
    const float max_act = act.max_act;
    auto cl = [max_act](float x) { return fminf(fmaxf(x, 0.f), max_act); };
    auto pr = [&](float p, float q) { return finish_l0(__fmul_rn(cl(p), cl(q)), act); };
    st_stream4(l0p + side * h4 + c, make_float4(pr(xa.x, xb.x), pr(xa.y, xb.y), pr(xa.z, xb.z), pr(xa.w, xb.w)));
}

constexpr int kPosPerCta = kWarpsPerCta / 2;  // a warp per (position, perspective)
// A table beyond kMaxAbsPacked (weights above 16.0) goes the fp32 route like one beyond the int16 range.

// bias: fp32 [L1 + P], already fake-quantized at `scale` (its L1 part is k / scale), PSQT part as the op adds it.
// psqt_tab: fp32 [N, P], the fake-quantized PSQT columns of the table.
// stats: [0] entries outside the int16 range (non-zero: fp32 route), [1] max |k| of the table.
// q16 holds N + 1 rows, the last one all zeros.
// Warp 2q gathers the white list of the CTA's q-th position, warp 2q + 1 its black list (half the
// accumulators per warp, twice the warps per position); the pair swaps its sums through shared memory
// and each warp finishes one half of the outputs.
template <int R, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
    k_fused_fwd_q16(const float* __restrict__ us, const float* __restrict__ them,
                    const int32_t* __restrict__ wi, const int32_t* __restrict__ bi,
                    const int64_t* __restrict__ psqt_idx, const int16_t* __restrict__ q16, int64_t pitch8,
                    const float* __restrict__ psqt_tab, const float* __restrict__ bias, float scale,
                    float inv_scale, const int* __restrict__ stats, int n_stat_parts,
                    const __grid_constant__ MasterBlocks mb,
                    FtAct act, float* __restrict__ l0, float* __restrict__ wpsqt, float* __restrict__ bpsqt,
                    float* __restrict__ saved, int64_t B, int K, int64_t N, int L1, int P, int n_pos_groups,
                    int want_stage, unsigned long long* status) {
    extern __shared__ __align__(16) int32_t s_idx[];
    __shared__ __align__(16) float4 s_swap[kWarpsPerCta][4][32];
    __shared__ __align__(8) uint64_t bar;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int side = warp & 1, pair = warp >> 1;
    const int tile = blockIdx.x / n_pos_groups;
    const int64_t p0 = (int64_t)(blockIdx.x % n_pos_groups) * kPosPerCta;
    const int64_t p = p0 + pair;

    // the lists of the CTA's positions: two contiguous blocks of kPosPerCta * K entries (full CTAs only)
    const int32_t* list = (side ? bi : wi) + p * K;
    const bool stage = want_stage != 0 && (p0 + kPosPerCta <= B);  // uniform across the CTA
    if (stage) {
        const unsigned bytes = (unsigned)(kPosPerCta * K * sizeof(int32_t));
        if (threadIdx.x == 0) {
            mbar_init(&bar, 1);
            fence_barrier_init();
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            mbar_expect_tx(&bar, 2 * bytes);
            bulk_g2s(s_idx, wi + p0 * K, bytes, &bar);
            bulk_g2s(s_idx + kPosPerCta * K, bi + p0 * K, bytes, &bar);
        }
        if (mbar_wait_bounded(&bar, 0)) list = s_idx + (side * kPosPerCta + pair) * K;
        else if (lane == 0) note_timeout(status);  // keep going on the global-memory list
    }
    if (p >= B) return;  // both warps of a pair leave together

    const int h4 = L1 >> 3;   // float4 per half
    const int h8 = L1 >> 4;   // 16-byte groups of eight int16 per half
    const int c8 = tile * 32 + lane;
    const bool ok = c8 < h8;
    const int n = count_active(list, K, lane);
    const float4* bias4 = reinterpret_cast<const float4*>(bias);

    float4 f[4];  // this perspective: columns 2*c8, 2*c8+1 of the first half, then of the second half
    int overflow = 0, max_abs = 0;
    for (int i = 0; i < n_stat_parts; ++i) {
        overflow |= __ldg(stats + 2 * i);
        max_abs = max(max_abs, __ldg(stats + 2 * i + 1));
    }
    if (overflow == 0 && max_abs <= kMaxAbsPacked) {
        const int rows_per_split = max_abs > 0 ? min(32767 / max_abs, 512) : 512;  // >= 8 > R
        PairAcc acc;
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
            const float4 b0 = ok ? ldg4(bias4 + hlf * h4 + 2 * c8) : f4_zero();
            const float4 b1 = ok ? ldg4(bias4 + hlf * h4 + 2 * c8 + 1) : f4_zero();
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                acc.lo[hlf][w] = __float2int_rn(__fmul_rn(bv[2 * w], scale));
                acc.hi[hlf][w] = __float2int_rn(__fmul_rn(bv[2 * w + 1], scale));
            }
        }
        // lanes beyond the last column read column group 0 (valid memory); their sums are never stored
        const uint4* base0 = reinterpret_cast<const uint4*>(q16) + (ok ? c8 : 0);
        gather_q16<R>(base0, base0 + h8, (int)pitch8, (int)N, list, n, rows_per_split, acc, lane, status);
        auto cv = [inv_scale](int a) { return __fmul_rn(__int2float_rn(a), inv_scale); };
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
            f[2 * hlf] = make_float4(cv(acc.lo[hlf][0]), cv(acc.hi[hlf][0]), cv(acc.lo[hlf][1]), cv(acc.hi[hlf][1]));
            f[2 * hlf + 1] = make_float4(cv(acc.lo[hlf][2]), cv(acc.hi[hlf][2]), cv(acc.lo[hlf][3]), cv(acc.hi[hlf][3]));
        }
    } else {
        // some entry does not fit int16: the fp32 route on the parameters themselves (its accumulators live
        // in local memory behind the call; they are copied out so that the common path keeps registers)
        float4 sl[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) sl[q] = ok ? ldg4(bias4 + (q >> 1) * h4 + 2 * c8 + (q & 1)) : f4_zero();
        if (mb.weight[0] != nullptr) gather_master(mb, L1 + P, N, list, n, c8, h4, ok, scale, inv_scale, sl, lane, status);
        else if (lane == 0 && tile == 0) atomicAdd(status + 3, 1ULL);  // nothing to fall back to: reported, sums = bias
#pragma unroll
        for (int q = 0; q < 4; ++q) f[q] = sl[q];
    }

    // swap with the partner warp (named barrier of the pair: 64 threads)
#pragma unroll
    for (int q = 0; q < 4; ++q) s_swap[warp][q][lane] = f[q];
    asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");
    float4 o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) o[q] = s_swap[warp ^ 1][q][lane];

    const float u_ = __ldg(us + p), t_ = __ldg(them + p);
    float4* l0p = reinterpret_cast<float4*>(l0 + p * L1);
    float4* sv = reinterpret_cast<float4*>(saved + p * 2 * (int64_t)L1);
    if (ok) {
        store_half(u_, t_, f[0], f[2], o[0], o[2], 2 * c8, h4, side, sv, l0p, act);
        store_half(u_, t_, f[1], f[3], o[1], o[3], 2 * c8 + 1, h4, side, sv, l0p, act);
    }

    if (tile == 0) {
        const int64_t pi = __ldg(psqt_idx + p);
        float* out = side ? bpsqt : wpsqt;
        if (pi >= 0 && pi < P) {
            const float s = psqt_sum(psqt_tab, P, N, list, n, (int)pi, __ldg(bias + L1 + pi), lane);
            if (lane == 0) out[p] = s;
        } else if (lane == 0) {
            if (side == 0) note_bad_index(status);
            out[p] = 0.f;
        }
    }
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_ft_fused_fwd_q16(const float* us, const float* them, const int32_t* white_idx,
                                     const int32_t* black_idx, const int64_t* psqt_idx, const int16_t* q16,
                                     int64_t q16_pitch, const float* psqt, const float* bias_fq, float scale_main,
                                     const int32_t* d_overflow, int32_t n_stat_parts, const nnue_ft_block* h_blocks,
                                     int32_t n_blocks,
                                     float max_act, float act_quant_scale, float act_quant_eps, float out_scale,
                                     float* l0, float* wpsqt, float* bpsqt, float* saved, int64_t B, int32_t K,
                                     int64_t N, int32_t L1, int32_t P, void* stream) {
    int sc_exp = 0;
    const bool pow2 = act_quant_scale > 0.f && frexpf(act_quant_scale, &sc_exp) == 0.5f;
    const FtAct act{max_act, act_quant_scale, act_quant_eps, out_scale, pow2 ? 1.0f / act_quant_scale : 0.f};
    NNUE_REQUIRE(B >= 0 && K >= 0 && N >= 0 && L1 > 0 && P >= 0, NNUE_ERR_ARG, "nnue_ft_fused_fwd_q16: negative size");
    NNUE_REQUIRE(L1 % 16 == 0 && P % 4 == 0, NNUE_ERR_UNSUPPORTED,
                 "nnue_ft_fused_fwd_q16: needs L1 %% 16 == 0 and P %% 4 == 0 (L1=%d P=%d)", L1, P);
    NNUE_REQUIRE(q16_pitch >= L1 && q16_pitch % 8 == 0, NNUE_ERR_ARG,
                 "nnue_ft_fused_fwd_q16: the row pitch (%lld) must be a multiple of 8 not below L1", (long long)q16_pitch);
    NNUE_REQUIRE((N + 1) * (q16_pitch / 8) < 0x7fffffffLL, NNUE_ERR_UNSUPPORTED,
                 "nnue_ft_fused_fwd_q16: table too large for 32-bit row offsets");
    NNUE_REQUIRE(K <= 511, NNUE_ERR_UNSUPPORTED,
                 "nnue_ft_fused_fwd_q16: at most 511 rows per list keep the integer sum exact (K=%d)", K);
    NNUE_REQUIRE(scale_main > 0.f && frexpf(scale_main, &sc_exp) == 0.5f, NNUE_ERR_UNSUPPORTED,
                 "nnue_ft_fused_fwd_q16: the scale must be a power of two (got %g)", (double)scale_main);
    NNUE_REQUIRE(n_stat_parts >= 1 && n_stat_parts <= 64, NNUE_ERR_ARG, "nnue_ft_fused_fwd_q16: 1..64 statistics parts");
    NNUE_REQUIRE(n_blocks >= 1 && n_blocks <= kMaxBlocks && h_blocks, NNUE_ERR_ARG,
                 "nnue_ft_fused_fwd_q16: 1..%d parameter blocks", kMaxBlocks);
    MasterBlocks mb;
    mb.n = n_blocks;
    long long at = 0;
    for (int i = 0; i < n_blocks; ++i) {
        const nnue_ft_block& b = h_blocks[i];
        NNUE_REQUIRE(b.rows >= 0 && (b.rows == 0 || b.weight || n_blocks == 1), NNUE_ERR_ARG,
                     "nnue_ft_fused_fwd_q16: block %d has no weights (allowed for a single block only)", i);
        NNUE_REQUIRE(!b.virtual_weight || (b.n_virtual > 0 && b.rows % b.n_virtual == 0), NNUE_ERR_ARG,
                     "nnue_ft_fused_fwd_q16: block %d: rows are not a multiple of the factor rows", i);
        NNUE_REQUIRE(aligned16(b.weight) && aligned16(b.virtual_weight), NNUE_ERR_ALIGN,
                     "nnue_ft_fused_fwd_q16: block %d is not 16-byte aligned", i);
        mb.weight[i] = b.weight;
        mb.virt[i] = b.virtual_weight;
        mb.n_virtual[i] = b.virtual_weight ? b.n_virtual : 1;
        mb.row0[i] = at;
        at += b.rows;
    }
    mb.row0[n_blocks] = at;
    NNUE_REQUIRE(at == N, NNUE_ERR_ARG, "nnue_ft_fused_fwd_q16: the blocks hold %lld rows, the table %lld", at, (long long)N);
    if (B == 0) return NNUE_OK;
    NNUE_REQUIRE(us && them && white_idx && black_idx && psqt_idx && q16 && bias_fq && d_overflow && l0 && wpsqt &&
                     bpsqt && saved && (psqt || P == 0),
                 NNUE_ERR_ARG, "nnue_ft_fused_fwd_q16: null pointer");
    NNUE_REQUIRE(aligned16(q16) && aligned16(bias_fq) && aligned16(l0) && aligned16(saved), NNUE_ERR_ALIGN,
                 "nnue_ft_fused_fwd_q16: 16-byte aligned buffers");
    NNUE_REQUIRE(B * (int64_t)K < (1LL << 40), NNUE_ERR_UNSUPPORTED, "nnue_ft_fused_fwd_q16: batch too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "nnue_ft_fused_fwd_q16: no device status word");

    const int h8 = L1 / 16;
    const int tiles = (h8 + 31) / 32;
    const int64_t groups = (B + kPosPerCta - 1) / kPosPerCta;
    NNUE_REQUIRE(groups * tiles <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "nnue_ft_fused_fwd_q16: grid too large");
    const size_t smem = (size_t)2 * kPosPerCta * K * sizeof(int32_t);
    // the bulk copies move kPosPerCta * K * 4 bytes from offsets that are multiples of it: K % 4 keeps both 16-byte aligned
    const int stage = tuning().stage_idx && K > 0 && K % 4 == 0 && smem <= 32 * 1024 && aligned16(white_idx) &&
                      aligned16(black_idx);
    const unsigned grid = (unsigned)(groups * tiles);
    const float inv_scale = 1.0f / scale_main;
    ProfScope prof("k_fused_fwd_q16", s);
#define LAUNCH_Q16(RR, MB)                                                                                  \
    k_fused_fwd_q16<RR, MB><<<grid, kThreads, stage ? smem : 0, s>>>(                                       \
        us, them, white_idx, black_idx, psqt_idx, q16, q16_pitch / 8, psqt, bias_fq, scale_main, inv_scale,    \
        d_overflow, n_stat_parts, mb,                                                                       \
        act, l0, wpsqt, bpsqt, saved, B, K, N, L1, P, (int)groups, stage, status)
    // variant = rows in flight per warp (R) and CTAs per SM the register budget must allow
    const int v = tuning().fwd_q16_variant;
    // measured at L1 = 3072, batch 16384: (3, 4) 0.49 ms, (4, 4) 0.52, (4, 3) 0.52, (6, 3) 0.53, (2, 5) 0.60
    if (v == 1) LAUNCH_Q16(4, 3);
    else if (v == 2) LAUNCH_Q16(4, 4);
    else if (v == 3) LAUNCH_Q16(2, 5);
    else if (v == 4) LAUNCH_Q16(6, 3);
    else LAUNCH_Q16(3, 4);
#undef LAUNCH_Q16
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
