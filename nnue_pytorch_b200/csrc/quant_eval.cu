// Integer evaluation of a quantized net: int16 feature-transformer gather,
// pairwise product >> ft_shift, three int8 layers of the selected layer
// stack, truncating output division and the PSQT term.  Integer restatement
// of the fake-quantized float forward of the reference project
// (model/quantize.py:36-56,133-147, model/modules/layer_stacks.py:33-84,
// model/model.py:107-133); the reference holds no integer evaluator.
//
// One CTA per position (grid-stride).  Thread t owns the 8 int16 columns
// [8t, 8t+8) of the first half of the accumulator and the same columns of the
// second half, for both perspectives: every row read is one 16-byte load per
// half per thread, 384 B contiguous per warp.
#include <algorithm>

#include "common.cuh"
#include "gather_q16.cuh"

namespace nnue {

constexpr int kQThreads = 192;
constexpr int kQMaxL2 = 64;   // widest hidden layers this kernel takes
constexpr int kQRowsInFlight = 4;

struct QuantDims {
    int K, L1, L2, L3, P, buckets;
    int64_t N;
};

__device__ __forceinline__ void add8(int (&acc)[8], uint4 v) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        acc[2 * j] += (int)(short)(w[j] & 0xffffu);
        acc[2 * j + 1] += (int)(short)(w[j] >> 16);
    }
}

__device__ __forceinline__ int clampi(int x, int lo, int hi) { return x < lo ? lo : (x > hi ? hi : x); }

// The three int8 layers of one position whose clipped products sit in s_x0; every thread of the
// CTA takes part (CTA-wide barriers inside).  The PSQT term enters as (side to move) - (other side):
// white - black with white to move, -(white - black) otherwise.
__device__ __forceinline__ void quant_layers(const int8_t* s_x0, int32_t* s_o1, int8_t* s_x1, int bk,
                                             const QuantDims& d, const nnue_quant_params& q,
                                             const int8_t* __restrict__ l1_w, const int32_t* __restrict__ l1_b,
                                             const int8_t* __restrict__ l2_w, const int32_t* __restrict__ l2_b,
                                             const int8_t* __restrict__ out_w, const int32_t* __restrict__ out_b,
                                             long long psq_us_minus_them, int32_t* out_p) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nwarps = blockDim.x >> 5;
    // layer 1: L2 outputs over L1 int8 inputs, dp4a on 16-byte chunks
    {
        const int chunks = d.L1 >> 4;
        const int4* xin = reinterpret_cast<const int4*>(s_x0);
        for (int o = warp; o < d.L2; o += nwarps) {
            const int4* wrow = reinterpret_cast<const int4*>(l1_w + ((int64_t)bk * d.L2 + o) * d.L1);
            int acc = 0;
            for (int ch = lane; ch < chunks; ch += 32) {
                const int4 w = __ldg(wrow + ch);
                const int4 a = xin[ch];
                acc = __dp4a(a.x, w.x, acc);
                acc = __dp4a(a.y, w.y, acc);
                acc = __dp4a(a.z, w.z, acc);
                acc = __dp4a(a.w, w.w, acc);
            }
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(kFullMask, acc, s);
            if (lane == 0) s_o1[o] = acc + l1_b[bk * d.L2 + o];
        }
    }
    __syncthreads();

    if (warp == 0) {
        // squared and linear activations of layer 1 -> x1[0 .. 2*L2)
        for (int o = lane; o < d.L2; o += 32) {
            const long long v = s_o1[o];
            const long long sq = (v * v + q.sqr_eps_l1) >> q.sqr_shift_l1;
            s_x1[o] = (int8_t)(sq > q.hidden_max ? q.hidden_max : sq);
            s_x1[d.L2 + o] = (int8_t)clampi((int)(v >> q.lin_shift_l1), 0, q.hidden_max);
        }
        __syncwarp();
        // layer 2: lane = output
        const int in2 = 2 * d.L2;
        for (int o = lane; o < d.L3; o += 32) {
            const int8_t* wrow = l2_w + ((int64_t)bk * d.L3 + o) * in2;
            int acc = l2_b[bk * d.L3 + o];
            if ((in2 & 3) == 0 && ((reinterpret_cast<uintptr_t>(wrow) | reinterpret_cast<uintptr_t>(s_x1)) & 3u) == 0) {
                const int* xi = reinterpret_cast<const int*>(s_x1);
                const int* wi = reinterpret_cast<const int*>(wrow);
                for (int i = 0; i < (in2 >> 2); ++i) acc = __dp4a(xi[i], __ldg(wi + i), acc);
            } else {
                for (int i = 0; i < in2; ++i) acc += (int)s_x1[i] * (int)wrow[i];
            }
            const long long v = acc;
            const long long sq = (v * v + q.sqr_eps_l2) >> q.sqr_shift_l2;
            s_x1[in2 + o] = (int8_t)(sq > q.hidden_max ? q.hidden_max : sq);
            s_x1[in2 + d.L3 + o] = (int8_t)clampi((int)(v >> q.lin_shift_l2), 0, q.hidden_max);
        }
        __syncwarp();
        // output layer: one value over 2*L2 + 2*L3 inputs
        const int in3 = 2 * d.L2 + 2 * d.L3;
        const int8_t* wrow = out_w + (int64_t)bk * in3;
        int acc = 0;
        for (int i = lane; i < in3; i += 32) acc += (int)s_x1[i] * (int)wrow[i];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(kFullMask, acc, s);
        if (lane == 0) {
            const long long o3 = (long long)acc + out_b[bk];
            const long long skip = ((long long)s_o1[d.L2 - 2] - (long long)s_o1[d.L2 - 1]) * q.skip_mul;
            const long long num = 2 * (o3 + skip) * (long long)q.out_mul;
            const long long pos = num / q.out_div;  // C++ division truncates toward zero
            *out_p = (int32_t)(2 * pos + psq_us_minus_them);
        }
    }
}

__global__ void __launch_bounds__(kQThreads)
    k_quant_eval(const int32_t* __restrict__ white_idx, const int32_t* __restrict__ black_idx,
                 const uint8_t* __restrict__ stm_white, const int32_t* __restrict__ bucket,
                 const int16_t* __restrict__ ft_w, const int32_t* __restrict__ ft_psqt,
                 const int32_t* __restrict__ ft_b, const int8_t* __restrict__ l1_w,
                 const int32_t* __restrict__ l1_b, const int8_t* __restrict__ l2_w,
                 const int32_t* __restrict__ l2_b, const int8_t* __restrict__ out_w,
                 const int32_t* __restrict__ out_b, int32_t* __restrict__ out, int64_t B, QuantDims d,
                 nnue_quant_params q, unsigned long long* status) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    int8_t* s_x0 = reinterpret_cast<int8_t*>(s_raw);                  // [L1]
    int32_t* s_o1 = reinterpret_cast<int32_t*>(s_raw + d.L1);         // [L2]
    int8_t* s_x1 = reinterpret_cast<int8_t*>(s_o1 + kQMaxL2);         // [2*L2 + 2*L3]
    __shared__ int s_psq[2];
    __shared__ int s_n[2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nwarps = kQThreads / 32;
    const int h = d.L1 >> 1;
    const int h8 = h >> 3;  // 16-byte chunks per half

    for (int64_t p = blockIdx.x; p < B; p += gridDim.x) {
        const int stm = stm_white[p] ? 1 : 0;
        int bk = bucket[p];
        if (bk < 0 || bk >= d.buckets || bk >= d.P) {
            if (tid == 0) note_bad_index(status);
            bk = 0;
        }
        // "us" is the side to move: its accumulator forms the first half of l0
        const int32_t* lists[2] = {stm ? white_idx + p * d.K : black_idx + p * d.K,
                                   stm ? black_idx + p * d.K : white_idx + p * d.K};
        if (tid < 2) s_psq[tid] = 0;
        if (warp < 2) {
            const int n = count_active(lists[warp], d.K, lane);
            if (lane == 0) s_n[warp] = n;
        }
        __syncthreads();
        // PSQT: integer adds commute, so any order gives the same sum
        for (int s = 0; s < 2; ++s) {
            int psq = 0;
            for (int k = tid; k < s_n[s]; k += kQThreads) {
                const int r = lists[s][k];
                if (r >= 0 && (int64_t)r < d.N) psq += ft_psqt[(int64_t)r * d.P + bk];
                else note_bad_index(status);
            }
            if (psq) atomicAdd(&s_psq[s], psq);
        }

        for (int c0 = 0; c0 < h8; c0 += kQThreads) {
            const int c = c0 + tid;
            const bool live = c < h8;
            int x[2][2][8];  // [perspective][half][column]
            for (int s = 0; s < 2; ++s) {
                if (live) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        x[s][0][j] = ft_b[8 * c + j];
                        x[s][1][j] = ft_b[h + 8 * c + j];
                    }
                }
                const int32_t* list = lists[s];
                const int n = s_n[s];
                for (int k0 = 0; k0 < n; k0 += kQRowsInFlight) {
                    uint4 v[kQRowsInFlight][2];
                    bool ok[kQRowsInFlight];
#pragma unroll
                    for (int t = 0; t < kQRowsInFlight; ++t) {
                        const int r = (k0 + t < n) ? list[k0 + t] : -1;
                        ok[t] = r >= 0 && (int64_t)r < d.N;
                        if (ok[t] && live) {
                            const uint4* row = reinterpret_cast<const uint4*>(ft_w + (int64_t)r * d.L1);
                            v[t][0] = __ldg(row + c);
                            v[t][1] = __ldg(row + h8 + c);
                        }
                    }
#pragma unroll
                    for (int t = 0; t < kQRowsInFlight; ++t) {
                        if (ok[t] && live) {
                            add8(x[s][0], v[t][0]);
                            add8(x[s][1], v[t][1]);
                        }
                    }
                }
            }
            if (live) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int a0 = clampi(x[0][0][j], 0, q.ft_max), a1 = clampi(x[0][1][j], 0, q.ft_max);
                    const int b0 = clampi(x[1][0][j], 0, q.ft_max), b1 = clampi(x[1][1][j], 0, q.ft_max);
                    s_x0[8 * c + j] = (int8_t)min((a0 * a1) >> q.ft_shift, q.hidden_max);
                    s_x0[h + 8 * c + j] = (int8_t)min((b0 * b1) >> q.ft_shift, q.hidden_max);
                }
            }
        }
        __syncthreads();

        quant_layers(s_x0, s_o1, s_x1, bk, d, q, l1_w, l1_b, l2_w, l2_b, out_w, out_b,
                     (long long)s_psq[0] - (long long)s_psq[1], out + p);
        __syncthreads();
    }
}

// ---- two-kernel form: gather with an L2-resident table slice, then the layers -----------------
// k_quant_gather is the integer twin of the fused feature-transformer forward: warp = (position,
// column tile of 256 int16 per half), tiles the slow grid dimension, so the 23232 x 512 B slice of
// the table a tile touches stays in the L2 while all positions pass over it.  It leaves the clipped
// pairwise products (int8 [B, L1]) and the PSQT difference in the workspace; k_quant_layers then
// runs the three small layers, one CTA per position.
constexpr int kQGatherRows = 4;

__global__ void __launch_bounds__(kThreads, 3)
    k_quant_gather(const int32_t* __restrict__ white_idx, const int32_t* __restrict__ black_idx,
                   const uint8_t* __restrict__ stm_white, const int32_t* __restrict__ bucket,
                   const int16_t* __restrict__ ft_w, const int32_t* __restrict__ ft_psqt,
                   const int32_t* __restrict__ ft_b, int8_t* __restrict__ x0, int32_t* __restrict__ psq,
                   int64_t p_begin, int64_t p_end, QuantDims d, nnue_quant_params q, int n_groups,
                   unsigned long long* status) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tile = blockIdx.x / n_groups;
    const int64_t p = p_begin + (int64_t)(blockIdx.x % n_groups) * kWarpsPerCta + warp;
    if (p >= p_end) return;
    const int h = d.L1 >> 1, h8 = h >> 3;
    const int c = tile * 32 + lane;
    const bool live = c < h8;
    const int stm = stm_white[p] ? 1 : 0;
    const int32_t* lists[2] = {stm ? white_idx + p * d.K : black_idx + p * d.K,
                               stm ? black_idx + p * d.K : white_idx + p * d.K};
    int x[2][2][8];  // [us / them][half][column]
    int n_act[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        if (live) {
            const int4* b0 = reinterpret_cast<const int4*>(ft_b + 8 * c);
            const int4* b1 = reinterpret_cast<const int4*>(ft_b + h + 8 * c);
            const int4 v0 = __ldg(b0), v1 = __ldg(b0 + 1), w0 = __ldg(b1), w1 = __ldg(b1 + 1);
            x[s][0][0] = v0.x, x[s][0][1] = v0.y, x[s][0][2] = v0.z, x[s][0][3] = v0.w;
            x[s][0][4] = v1.x, x[s][0][5] = v1.y, x[s][0][6] = v1.z, x[s][0][7] = v1.w;
            x[s][1][0] = w0.x, x[s][1][1] = w0.y, x[s][1][2] = w0.z, x[s][1][3] = w0.w;
            x[s][1][4] = w1.x, x[s][1][5] = w1.y, x[s][1][6] = w1.z, x[s][1][7] = w1.w;
        }
        const int32_t* list = lists[s];
        const int n = count_active(list, d.K, lane);
        n_act[s] = n;
        for (int k0 = 0; k0 < n; k0 += 32) {
            const int m = min(32, n - k0);
            int mine = (lane < m) ? list[k0 + lane] : -1;
            if (lane < m && (mine < 0 || (int64_t)mine >= d.N)) {
                if (tile == 0) note_bad_index(status);
                mine = -1;
            }
            for (int j = 0; j < m; j += kQGatherRows) {
                uint4 v[kQGatherRows][2];
                bool ok[kQGatherRows];
#pragma unroll
                for (int t = 0; t < kQGatherRows; ++t) {
                    const int r = __shfl_sync(kFullMask, mine, (j + t) & 31);
                    ok[t] = (j + t < m) && r >= 0 && live;
                    if (ok[t]) {
                        const uint4* row = reinterpret_cast<const uint4*>(ft_w + (int64_t)r * d.L1);
                        v[t][0] = __ldg(row + c);
                        v[t][1] = __ldg(row + h8 + c);
                    }
                }
#pragma unroll
                for (int t = 0; t < kQGatherRows; ++t) {
                    if (ok[t]) {
                        add8(x[s][0], v[t][0]);
                        add8(x[s][1], v[t][1]);
                    }
                }
            }
        }
    }
    if (live) {
        unsigned lo[2] = {0, 0}, hi[2] = {0, 0};  // 8 int8 each: products of "us", of "them"
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int a0 = clampi(x[0][0][j], 0, q.ft_max), a1 = clampi(x[0][1][j], 0, q.ft_max);
            const int b0 = clampi(x[1][0][j], 0, q.ft_max), b1 = clampi(x[1][1][j], 0, q.ft_max);
            const unsigned pa = (unsigned)min((a0 * a1) >> q.ft_shift, q.hidden_max) & 0xffu;
            const unsigned pb = (unsigned)min((b0 * b1) >> q.ft_shift, q.hidden_max) & 0xffu;
            lo[j >> 2] |= pa << (8 * (j & 3));
            hi[j >> 2] |= pb << (8 * (j & 3));
        }
        int8_t* row = x0 + (p - p_begin) * d.L1;
        *reinterpret_cast<uint2*>(row + 8 * c) = make_uint2(lo[0], lo[1]);
        *reinterpret_cast<uint2*>(row + h + 8 * c) = make_uint2(hi[0], hi[1]);
    }
    if (tile == 0) {  // PSQT: integer adds commute, any order gives the same sum
        int bk = bucket[p];
        if (bk < 0 || bk >= d.buckets || bk >= d.P) bk = 0;  // k_quant_layers reports it
        int diff = 0;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            int acc = 0;
            for (int k = lane; k < n_act[s]; k += 32) {
                const int r = lists[s][k];
                if (r >= 0 && (int64_t)r < d.N) acc += __ldg(ft_psqt + (int64_t)r * d.P + bk);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(kFullMask, acc, o);
            diff += s == 0 ? acc : -acc;
        }
        if (lane == 0) psq[p - p_begin] = diff;
    }
}

// The gather on the packed form of the table (nnue_quant_pack_table: neighbouring columns as ONE int32 number,
// one more row of zeros), with the training forward's loop: a warp per (position, perspective), branch-free batches
// of R rows, one 32-bit add per two columns, split into int32 sums before the low half can overflow.  Taken when
// every |ft_w| <= kMaxAbsPacked; same bits as k_quant_gather.
constexpr int kQPackedPos = kWarpsPerCta / 2;
template <int R>
__global__ void __launch_bounds__(kThreads, 4)
    k_quant_gather_packed(const int32_t* __restrict__ white_idx, const int32_t* __restrict__ black_idx,
                          const uint8_t* __restrict__ stm_white, const int32_t* __restrict__ bucket,
                          const int16_t* __restrict__ ft_w_packed, const int32_t* __restrict__ ft_psqt,
                          const int32_t* __restrict__ ft_b, int8_t* __restrict__ x0, int32_t* __restrict__ psq,
                          int64_t p_begin, int64_t p_end, QuantDims d, nnue_quant_params q, int n_groups,
                          int rows_per_split, unsigned long long* status) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int side = warp & 1, pair = warp >> 1;
    const int tile = blockIdx.x / n_groups;
    const int64_t p = p_begin + (int64_t)(blockIdx.x % n_groups) * kQPackedPos + pair;
    if (p >= p_end) return;
    const int h = d.L1 >> 1, h8 = h >> 3;
    const int c = tile * 32 + lane;
    const bool live = c < h8;
    const int stm = stm_white[p] ? 1 : 0;
    // side 0 is the side to move ("us"), side 1 the other
    const int32_t* list = ((side == 0) == (stm != 0) ? white_idx : black_idx) + p * d.K;
    const int n = count_active(list, d.K, lane);

    PairAcc acc;
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
        const int4* b = reinterpret_cast<const int4*>(ft_b + hlf * h + 8 * (live ? c : 0));
        const int4 v0 = __ldg(b), v1 = __ldg(b + 1);
        acc.lo[hlf][0] = v0.x, acc.hi[hlf][0] = v0.y, acc.lo[hlf][1] = v0.z, acc.hi[hlf][1] = v0.w;
        acc.lo[hlf][2] = v1.x, acc.hi[hlf][2] = v1.y, acc.lo[hlf][3] = v1.z, acc.hi[hlf][3] = v1.w;
    }
    // lanes beyond the last column read column group 0 (valid memory); their sums are never stored
    const uint4* base0 = reinterpret_cast<const uint4*>(ft_w_packed) + (live ? c : 0);
    gather_q16<R>(base0, base0 + h8, d.L1 >> 3, (int)d.N, list, n, rows_per_split, acc, lane, status);
    if (live) {
        unsigned w[2] = {0, 0};  // 8 int8: the clipped products of this perspective
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int a0 = clampi((j & 1) ? acc.hi[0][j >> 1] : acc.lo[0][j >> 1], 0, q.ft_max);
            const int a1 = clampi((j & 1) ? acc.hi[1][j >> 1] : acc.lo[1][j >> 1], 0, q.ft_max);
            w[j >> 2] |= ((unsigned)min((a0 * a1) >> q.ft_shift, q.hidden_max) & 0xffu) << (8 * (j & 3));
        }
        *reinterpret_cast<uint2*>(x0 + (p - p_begin) * d.L1 + side * h + 8 * c) = make_uint2(w[0], w[1]);
    }
    if (tile == 0) {  // PSQT of this perspective; the two warps of a position add their halves of the difference
        int bk = bucket[p];
        if (bk < 0 || bk >= d.buckets || bk >= d.P) bk = 0;  // k_quant_layers reports it
        int s = 0;
        for (int k = lane; k < n; k += 32) {
            const int r = list[k];
            if (r >= 0 && (int64_t)r < d.N) s += __ldg(ft_psqt + (int64_t)r * d.P + bk);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(kFullMask, s, o);
        if (lane == 0) atomicAdd(psq + (p - p_begin), side == 0 ? s : -s);  // integer: the order does not matter
    }
}

// int16 [N, L1] -> the packed form: [N + 1, L1] int16 read as int32 numbers k[c + 1] * 65536 + k[c], last row zeros.
__global__ void __launch_bounds__(kThreads)
    k_quant_pack_table(const int16_t* __restrict__ ft_w, int32_t* __restrict__ packed, int64_t n_words, int64_t n_src_words,
                       int32_t* __restrict__ max_abs) {
    int m = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += stride) {
        int word = 0;
        if (i < n_src_words) {
            const int k0 = ft_w[2 * i], k1 = ft_w[2 * i + 1];
            word = k1 * 65536 + k0;
            m = max(m, max(abs(k0), abs(k1)));
        }
        packed[i] = word;
    }
    m = __reduce_max_sync(kFullMask, m);
    if ((threadIdx.x & 31) == 0 && m > 0) atomicMax(max_abs, m);
}

constexpr int kQLayerThreads = 128;
__global__ void __launch_bounds__(kQLayerThreads)
    k_quant_layers(const int8_t* __restrict__ x0, const int32_t* __restrict__ psq,
                   const int32_t* __restrict__ bucket, const int8_t* __restrict__ l1_w,
                   const int32_t* __restrict__ l1_b, const int8_t* __restrict__ l2_w,
                   const int32_t* __restrict__ l2_b, const int8_t* __restrict__ out_w,
                   const int32_t* __restrict__ out_b, int32_t* __restrict__ out, int64_t p_begin, int64_t p_end,
                   QuantDims d, nnue_quant_params q, unsigned long long* status) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    int8_t* s_x0 = reinterpret_cast<int8_t*>(s_raw);           // [L1]
    int32_t* s_o1 = reinterpret_cast<int32_t*>(s_raw + d.L1);  // [L2]
    int8_t* s_x1 = reinterpret_cast<int8_t*>(s_o1 + kQMaxL2);  // [2*L2 + 2*L3]
    const int tid = threadIdx.x;
    for (int64_t p = p_begin + blockIdx.x; p < p_end; p += gridDim.x) {
        int bk = bucket[p];
        if (bk < 0 || bk >= d.buckets || bk >= d.P) {
            if (tid == 0) note_bad_index(status);
            bk = 0;
        }
        const int4* src = reinterpret_cast<const int4*>(x0 + (p - p_begin) * d.L1);
        for (int i = tid; i < (d.L1 >> 4); i += kQLayerThreads) reinterpret_cast<int4*>(s_x0)[i] = __ldcs(src + i);
        __syncthreads();
        quant_layers(s_x0, s_o1, s_x1, bk, d, q, l1_w, l1_b, l2_w, l2_b, out_w, out_b, (long long)psq[p - p_begin],
                     out + p);
        __syncthreads();
    }
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_quant_eval(const int32_t* white_idx, const int32_t* black_idx,
                               const uint8_t* stm_white, const int32_t* bucket, const int16_t* ft_w,
                               const int32_t* ft_psqt, const int32_t* ft_b, const int8_t* l1_w,
                               const int32_t* l1_b, const int8_t* l2_w, const int32_t* l2_b,
                               const int8_t* out_w, const int32_t* out_b, int32_t* out, int64_t B,
                               int32_t K, int64_t N, int32_t L1, int32_t L2, int32_t L3, int32_t P,
                               int32_t buckets, const nnue_quant_params* qp, void* stream) {
    NNUE_REQUIRE(qp != nullptr, NNUE_ERR_ARG, "nnue_quant_eval: null quantization parameters");
    NNUE_REQUIRE(B >= 0 && K >= 0 && N >= 0 && L1 > 0 && L2 > 1 && L3 > 0 && P > 0 && buckets > 0,
                 NNUE_ERR_ARG, "nnue_quant_eval: bad size");
    if (B == 0) return NNUE_OK;
    NNUE_REQUIRE(white_idx && black_idx && stm_white && bucket && ft_w && ft_psqt && ft_b && l1_w &&
                     l1_b && l2_w && l2_b && out_w && out_b && out,
                 NNUE_ERR_ARG, "nnue_quant_eval: null pointer");
    NNUE_REQUIRE(L1 % 32 == 0, NNUE_ERR_UNSUPPORTED,
                 "nnue_quant_eval: L1 must be a multiple of 32 (16-byte int16 chunks per half), got %d", L1);
    NNUE_REQUIRE(L2 <= kQMaxL2 && L3 <= kQMaxL2, NNUE_ERR_UNSUPPORTED,
                 "nnue_quant_eval: hidden layers wider than %d are not covered", kQMaxL2);
    NNUE_REQUIRE(aligned16(ft_w) && aligned16(l1_w), NNUE_ERR_ALIGN,
                 "nnue_quant_eval: ft_w / l1_w must be 16-byte aligned");
    NNUE_REQUIRE(qp->out_div > 0 && qp->ft_shift >= 0 && qp->sqr_shift_l1 >= 0 && qp->sqr_shift_l2 >= 0,
                 NNUE_ERR_ARG, "nnue_quant_eval: bad quantization parameters");
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "nnue_quant_eval: no device status word");
    QuantDims d{K, L1, L2, L3, P, buckets, N};
    const size_t smem = (size_t)L1 + kQMaxL2 * sizeof(int32_t) + 4 * kQMaxL2 + 16;
    NNUE_REQUIRE(smem <= 48 * 1024, NNUE_ERR_UNSUPPORTED, "nnue_quant_eval: L1 too large");
    const unsigned grid = (unsigned)std::min<int64_t>(B, (int64_t)sm_count() * 10);
    k_quant_eval<<<grid, kQThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        white_idx, black_idx, stm_white, bucket, ft_w, ft_psqt, ft_b, l1_w, l1_b, l2_w, l2_b, out_w,
        out_b, out, B, d, *qp, status);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

extern "C" size_t nnue_quant_eval_workspace_bytes(int64_t B, int32_t L1) {
    if (B <= 0 || L1 <= 0) return 0;
    const int64_t chunk = std::min<int64_t>(B, 131072);  // positions per pass
    return (size_t)chunk * ((size_t)L1 + sizeof(int32_t)) + 256;
}

extern "C" int nnue_quant_pack_table(const int16_t* ft_w, int16_t* packed, int32_t* d_max_abs, int64_t N, int32_t L1,
                                     void* stream) {
    NNUE_REQUIRE(N >= 0 && L1 > 0 && L1 % 2 == 0, NNUE_ERR_ARG, "nnue_quant_pack_table: bad size (L1 must be even)");
    NNUE_REQUIRE(ft_w && packed && d_max_abs && (reinterpret_cast<uintptr_t>(packed) & 3u) == 0, NNUE_ERR_ARG,
                 "nnue_quant_pack_table: null or unaligned pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    NNUE_CUDA_TRY(cudaMemsetAsync(d_max_abs, 0, sizeof(int32_t), s));
    const int64_t src = N * (L1 / 2), all = (N + 1) * (L1 / 2);
    const unsigned grid = (unsigned)std::min<int64_t>((all + kThreads - 1) / kThreads, (int64_t)sm_count() * 8);
    k_quant_pack_table<<<grid, kThreads, 0, s>>>(ft_w, reinterpret_cast<int32_t*>(packed), all, src, d_max_abs);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

static int quant_eval_tiled_impl(const int32_t* white_idx, const int32_t* black_idx,
                                     const uint8_t* stm_white, const int32_t* bucket, const int16_t* ft_w,
                                     const int16_t* ft_w_packed, int32_t max_abs,
                                     const int32_t* ft_psqt, const int32_t* ft_b, const int8_t* l1_w,
                                     const int32_t* l1_b, const int8_t* l2_w, const int32_t* l2_b,
                                     const int8_t* out_w, const int32_t* out_b, int32_t* out, int64_t B,
                                     int32_t K, int64_t N, int32_t L1, int32_t L2, int32_t L3, int32_t P,
                                     int32_t buckets, const nnue_quant_params* qp, void* workspace,
                                     size_t workspace_bytes, void* stream) {
    NNUE_REQUIRE(qp != nullptr, NNUE_ERR_ARG, "nnue_quant_eval_tiled: null quantization parameters");
    NNUE_REQUIRE(B >= 0 && K >= 0 && N >= 0 && L1 > 0 && L2 > 1 && L3 > 0 && P > 0 && buckets > 0,
                 NNUE_ERR_ARG, "nnue_quant_eval_tiled: bad size");
    if (B == 0) return NNUE_OK;
    NNUE_REQUIRE(white_idx && black_idx && stm_white && bucket && (ft_w || ft_w_packed) && ft_psqt && ft_b && l1_w &&
                     l1_b && l2_w && l2_b && out_w && out_b && out,
                 NNUE_ERR_ARG, "nnue_quant_eval_tiled: null pointer");
    if (ft_w_packed) {
        NNUE_REQUIRE(max_abs >= 0 && max_abs <= kMaxAbsPacked, NNUE_ERR_UNSUPPORTED,
                     "nnue_quant_eval_packed: the packed gather takes |ft_w| <= %d (got %d)", kMaxAbsPacked, max_abs);
        NNUE_REQUIRE(K <= 511 && (N + 1) * (int64_t)(L1 / 8) < 0x7fffffffLL && aligned16(ft_w_packed), NNUE_ERR_UNSUPPORTED,
                     "nnue_quant_eval_packed: at most 511 rows per list, 32-bit row offsets, 16-byte aligned table");
    }
    NNUE_REQUIRE(L1 % 32 == 0, NNUE_ERR_UNSUPPORTED,
                 "nnue_quant_eval_tiled: L1 must be a multiple of 32 (16-byte int16 chunks per half), got %d", L1);
    NNUE_REQUIRE(L2 <= kQMaxL2 && L3 <= kQMaxL2, NNUE_ERR_UNSUPPORTED,
                 "nnue_quant_eval_tiled: hidden layers wider than %d are not covered", kQMaxL2);
    NNUE_REQUIRE((ft_w_packed || aligned16(ft_w)) && aligned16(l1_w) && aligned16(ft_b), NNUE_ERR_ALIGN,
                 "nnue_quant_eval_tiled: ft_w / ft_b / l1_w must be 16-byte aligned");
    NNUE_REQUIRE(qp->out_div > 0 && qp->ft_shift >= 0 && qp->sqr_shift_l1 >= 0 && qp->sqr_shift_l2 >= 0,
                 NNUE_ERR_ARG, "nnue_quant_eval_tiled: bad quantization parameters");
    char* ws = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t)255);
    const size_t usable = workspace ? workspace_bytes - (size_t)(ws - static_cast<char*>(workspace)) : 0;
    const size_t per_pos = (size_t)L1 + sizeof(int32_t);
    NNUE_REQUIRE(workspace && workspace_bytes >= 256 + per_pos && usable >= per_pos, NNUE_ERR_WORKSPACE,
                 "nnue_quant_eval_tiled: workspace too small (see nnue_quant_eval_workspace_bytes)");
    // positions per pass: what the workspace holds, rounded down to whole groups of 16 (keeps x0 rows and the
    // psq array 16-byte aligned)
    int64_t chunk = (int64_t)(usable / per_pos);
    if (chunk >= 16) chunk &= ~(int64_t)15;
    chunk = std::min<int64_t>(chunk, B);
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "nnue_quant_eval_tiled: no device status word");
    QuantDims d{K, L1, L2, L3, P, buckets, N};
    const size_t smem = (size_t)L1 + kQMaxL2 * sizeof(int32_t) + 4 * kQMaxL2 + 16;
    NNUE_REQUIRE(smem <= 48 * 1024, NNUE_ERR_UNSUPPORTED, "nnue_quant_eval_tiled: L1 too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int h8 = L1 / 16;
    const int tiles = (h8 + 31) / 32;
    for (int64_t p0 = 0; p0 < B; p0 += chunk) {
        const int64_t p1 = std::min(B, p0 + chunk);
        int8_t* x0 = reinterpret_cast<int8_t*>(ws);
        int32_t* psq = reinterpret_cast<int32_t*>(ws + (size_t)chunk * L1);
        const int64_t groups = (p1 - p0 + kWarpsPerCta - 1) / kWarpsPerCta;
        NNUE_REQUIRE(groups * tiles <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "nnue_quant_eval_tiled: grid too large");
        if (ft_w_packed) {
            const int64_t groups4 = (p1 - p0 + kQPackedPos - 1) / kQPackedPos;
            NNUE_REQUIRE(groups4 * tiles <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "nnue_quant_eval_packed: grid too large");
            NNUE_CUDA_TRY(cudaMemsetAsync(psq, 0, (size_t)(p1 - p0) * sizeof(int32_t), s));  // the two perspectives add into it
            const int rows_per_split = max_abs > 0 ? std::min(32767 / max_abs, 512) : 512;
            ProfScope prof("k_quant_gather_packed", s);
            k_quant_gather_packed<3><<<(unsigned)(groups4 * tiles), kThreads, 0, s>>>(
                white_idx, black_idx, stm_white, bucket, ft_w_packed, ft_psqt, ft_b, x0, psq, p0, p1, d, *qp, (int)groups4,
                rows_per_split, status);
        } else {
            ProfScope prof("k_quant_gather", s);
            k_quant_gather<<<(unsigned)(groups * tiles), kThreads, 0, s>>>(white_idx, black_idx, stm_white, bucket,
                                                                          ft_w, ft_psqt, ft_b, x0, psq, p0, p1, d,
                                                                          *qp, (int)groups, status);
        }
        const unsigned grid = (unsigned)std::min<int64_t>(p1 - p0, (int64_t)sm_count() * 16);
        ProfScope prof("k_quant_layers", s);
        k_quant_layers<<<grid, kQLayerThreads, smem, s>>>(x0, psq, bucket, l1_w, l1_b, l2_w, l2_b, out_w, out_b, out,
                                                         p0, p1, d, *qp, status);
        NNUE_CUDA_TRY(cudaGetLastError());
        note_launches(2);
    }
    return NNUE_OK;
}

extern "C" int nnue_quant_eval_tiled(const int32_t* white_idx, const int32_t* black_idx,
                                     const uint8_t* stm_white, const int32_t* bucket, const int16_t* ft_w,
                                     const int32_t* ft_psqt, const int32_t* ft_b, const int8_t* l1_w,
                                     const int32_t* l1_b, const int8_t* l2_w, const int32_t* l2_b,
                                     const int8_t* out_w, const int32_t* out_b, int32_t* out, int64_t B,
                                     int32_t K, int64_t N, int32_t L1, int32_t L2, int32_t L3, int32_t P,
                                     int32_t buckets, const nnue_quant_params* qp, void* workspace,
                                     size_t workspace_bytes, void* stream) {
    return quant_eval_tiled_impl(white_idx, black_idx, stm_white, bucket, ft_w, nullptr, 0, ft_psqt, ft_b, l1_w, l1_b, l2_w,
                                 l2_b, out_w, out_b, out, B, K, N, L1, L2, L3, P, buckets, qp, workspace, workspace_bytes,
                                 stream);
}

extern "C" int nnue_quant_eval_packed(const int32_t* white_idx, const int32_t* black_idx,
                                      const uint8_t* stm_white, const int32_t* bucket, const int16_t* ft_w_packed,
                                      int32_t max_abs, const int32_t* ft_psqt, const int32_t* ft_b, const int8_t* l1_w,
                                      const int32_t* l1_b, const int8_t* l2_w, const int32_t* l2_b,
                                      const int8_t* out_w, const int32_t* out_b, int32_t* out, int64_t B,
                                      int32_t K, int64_t N, int32_t L1, int32_t L2, int32_t L3, int32_t P,
                                      int32_t buckets, const nnue_quant_params* qp, void* workspace,
                                      size_t workspace_bytes, void* stream) {
    NNUE_REQUIRE(ft_w_packed != nullptr, NNUE_ERR_ARG, "nnue_quant_eval_packed: null table");
    return quant_eval_tiled_impl(white_idx, black_idx, stm_white, bucket, nullptr, ft_w_packed, max_abs, ft_psqt, ft_b, l1_w,
                                 l1_b, l2_w, l2_b, out_w, out_b, out, B, K, N, L1, L2, L3, P, buckets, qp, workspace,
                                 workspace_bytes, stream);
}
