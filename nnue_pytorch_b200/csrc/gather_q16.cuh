// Gather-sum over an int16 table stored as packed column pairs: shared by the training forward
// (ft_fused_q16.cu) and the integer evaluation (quant_eval.cu).
#pragma once

#include "common.cuh"

namespace nnue {

// Packed sums.  The table stores every pair of neighbouring columns (c, c + 1) as ONE int32,
// k[c + 1] * 65536 + k[c] (a number, not two independent halves: a negative low value borrows from
// the high half), so a plain 32-bit add sums both columns at once.  The low part of such a sum can
// be told from the high part as long as it stays within int16, i.e. for at most
// G = 32767 / max|k| rows; the emitting kernel records max|k| of the table, and after every G
// rows the pair sum is split into two int32 accumulators.  Trained weights are a few units at
// most (|k| in the hundreds), so G is 32 or more and the split is rare: one add per two values.
struct PairAcc {
    int lo[2][4], hi[2][4];   // per half: four column pairs
};

__device__ __forceinline__ void split_pairs(int (&pk)[2][4], PairAcc& acc) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int lo = (int)(short)pk[h][w];
            acc.lo[h][w] += lo;
            acc.hi[h][w] += (pk[h][w] - lo) >> 16;
            pk[h][w] = 0;
        }
    }
}

// acc += sum over the listed rows of this lane's column pairs in both halves.
// The loop carries no predicates: the table has one more row than the feature set, all zeros
// (row `zero_row`), and list entries that are padding, out of range or beyond the end of the list
// read that row, so every batch of R rows is complete and is loaded and added unconditionally.
// base0 / base1 point at this lane's 16-byte group in the first / second half of row 0.
template <int R>
__device__ __forceinline__ void gather_q16(const uint4* __restrict__ base0, const uint4* __restrict__ base1,
                                           int stride8, int zero_row, const int32_t* list, int n,
                                           int rows_per_split, PairAcc& acc, int lane, unsigned long long* status) {
    constexpr int kChunk = (32 / R) * R;  // list entries per pass: a multiple of R, so a batch never wraps the warp
    int pk[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    int pending = 0;
    for (int k0 = 0; k0 < n; k0 += kChunk) {
        const int m = min(kChunk, n - k0);
        int mine = (lane < m) ? list[k0 + lane] : zero_row;
        if ((unsigned)mine >= (unsigned)zero_row) {  // negative or too large (padding lanes hold zero_row itself)
            if (lane < m) note_bad_index(status);
            mine = zero_row;
        }
        for (int j = 0; j < m; j += R) {
            uint4 v[R][2];
#pragma unroll
            for (int t = 0; t < R; ++t) {
                const int off = __shfl_sync(kFullMask, mine, j + t) * stride8;
                v[t][0] = __ldg(base0 + off);
                v[t][1] = __ldg(base1 + off);
            }
#pragma unroll
            for (int t = 0; t < R; ++t) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    pk[h][0] += (int)v[t][h].x;
                    pk[h][1] += (int)v[t][h].y;
                    pk[h][2] += (int)v[t][h].z;
                    pk[h][3] += (int)v[t][h].w;
                }
            }
            pending += R;
            if (pending + R > rows_per_split) {
                split_pairs(pk, acc);
                pending = 0;
            }
        }
    }
    if (pending) split_pairs(pk, acc);
}

// Largest |k| the packed sums take: 32767 / 4095 = 8 rows per split, above the deepest batch (R <= 6).
constexpr int kMaxAbsPacked = 4095;

}  // namespace nnue
