// Warp-level gather-sum of table rows: the one access pattern shared by the
// sparse-linear forward, the fused double-FT forward and the segment-reduce
// backward.  A warp owns C float4 column slots per lane (C*32 float4 = C*512
// bytes of each row, every load a fully coalesced 512-byte warp request) and
// adds the listed rows in list order.
//
// Two forms, chosen by measurement on B200:
//   gather_sum            R rows (C*R independent 16-byte loads per lane) are
//                         loaded, then added; fewest instructions per load.
//                         Fastest for the forward kernels, which run at
//                         4 CTAs per SM and are close to the L2 fabric limit.
//   gather_sum_pipelined  two register buffers of R rows; the loads of batch
//                         b+1 are issued before the adds of batch b and the ids
//                         of the next 32 entries are fetched early.  Fastest
//                         for the segment reduction, whose per-entry hook
//                         (row boundaries) lengthens the add phase.
#pragma once

#include "common.cuh"

namespace nnue {

// list : n row ids (shared or global memory).  Ids outside [0, n_rows) are
// skipped and tallied in `status`.
template <int C, int R>
__device__ __forceinline__ void gather_sum(const float4* __restrict__ table, int64_t stride4,
                                           int64_t n_rows, const int32_t* list, int n,
                                           const int (&col)[C], const bool (&ok)[C],
                                           float4 (&acc)[C], int lane,
                                           unsigned long long* status) {
    for (int k0 = 0; k0 < n; k0 += 32) {
        const int m = min(32, n - k0);
        int mine = (lane < m) ? list[k0 + lane] : 0;
        if ((unsigned)mine >= (unsigned long long)n_rows) {  // negative or too large
            if (lane < m) note_bad_index(status);
            mine = -1;
        }
        for (int j = 0; j < m; j += R) {
            float4 v[R][C];
            int r[R];
#pragma unroll
            for (int t = 0; t < R; ++t) {
                // lanes >= m hold 0/-1; the (j + t < m) test keeps them out
                r[t] = __shfl_sync(kFullMask, mine, (j + t) & 31);
                const bool live = (j + t < m) && (r[t] >= 0);
                const float4* row = table + (int64_t)(live ? r[t] : 0) * stride4;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    v[t][c] = (live && ok[c]) ? ldg4(row + col[c]) : f4_zero();
                }
                r[t] = live ? 1 : 0;
            }
#pragma unroll
            for (int t = 0; t < R; ++t) {
                if (r[t]) {
#pragma unroll
                    for (int c = 0; c < C; ++c) acc[c] = f4_add(acc[c], v[t][c]);
                }
            }
        }
    }
}

// pre(i) runs before entry i (0-based position in `list`) is added, in order;
// the segment kernel uses it to close a row when i crosses a row boundary.
// Bad ids are tallied only when `count_bad`.
// The loads carry no predicate: a slot past the end of the list, a bad id or a lane beyond the
// last column reads row 0 / column 0 (valid memory) and the value is dropped, by the warp-uniform
// test around the add or by the caller's masked store.
template <int C, int R, class Pre>
__device__ __forceinline__ void gather_sum_pipelined(const float4* __restrict__ table,
                                                     int64_t stride4, int64_t n_rows,
                                                     const int32_t* list, int n,
                                                     const int (&col)[C], const bool (&ok)[C],
                                                     float4 (&acc)[C], int lane,
                                                     unsigned long long* status, bool count_bad,
                                                     Pre pre) {
    const float4* base[C];
#pragma unroll
    for (int c = 0; c < C; ++c) base[c] = table + (ok[c] ? col[c] : 0);
    int next_mine = (lane < min(32, n)) ? list[lane] : 0;
    for (int k0 = 0; k0 < n; k0 += 32) {
        const int m = min(32, n - k0);
        int mine = next_mine;
        if (k0 + 32 < n) next_mine = (lane < min(32, n - k0 - 32)) ? list[k0 + 32 + lane] : 0;
        if ((unsigned)mine >= (unsigned long long)n_rows) {
            if (lane < m && count_bad) note_bad_index(status);
            mine = -1;
        }
        const int nb = (m + R - 1) / R;
        float4 va[R][C], vb[R][C];
        int ra[R], rb[R];

        auto issue = [&](float4 (&v)[R][C], int (&rr)[R], int b) {
#pragma unroll
            for (int t = 0; t < R; ++t) {
                rr[t] = __shfl_sync(kFullMask, mine, (b * R + t) & 31);  // lanes >= m hold 0: row 0
                const int64_t off = (int64_t)max(rr[t], 0) * stride4;
#pragma unroll
                for (int c = 0; c < C; ++c) v[t][c] = ldg4(base[c] + off);
            }
        };
        auto consume = [&](float4 (&v)[R][C], int (&rr)[R], int b) {
#pragma unroll
            for (int t = 0; t < R; ++t) {
                const int j = b * R + t;
                if (j < m) {  // warp-uniform
                    pre(k0 + j);
                    if (rr[t] >= 0) {
#pragma unroll
                        for (int c = 0; c < C; ++c) acc[c] = f4_add(acc[c], v[t][c]);
                    }
                }
            }
        };

        issue(va, ra, 0);
        for (int b = 0; b < nb; b += 2) {
            if (b + 1 < nb) issue(vb, rb, b + 1);
            consume(va, ra, b);
            if (b + 2 < nb) issue(va, ra, b + 2);
            if (b + 1 < nb) consume(vb, rb, b + 1);
        }
    }
}

}  // namespace nnue
