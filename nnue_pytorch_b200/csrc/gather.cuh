// Warp-level gather-sum of table rows: the one access pattern shared by the
// sparse-linear forward, the fused double-FT forward and the segment-reduce
// backward.  A warp owns C float4 column slots per lane (C*32 float4 = C*512
// bytes of each row, every load a fully coalesced 512-byte warp request) and
// adds the listed rows in list order, R rows (C*R independent 16-byte loads
// per lane) in flight at a time.
#pragma once

#include "common.cuh"

namespace nnue {

// list : n row ids (shared or global memory); every id must be >= 0.
// rows >= n_rows are skipped and counted in `status`.
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

}  // namespace nnue
