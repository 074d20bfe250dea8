// Host-side interface of the CSR-by-row builder and the segment gather-sum
// that turn a scatter-add into "every gradient row written exactly once".
#pragma once

#include "common.cuh"

namespace nnue {

// Scratch for a CSR over at most `max_entries` (position, slot) pairs and
// `n_rows` table rows: counts, offsets, cursors, entry ids.
size_t csr_workspace_bytes(int64_t max_entries, int64_t n_rows);

// out[c] = sum over rows of src[row, c], rows added in ascending order inside
// fixed slices (bitwise reproducible).  `scratch` (may be NULL when
// rows <= kColumnSumDirectRows) holds kColumnSumSlices * W floats.
constexpr int kColumnSumDirectRows = 2048;
constexpr int kColumnSumSlices = 64;
int column_sum(const float* src, int64_t rows, int W, float* out, cudaStream_t s,
               float* scratch = nullptr);

// lists[l] is an int32 [B, K] index tensor; entry id of (p, l, k) is
// p * n_lists + l, which is the row of `src` ([B * n_lists, W]) that the
// entry contributes.  Writes out[r, :] = sum of those rows for every r < N.
int csr_build_and_reduce(const int32_t* const* lists, int n_lists, int64_t B, int K, int64_t N,
                         const float* src, int W, float* out, void* ws, size_t ws_bytes,
                         cudaStream_t s);

}  // namespace nnue
