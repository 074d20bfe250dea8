// Host-side interface of the CSR-by-row builder and the segment gather-sum
// that turn a scatter-add into "every gradient row written exactly once".
#pragma once

#include "common.cuh"

namespace nnue {

// Scratch for a CSR over at most `max_entries` (position, slot) pairs and
// `n_rows` table rows of width W: counts, offsets, ranks, entry ids, chunk
// table and the partial sums of rows that cross a chunk border.
size_t csr_workspace_bytes(int64_t max_entries, int64_t n_rows, int W);

// out[c] = sum over rows of src[row, c], rows added in ascending order inside
// fixed slices (bitwise reproducible).  `scratch` (may be NULL when
// rows <= kColumnSumDirectRows) holds kColumnSumSlices * W floats.
constexpr int kColumnSumDirectRows = 2048;
constexpr int kColumnSumSlices = 64;
int column_sum(const float* src, int64_t rows, int W, float* out, cudaStream_t s,
               float* scratch = nullptr);

// Pointers into the caller's workspace.
struct CsrPlan {
    int n_lists = 0, K = 0, S = 0;
    int64_t B = 0, N = 0, max_chunks = 0;
    int32_t *counts = nullptr, *n_long = nullptr, *long_list = nullptr, *offsets = nullptr;
    int32_t *ranks = nullptr, *entries = nullptr, *chunk_row = nullptr;
    float* partial = nullptr;
};
struct CsrJoin {
    bool pending = false;
    cudaEvent_t event = nullptr;
};

int csr_plan(CsrPlan& plan, int n_lists, int64_t B, int K, int64_t N, int W, void* ws,
             size_t ws_bytes);

// lists[l] is an int32 [B, K] index tensor; the entry id of (p, l, k) is
// p * n_lists + l, which is the row of the [B * n_lists, W] source that the
// entry contributes.  Builds offsets / ordered entries / the chunk table.
int csr_build(const CsrPlan& plan, const int32_t* const* lists, cudaStream_t s);

// Same, on the library's helper stream so it overlaps with what the caller
// enqueues on `s` next; csr_join() makes `s` wait for it.
int csr_build_overlapped(const CsrPlan& plan, const int32_t* const* lists, cudaStream_t s,
                         CsrJoin& join);
int csr_join(CsrJoin& join, cudaStream_t s);

// The library's per-device helper stream with its fork / join events, for work that may run
// beside the caller's stream: record `fork` on the caller's stream, make `stream` wait for it,
// enqueue, record `join` on `stream`, make the caller's stream wait for `join`.
struct SideStreamView {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
bool side_stream_get(SideStreamView& out);

// out[r, :] = sum of the source rows named by the entries of r, for every r < N.
// Rows [row_begin, row_end) only (row_end < 0: to the last row); the chunked
// vector path supports any range, the fallbacks only the whole table.
// Columns [col_begin, col_end) only (floats; col_end < 0: to the last column): the chunked vector path, bounds on
// whole column tiles (csr_column_tile).
int csr_reduce(const CsrPlan& plan, const float* src, int W, float* out, cudaStream_t s, int64_t row_begin = 0,
               int64_t row_end = -1, int64_t col_begin = 0, int64_t col_end = -1);
// Floats per column tile of the chunked vector path for rows of W floats (0: W is not a multiple of 4).
int csr_column_tile(int W);

}  // namespace nnue
