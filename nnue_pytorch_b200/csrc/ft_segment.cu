// CSR-by-row construction for one batch of index lists and the segment
// gather-sum that replaces the reference's scalar atomicAdd scatter
// (sparse_linear_kernel.py:237-288, fused_ft_kernel.py:222-251 in the
// reference project).  Every row of the output gradient is written exactly
// once with plain stores, rows nobody touched get zeros, so the caller's
// dense torch.zeros pass disappears and the result is reproducible.
#include "gather.cuh"
#include "segment.cuh"

#include <algorithm>

namespace nnue {

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static int64_t max_chunks_for(int64_t max_entries, int S) { return (max_entries + S - 1) / S + 1; }

size_t csr_workspace_bytes(int64_t max_entries, int64_t n_rows, int W) {
    size_t b = 0;
    const int S = tuning().seg_chunk;
    if (S > 0) {
        const int64_t mc = max_chunks_for(max_entries, S);
        b += align_up((size_t)mc * sizeof(int32_t), 256);               // chunk -> first row
        b += align_up((size_t)mc * 2 * (size_t)W * sizeof(float), 256);  // partial sums
    }
    b += align_up((size_t)(n_rows + 1) * sizeof(int32_t), 256);  // counts + long-row counter
    b += align_up((size_t)n_rows * sizeof(int32_t), 256);        // long-row list
    b += align_up((size_t)(n_rows + 1) * sizeof(int32_t), 256);  // offsets
    b += 2 * align_up((size_t)(max_entries > 0 ? max_entries : 1) * sizeof(int32_t), 256);  // ranks, entries
    return b + 256;
}

// ---- pass 1 / pass 3: one warp per (position, list) ----------------------
template <bool FILL>
__global__ void __launch_bounds__(kThreads)
    k_csr_scan_lists(const int32_t* __restrict__ list0, const int32_t* __restrict__ list1,
                     int n_lists, int64_t B, int K, int64_t N, int32_t* __restrict__ counts_or_cursor,
                     int32_t* __restrict__ ranks, int32_t* __restrict__ entries,
                     unsigned long long* status) {
    const int lane = threadIdx.x & 31;
    const int64_t wid = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (wid >= B * n_lists) return;
    const int64_t p = wid / n_lists;
    const int l = (int)(wid % n_lists);
    const int32_t* list = (l ? list1 : list0) + p * K;
    const int32_t e = (int32_t)wid;  // = p * n_lists + l
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int k = k0 + lane;
        const int r = (k < K) ? __ldg(list + k) : -1;
        const unsigned neg = __ballot_sync(kFullMask, r < 0);
        const int m = neg ? (__ffs(neg) - 1) : 32;
        if (lane < m) {
            if ((int64_t)r < N) {
                // count pass: the value the atomic returns is this entry's slot
                // inside its row; the fill pass needs no atomics
                if (FILL) entries[counts_or_cursor[r] + ranks[wid * K + k]] = e;
                else ranks[wid * K + k] = atomicAdd(counts_or_cursor + r, 1);
            } else if (!FILL) {
                note_bad_index(status);
            }
        }
        if (neg) break;
    }
}

// ---- pass 2: exclusive scan of the counts (single CTA, chunked) ----------
__global__ void __launch_bounds__(1024)
    k_csr_scan(const int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
               int32_t* __restrict__ cursor, int64_t N, int32_t* __restrict__ long_list,
               int32_t* __restrict__ n_long, int long_thresh) {
    __shared__ int s_warp[32];
    __shared__ int s_carry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_carry = 0;
    __syncthreads();
    constexpr int ITEMS = 4;
    for (int64_t base = 0; base < N; base += 1024 * ITEMS) {
        const int64_t i0 = base + (int64_t)tid * ITEMS;
        int v[ITEMS];
        int local = 0;
#pragma unroll
        for (int j = 0; j < ITEMS; ++j) {
            v[j] = (i0 + j < N) ? counts[i0 + j] : 0;
            local += v[j];
        }
        int incl = local;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(kFullMask, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = s_warp[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(kFullMask, w, d);
                if (lane >= d) w += t;
            }
            s_warp[lane] = w;  // inclusive over warps
        }
        __syncthreads();
        const int carry = s_carry;
        int run = carry + (warp ? s_warp[warp - 1] : 0) + (incl - local);
#pragma unroll
        for (int j = 0; j < ITEMS; ++j) {
            if (i0 + j < N) {
                offsets[i0 + j] = run;
                cursor[i0 + j] = run;
                if (v[j] > long_thresh) long_list[atomicAdd(n_long, 1)] = (int32_t)(i0 + j);
            }
            run += v[j];
        }
        __syncthreads();
        if (tid == 1023) s_carry = carry + s_warp[31];
        __syncthreads();
    }
    if (tid == 0) offsets[N] = s_carry;
}

// ---- pass 4: put every segment in ascending entry order -------------------
// The fill pass hands out slots with atomics, so the order inside a segment
// depends on scheduling.  Ordering the segments makes the summation order,
// and with it every bit of the gradient, independent of scheduling.
//   len <= 32           : bitonic network in registers (one warp per row)
//   len <= kWarpSortMax : bitonic network in this warp's shared-memory slab
//   longer              : listed by the scan pass; a CTA per row marks the
//                         entry ids in a shared-memory bitmap over the key
//                         space [0, B * n_lists) and reads them back in order
//                         (ids are unique unless a position names the same
//                         feature twice; such rows take a bitonic network if
//                         they have at most kCtaBitonicMax entries, else they
//                         stay as filled and status word 2 counts them).
constexpr int kWarpSortMax = 128;
constexpr int kCtaBitonicMax = 4096;
constexpr int64_t kBitmapMaxBits = 1 << 20;  // 128 KiB of shared memory

__device__ __forceinline__ void bitonic_smem(int32_t* a, int m, int tid, int nthreads, bool cta) {
    for (int k = 2; k <= m; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < m; i += nthreads) {
                const int q = i ^ j;
                if (q > i) {
                    const int x = a[i], y = a[q];
                    const bool up = (i & k) == 0;
                    if ((x > y) == up) {
                        a[i] = y;
                        a[q] = x;
                    }
                }
            }
            if (cta) __syncthreads(); else __syncwarp();
        }
    }
}

__global__ void __launch_bounds__(kThreads)
    k_csr_sort_short(const int32_t* __restrict__ offsets, int32_t* __restrict__ entries, int64_t N) {
    __shared__ int32_t s_sort[kWarpsPerCta][kWarpSortMax];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + warp;
    if (row >= N) return;
    const int beg = offsets[row], len = offsets[row + 1] - beg;
    if (len > 1 && len <= 32) {
        int key = lane < len ? entries[beg + lane] : 0x7fffffff;
#pragma unroll
        for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
            for (int j = k >> 1; j > 0; j >>= 1) {
                const int other = __shfl_xor_sync(kFullMask, key, j);
                const bool up = (lane & k) == 0, low = (lane & j) == 0;
                key = (low == up) ? min(key, other) : max(key, other);
            }
        }
        if (lane < len) entries[beg + lane] = key;
    } else if (len > 32 && len <= kWarpSortMax) {
        int32_t* a = s_sort[warp];
        const int m = len <= 64 ? 64 : 128;
        for (int i = lane; i < m; i += 32) a[i] = i < len ? entries[beg + i] : 0x7fffffff;
        __syncwarp();
        bitonic_smem(a, m, lane, 32, false);
        for (int i = lane; i < len; i += 32) entries[beg + i] = a[i];
    }
}

__global__ void __launch_bounds__(kThreads)
    k_csr_sort_long(const int32_t* __restrict__ offsets, int32_t* __restrict__ entries,
                    const int32_t* __restrict__ long_list, const int32_t* __restrict__ n_long_ptr,
                    int bitmap_words, unsigned long long* status) {
    extern __shared__ uint32_t s_mem[];  // bitmap | bitonic fallback
    __shared__ int s_warp[kWarpsPerCta];
    __shared__ int s_dup;
    uint32_t* bm = s_mem;
    int32_t* fb = reinterpret_cast<int32_t*>(s_mem + bitmap_words);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_long = *n_long_ptr;
    const int wpt = (bitmap_words + kThreads - 1) / kThreads;  // words per thread
    for (int i = blockIdx.x; i < n_long; i += gridDim.x) {
        const int row = long_list[i];
        const int beg = offsets[row], len = offsets[row + 1] - beg;
        for (int w = tid; w < bitmap_words; w += kThreads) bm[w] = 0u;
        if (tid == 0) s_dup = 0;
        __syncthreads();
        for (int j = tid; j < len; j += kThreads) {
            const unsigned e = (unsigned)entries[beg + j];
            const unsigned bit = 1u << (e & 31u);
            if ((int)(e >> 5) < bitmap_words) {
                if (atomicOr(bm + (e >> 5), bit) & bit) s_dup = 1;
            } else {
                s_dup = 1;
            }
        }
        __syncthreads();
        if (s_dup) {  // uniform over the CTA
            if (len <= kCtaBitonicMax) {
                int m = 256;
                while (m < len) m <<= 1;
                for (int j = tid; j < m; j += kThreads) fb[j] = j < len ? entries[beg + j] : 0x7fffffff;
                __syncthreads();
                bitonic_smem(fb, m, tid, kThreads, true);
                for (int j = tid; j < len; j += kThreads) entries[beg + j] = fb[j];
            } else if (tid == 0) {
                atomicAdd(status + 2, 1ULL);
            }
        } else {
            const int w_beg = min(bitmap_words, tid * wpt), w_end = min(bitmap_words, w_beg + wpt);
            int cnt = 0;
            for (int w = w_beg; w < w_end; ++w) cnt += __popc(bm[w]);
            int incl = cnt;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(kFullMask, incl, d);
                if (lane >= d) incl += t;
            }
            if (lane == 31) s_warp[warp] = incl;
            __syncthreads();
            int pos = incl - cnt;
            for (int x = 0; x < warp; ++x) pos += s_warp[x];
            for (int w = w_beg; w < w_end; ++w) {
                uint32_t bits = bm[w];
                while (bits) {
                    const int b = __ffs(bits) - 1;
                    entries[beg + pos++] = w * 32 + b;
                    bits &= bits - 1;
                }
            }
        }
        __syncthreads();
    }
}

// ---- pass 5: segment gather-sum ------------------------------------------
// One warp per (row, column tile); tiles are the slow grid dimension so the
// slice of `src` a tile reads (src_rows * U * 512 bytes) is L2 resident while
// the rows of that tile are produced.  Rows with more than `long_row` hits
// are split over the 8 warps of the CTA and combined in a fixed order.
template <int U>
__global__ void __launch_bounds__(kThreads)
    k_segment_reduce(const float4* __restrict__ src, int64_t W4, int64_t src_rows,
                     const int32_t* __restrict__ offsets, const int32_t* __restrict__ entries,
                     float4* __restrict__ out, int64_t N, int n_row_groups, int long_row,
                     unsigned long long* status) {
    __shared__ float4 s_part[kWarpsPerCta][U][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / n_row_groups;
    const int64_t row0 = (int64_t)(blockIdx.x % n_row_groups) * kWarpsPerCta;
    const int64_t row = row0 + warp;

    int col[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        col[u] = tile * (32 * U) + u * 32 + lane;
        ok[u] = col[u] < W4;
    }
    if (row < N) {
        const int beg = __ldg(offsets + row), len = __ldg(offsets + row + 1) - beg;
        if (len <= long_row) {
            float4 acc[U];
#pragma unroll
            for (int u = 0; u < U; ++u) acc[u] = f4_zero();
            gather_sum<U, 8 / U>(src, W4, src_rows, entries + beg, len, col, ok, acc, lane, status);
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (ok[u]) out[row * W4 + col[u]] = acc[u];
        }
    }
    for (int w = 0; w < kWarpsPerCta; ++w) {
        const int64_t r2 = row0 + w;
        if (r2 >= N) break;
        const int beg = __ldg(offsets + r2), len = __ldg(offsets + r2 + 1) - beg;
        if (len <= long_row) continue;  // uniform over the CTA
        const int per = (len + kWarpsPerCta - 1) / kWarpsPerCta;
        const int mb = min(len, warp * per), me = min(len, mb + per);
        float4 acc[U];
#pragma unroll
        for (int u = 0; u < U; ++u) acc[u] = f4_zero();
        gather_sum<U, 8 / U>(src, W4, src_rows, entries + beg + mb, me - mb, col, ok, acc, lane, status);
        __syncthreads();
#pragma unroll
        for (int u = 0; u < U; ++u) s_part[warp][u][lane] = acc[u];
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float4 s = s_part[0][u][lane];
                for (int x = 1; x < kWarpsPerCta; ++x) s = f4_add(s, s_part[x][u][lane]);
                if (ok[u]) out[r2 * W4 + col[u]] = s;
            }
        }
    }
}

// ---- pass 5, balanced form: one warp per CHUNK of the entry array ---------
// A chunk is `S` consecutive entries of the CSR, whatever rows they belong to,
// so every warp streams the same number of source rows and the load pipeline
// never drains at a row end; rows that one batch hits 16 000 times cost the
// same per entry as rows hit twice.  Inside a chunk the warp walks the row
// boundaries (warp-uniform branches).  A row that lies wholly inside the chunk
// is stored straight to `out`.  A row that crosses a chunk border leaves
// partial sums in `partial[chunk][0]` (piece that started in an earlier chunk)
// or `partial[chunk][1]` (piece that runs on into the next chunk);
// k_segment_fixup adds them in chunk order, k_zero_empty_rows writes the rows
// nobody touched.  Every order is fixed, so the result is reproducible.
// Rows [begin, end) whose gradient a launch has to finish (a slice of the
// table; the whole table by default).  A chunk takes part when any of its
// entries can belong to such a row: its first row lies before `end` and the
// next chunk's first row (>= this chunk's last row) not before `begin`.  A
// chunk on a slice border runs in both slices and writes the same values twice.
struct RowRange {
    int begin, end, max_chunks;
    int tile0;  // first column tile of the launch (column slices); blockIdx.x counts tiles from it
};
__device__ __forceinline__ bool chunk_in_range(const int32_t* __restrict__ chunk_row, int c, const RowRange& rr) {
    if (__ldg(chunk_row + c) >= rr.end) return false;
    if (c + 1 >= rr.max_chunks) return true;
    const int next = __ldg(chunk_row + c + 1);  // -1: no entries beyond this chunk
    return next < 0 || next >= rr.begin;
}

__global__ void __launch_bounds__(kThreads)
    k_chunk_rows(const int32_t* __restrict__ offsets, int64_t N, int S, int max_chunks,
                 int32_t* __restrict__ chunk_row) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= max_chunks) return;
    const int64_t e = (int64_t)c * S;
    if (e >= offsets[N]) {
        chunk_row[c] = -1;
        return;
    }
    // first index with offsets[i] > e, minus one: offsets[r] <= e < offsets[r+1]
    int64_t lo = 0, hi = N;  // answer in (lo, hi]
    while (hi - lo > 1) {
        const int64_t mid = (lo + hi) >> 1;
        if (offsets[mid] <= e) lo = mid; else hi = mid;
    }
    chunk_row[c] = (int32_t)lo;
}

// OFFS: the launch covers the column tiles from rr.tile0 on (column slices).  A template parameter, because the
// added offset alone cost the whole-table launch 3 % (0.852 -> 0.878 ms at the benchmark shape, measured on one GPU
// with the two builds side by side).
template <int U, int R, int MINB, bool OFFS>
__global__ void __launch_bounds__(kThreads, MINB)
    k_segment_chunks(const float4* __restrict__ src, int64_t W4, int64_t src_rows,
                     const int32_t* __restrict__ offsets, const int32_t* __restrict__ entries,
                     const int32_t* __restrict__ chunk_row, float4* __restrict__ out,
                     float4* __restrict__ partial, int64_t N, int n_chunk_groups, int S,
                     unsigned long long* status, RowRange rr) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = OFFS ? rr.tile0 + blockIdx.x / n_chunk_groups : blockIdx.x / n_chunk_groups;
    const int c = (blockIdx.x % n_chunk_groups) * kWarpsPerCta + warp;
    const int E = __ldg(offsets + N);
    const int e_beg = c * S;
    if (e_beg >= E) return;  // warp-uniform
    if (!chunk_in_range(chunk_row, c, rr)) return;
    const int e_end = min(E, e_beg + S);

    int col[U];
    bool ok[U];
    float4 acc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        col[u] = tile * (32 * U) + u * 32 + lane;
        ok[u] = col[u] < W4;
        acc[u] = f4_zero();
    }
    int row = __ldg(chunk_row + c);
    int row_beg = __ldg(offsets + row), next_b = __ldg(offsets + row + 1);
    int piece_beg = e_beg;

    auto flush = [&](int pe) {  // piece [piece_beg, pe) of `row`
        if (next_b == row_beg) return;  // empty row: k_zero_empty_rows owns it
        float4* dst;
        if (piece_beg == row_beg && pe == next_b) {
            if (row < rr.begin || row >= rr.end) return;  // a border chunk: that row belongs to another slice
            dst = out + (int64_t)row * W4;
        }
        else if (piece_beg == e_beg && row_beg < e_beg) dst = partial + ((int64_t)c * 2 + 0) * W4;
        else dst = partial + ((int64_t)c * 2 + 1) * W4;
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (ok[u]) dst[col[u]] = acc[u];
    };

    // entry i of this chunk is entry e_beg + i of the CSR; a row ends where the
    // running index meets `next_b` (the loop also steps over empty rows)
    auto at_entry = [&](int i) {
        const int e = e_beg + i;
        while (e == next_b) {
            flush(e);
            ++row;
            row_beg = next_b;
            next_b = __ldg(offsets + row + 1);
            piece_beg = e;
#pragma unroll
            for (int u = 0; u < U; ++u) acc[u] = f4_zero();
        }
    };
    gather_sum_pipelined<U, R>(src, W4, src_rows, entries + e_beg, e_end - e_beg, col, ok, acc, lane,
                               status, tile == 0, at_entry);
    flush(e_end);
}

// One warp per (chunk, tile): if the row whose piece opens this chunk also ends
// in this chunk, add up its pieces from the chunk it started in to this one.
template <int U, bool OFFS>
__global__ void __launch_bounds__(kThreads)
    k_segment_fixup(const int32_t* __restrict__ offsets, const int32_t* __restrict__ chunk_row,
                    const float4* __restrict__ partial, float4* __restrict__ out, int64_t W4,
                    int64_t N, int n_chunk_groups, int S, RowRange rr) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = OFFS ? rr.tile0 + blockIdx.x / n_chunk_groups : blockIdx.x / n_chunk_groups;
    const int c = (blockIdx.x % n_chunk_groups) * kWarpsPerCta + warp;
    const int E = __ldg(offsets + N);
    const int e_beg = c * S;
    if (e_beg >= E) return;
    const int r = __ldg(chunk_row + c);
    if (r < rr.begin || r >= rr.end) return;  // the row this warp would finish belongs to another slice
    const int rb = __ldg(offsets + r), re = __ldg(offsets + r + 1);
    if (rb >= e_beg) return;        // the opening row starts here: it has no earlier piece
    if (re > e_beg + S) return;     // it runs on: a later chunk finishes it
    const int a = rb / S;           // chunk the row started in (its piece there is a [1] piece)
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int cc = tile * (32 * U) + u * 32 + lane;
        if (cc >= W4) continue;
        float4 s = partial[((int64_t)a * 2 + 1) * W4 + cc];
        for (int x = a + 1; x <= c; ++x) s = f4_add(s, partial[((int64_t)x * 2 + 0) * W4 + cc]);
        out[(int64_t)r * W4 + cc] = s;
    }
}

// One warp per row: rows without a single entry get zeros.
__global__ void __launch_bounds__(kThreads)
    k_zero_empty_rows(const int32_t* __restrict__ offsets, float4* __restrict__ out, int64_t W4,
                      int64_t row0, int64_t N) {
    const int lane = threadIdx.x & 31;
    const int64_t row = row0 + (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (row >= N) return;
    if (__ldg(offsets + row) != __ldg(offsets + row + 1)) return;
    for (int64_t c = lane; c < W4; c += 32) out[row * W4 + c] = f4_zero();
}

// Scalar twin for W % 4 != 0 or unaligned buffers: lane = one column.
__global__ void __launch_bounds__(kThreads)
    k_segment_reduce_scalar(const float* __restrict__ src, int W, int64_t src_rows,
                            const int32_t* __restrict__ offsets,
                            const int32_t* __restrict__ entries, float* __restrict__ out, int64_t N,
                            int n_row_groups, unsigned long long* status) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / n_row_groups;
    const int64_t row = (int64_t)(blockIdx.x % n_row_groups) * kWarpsPerCta + warp;
    const int c = tile * 32 + lane;
    if (row >= N || c >= W) return;
    const int beg = offsets[row], end = offsets[row + 1];
    float acc = 0.f;
    for (int i = beg; i < end; ++i) {
        const int e = entries[i];
        if ((int64_t)e >= src_rows || e < 0) { if (lane == 0) note_bad_index(status); continue; }
        acc = __fadd_rn(acc, src[(int64_t)e * W + c]);
    }
    out[row * W + c] = acc;
}

// ---- column sums ----------------------------------------------------------
// grid.x = column chunk (32 float4), grid.y = row slice; the 8 warps of a CTA
// take rows slice_beg + w, + 8, ...; combined in warp order.
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
    k_column_sum(const float* __restrict__ src, int64_t rows, int W, float* __restrict__ out,
                 int n_slices) {
    __shared__ float4 s_part[kWarpsPerCta][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t per = (rows + n_slices - 1) / n_slices;
    const int64_t r_beg = (int64_t)blockIdx.y * per;
    const int64_t r_end = min(rows, r_beg + per);
    const int c = blockIdx.x * 32 + lane;
    float4 acc = f4_zero();
    if (VEC) {
        const int W4 = W >> 2;
        const float4* s4 = reinterpret_cast<const float4*>(src);
        if (c < W4) {
            int64_t r = r_beg + warp;
            for (; r + 3 * kWarpsPerCta < r_end; r += 4 * kWarpsPerCta) {
                const float4 a0 = ldg4(s4 + r * W4 + c);
                const float4 a1 = ldg4(s4 + (r + kWarpsPerCta) * W4 + c);
                const float4 a2 = ldg4(s4 + (r + 2 * kWarpsPerCta) * W4 + c);
                const float4 a3 = ldg4(s4 + (r + 3 * kWarpsPerCta) * W4 + c);
                acc = f4_add(f4_add(f4_add(f4_add(acc, a0), a1), a2), a3);
            }
            for (; r < r_end; r += kWarpsPerCta) acc = f4_add(acc, ldg4(s4 + r * W4 + c));
        }
    } else {
        if (c < W) {
            for (int64_t r = r_beg + warp; r < r_end; r += kWarpsPerCta)
                acc.x = __fadd_rn(acc.x, src[r * W + c]);
        }
    }
    s_part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0) {
        float4 s = s_part[0][lane];
        for (int x = 1; x < kWarpsPerCta; ++x) s = f4_add(s, s_part[x][lane]);
        float* dst = out + (int64_t)blockIdx.y * W;
        if (VEC) {
            if (c < (W >> 2)) reinterpret_cast<float4*>(dst)[c] = s;
        } else if (c < W) {
            dst[c] = s.x;
        }
    }
}

int column_sum(const float* src, int64_t rows, int W, float* out, cudaStream_t s, float* scratch) {
    if (W <= 0) return NNUE_OK;
    if (rows <= 0) {
        NNUE_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)W * sizeof(float), s));
        return NNUE_OK;
    }
    const bool two_stage = scratch != nullptr && rows > kColumnSumDirectRows;
    const bool vec = (W % 4 == 0) && aligned16(src) && aligned16(out) &&
                     (!two_stage || aligned16(scratch));
    const int cols = vec ? W / 4 : W;
    const unsigned gx = (unsigned)((cols + 31) / 32);
    ProfScope prof("k_column_sum", s);
    auto launch = [&](const float* in, int64_t n, float* dst, int slices) {
        dim3 grid(gx, (unsigned)slices);
        if (vec) k_column_sum<true><<<grid, kThreads, 0, s>>>(in, n, W, dst, slices);
        else k_column_sum<false><<<grid, kThreads, 0, s>>>(in, n, W, dst, slices);
    };
    if (two_stage) {
        launch(src, rows, scratch, kColumnSumSlices);
        launch(scratch, kColumnSumSlices, out, 1);
        note_launches(2);
    } else {
        launch(src, rows, out, 1);
        note_launches(1);
    }
    NNUE_CUDA_TRY(cudaGetLastError());
    return NNUE_OK;
}

int csr_plan(CsrPlan& plan, int n_lists, int64_t B, int K, int64_t N, int W, void* ws,
             size_t ws_bytes) {
    NNUE_REQUIRE(n_lists == 1 || n_lists == 2, NNUE_ERR_ARG, "csr: n_lists must be 1 or 2");
    NNUE_REQUIRE(N < 0x7fffffffLL && B * n_lists < 0x7fffffffLL &&
                     B * (int64_t)n_lists * K < 0x7fffffffLL,
                 NNUE_ERR_UNSUPPORTED, "csr: sizes exceed 31-bit entry ids");
    const int64_t max_entries = B * (int64_t)n_lists * K;
    const size_t need = csr_workspace_bytes(max_entries, N, W);
    NNUE_REQUIRE(ws && ws_bytes >= need, NNUE_ERR_WORKSPACE, "csr: workspace %zu < required %zu",
                 ws_bytes, need);
    plan.n_lists = n_lists;
    plan.B = B;
    plan.K = K;
    plan.N = N;
    plan.S = tuning().seg_chunk;
    plan.max_chunks = plan.S > 0 ? max_chunks_for(max_entries, plan.S) : 0;
    char* p = reinterpret_cast<char*>(align_up(reinterpret_cast<uintptr_t>(ws), 256));
    auto take = [&p](size_t bytes) {
        char* r = p;
        p += align_up(bytes, 256);
        return r;
    };
    const size_t ent = (size_t)(max_entries > 0 ? max_entries : 1) * sizeof(int32_t);
    plan.counts = reinterpret_cast<int32_t*>(take((size_t)(N + 1) * sizeof(int32_t)));
    plan.n_long = plan.counts + N;  // counts[N] is the long-row counter
    plan.long_list = reinterpret_cast<int32_t*>(take((size_t)N * sizeof(int32_t)));
    plan.offsets = reinterpret_cast<int32_t*>(take((size_t)(N + 1) * sizeof(int32_t)));
    plan.ranks = reinterpret_cast<int32_t*>(take(ent));
    plan.entries = reinterpret_cast<int32_t*>(take(ent));
    plan.chunk_row = reinterpret_cast<int32_t*>(take((size_t)plan.max_chunks * sizeof(int32_t)));
    plan.partial = reinterpret_cast<float*>(p);
    return NNUE_OK;
}

int csr_build(const CsrPlan& plan, const int32_t* const* lists, cudaStream_t s) {
    const int64_t N = plan.N, B = plan.B;
    const int K = plan.K, n_lists = plan.n_lists;
    if (N == 0) return NNUE_OK;
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "csr: no device status word");
    ProfScope prof("csr_build (7 kernels)", s);
    NNUE_CUDA_TRY(cudaMemsetAsync(plan.counts, 0, (size_t)(N + 1) * sizeof(int32_t), s));
    const int64_t warps = B * n_lists;
    const unsigned lgrid = (unsigned)((warps + kWarpsPerCta - 1) / kWarpsPerCta);
    const int32_t* l0 = lists[0];
    const int32_t* l1 = n_lists > 1 ? lists[1] : lists[0];
    if (warps > 0 && K > 0) {
        k_csr_scan_lists<false><<<lgrid, kThreads, 0, s>>>(l0, l1, n_lists, B, K, N, plan.counts,
                                                          plan.ranks, plan.entries, status);
        note_launches(1);
    }
    k_csr_scan<<<1, 1024, 0, s>>>(plan.counts, plan.offsets, plan.offsets, N, plan.long_list,
                                  plan.n_long, kWarpSortMax);
    note_launches(1);
    if (warps > 0 && K > 0) {
        k_csr_scan_lists<true><<<lgrid, kThreads, 0, s>>>(l0, l1, n_lists, B, K, N, plan.offsets,
                                                         plan.ranks, plan.entries, status);
        note_launches(1);
    }
    const int64_t row_groups = (N + kWarpsPerCta - 1) / kWarpsPerCta;
    if (tuning().sort_segments && warps > 0 && K > 0) {
        k_csr_sort_short<<<(unsigned)row_groups, kThreads, 0, s>>>(plan.offsets, plan.entries, N);
        note_launches(1);
        const int64_t key_space = B * n_lists;
        if (key_space <= kBitmapMaxBits) {
            const int words = (int)((key_space + 31) / 32);
            const size_t smem = (size_t)words * 4 + (size_t)kCtaBitonicMax * 4;
            static size_t attr_smem = 0;  // largest size opted in so far
            if (smem > 48 * 1024 && smem > attr_smem) {
                NNUE_CUDA_TRY(cudaFuncSetAttribute(
                    k_csr_sort_long, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                attr_smem = smem;
            }
            const unsigned g = (unsigned)std::min<int64_t>(N, (int64_t)sm_count() * 4);
            k_csr_sort_long<<<g, kThreads, smem, s>>>(plan.offsets, plan.entries, plan.long_list,
                                                     plan.n_long, words, status);
            note_launches(1);
        }
    }
    if (plan.S > 0) {
        k_chunk_rows<<<(unsigned)((plan.max_chunks + kThreads - 1) / kThreads), kThreads, 0, s>>>(
            plan.offsets, N, plan.S, (int)plan.max_chunks, plan.chunk_row);
        note_launches(1);
    }
    NNUE_CUDA_TRY(cudaGetLastError());
    return NNUE_OK;
}

static int segment_unroll(int64_t W4) {
    int U = tuning().bwd_u;
    if (U != 1 && U != 2 && U != 4) U = 2;
    while (U > 1 && W4 <= 32 * (U / 2)) U /= 2;
    return U;
}

int csr_column_tile(int W) { return W % 4 == 0 ? 32 * segment_unroll(W / 4) * 4 : 0; }

int csr_reduce(const CsrPlan& plan, const float* src, int W, float* out, cudaStream_t s, int64_t row_begin,
               int64_t row_end, int64_t col_begin, int64_t col_end) {
    const int64_t N = plan.N, src_rows = plan.B * plan.n_lists;
    if (N == 0) return NNUE_OK;
    if (row_end < 0 || row_end > N) row_end = N;
    if (col_end < 0 || col_end > W) col_end = W;
    NNUE_REQUIRE(row_begin >= 0 && row_begin <= row_end, NNUE_ERR_ARG, "csr: bad row range");
    NNUE_REQUIRE(col_begin >= 0 && col_begin <= col_end, NNUE_ERR_ARG, "csr: bad column range");
    if (row_begin == row_end || col_begin == col_end) return NNUE_OK;
    const bool whole = row_begin == 0 && row_end == N && col_begin == 0 && col_end == W;
    RowRange rr{(int)row_begin, (int)row_end, (int)plan.max_chunks, 0};
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "csr: no device status word");
    const int64_t row_groups = (N + kWarpsPerCta - 1) / kWarpsPerCta;
    const int S = plan.S;
    const bool vec = (W % 4 == 0) && aligned16(src) && aligned16(out);
    if (vec) {
        const int64_t W4 = W / 4;
        const int U = segment_unroll(W4);
        const int64_t all_tiles = (W4 + 32 * U - 1) / (32 * U);
        const int tile_w = 32 * U * 4;
        NNUE_REQUIRE(col_begin % tile_w == 0 && (col_end % tile_w == 0 || col_end == W), NNUE_ERR_ARG,
                     "csr: column bounds must be multiples of %d floats", tile_w);
        const int64_t tile_b = col_begin / tile_w, tile_e = col_end == W ? all_tiles : col_end / tile_w;
        const int64_t tiles = S > 0 ? tile_e - tile_b : all_tiles;
        rr.tile0 = (int)tile_b;
        const float4* s4 = reinterpret_cast<const float4*>(src);
        float4* o4 = reinterpret_cast<float4*>(out);
        if (S > 0) {
            const int64_t groups = (plan.max_chunks + kWarpsPerCta - 1) / kWarpsPerCta;
            NNUE_REQUIRE(tiles * groups <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "csr: grid too large");
            const unsigned grid = (unsigned)(tiles * groups);
            float4* p4 = reinterpret_cast<float4*>(plan.partial);
            if (tile_b == 0) {  // whole rows, with the first column slice
                ProfScope prof("k_zero_empty_rows", s);
                k_zero_empty_rows<<<(unsigned)((row_end - row_begin + kWarpsPerCta - 1) / kWarpsPerCta), kThreads, 0, s>>>(
                    plan.offsets, o4, W4, row_begin, row_end);
            }
            // variant = rows per register buffer (R) and CTAs per SM the register budget must allow
            const int v = tuning().bwd_r;
            const bool offs = tile_b != 0;
#define LAUNCH_CHUNKS(UU, RR, MB)                                                                            \
    do {                                                                                                     \
        if (offs)                                                                                            \
            k_segment_chunks<UU, RR, MB, true><<<grid, kThreads, 0, s>>>(s4, W4, src_rows, plan.offsets, plan.entries, \
                                                                         plan.chunk_row, o4, p4, N, (int)groups, S, status, rr); \
        else                                                                                                 \
            k_segment_chunks<UU, RR, MB, false><<<grid, kThreads, 0, s>>>(s4, W4, src_rows, plan.offsets, plan.entries, \
                                                                          plan.chunk_row, o4, p4, N, (int)groups, S, status, rr); \
    } while (0)
            {
            ProfScope prof("k_segment_chunks", s);
            if (U == 1) {
                if (v == 1) LAUNCH_CHUNKS(1, 2, 6); else if (v == 2) LAUNCH_CHUNKS(1, 4, 4);
                else LAUNCH_CHUNKS(1, 2, 4);
            } else if (U == 2) {
                if (v == 1) LAUNCH_CHUNKS(2, 1, 6); else if (v == 2) LAUNCH_CHUNKS(2, 2, 4);
                else if (v == 3) LAUNCH_CHUNKS(2, 1, 5); else if (v == 4) LAUNCH_CHUNKS(2, 2, 3);
                else LAUNCH_CHUNKS(2, 1, 4);
            } else {
                if (v == 1) LAUNCH_CHUNKS(4, 1, 3); else LAUNCH_CHUNKS(4, 1, 4);
            }
            }
#undef LAUNCH_CHUNKS
            ProfScope prof_fix("k_segment_fixup", s);
#define LAUNCH_FIXUP(UU)                                                                                              \
    do {                                                                                                              \
        if (offs) k_segment_fixup<UU, true><<<grid, kThreads, 0, s>>>(plan.offsets, plan.chunk_row, p4, o4, W4, N, (int)groups, S, rr); \
        else k_segment_fixup<UU, false><<<grid, kThreads, 0, s>>>(plan.offsets, plan.chunk_row, p4, o4, W4, N, (int)groups, S, rr);    \
    } while (0)
            if (U == 1) LAUNCH_FIXUP(1);
            else if (U == 2) LAUNCH_FIXUP(2);
            else LAUNCH_FIXUP(4);
#undef LAUNCH_FIXUP
            note_launches(3);
        } else {
            NNUE_REQUIRE(whole, NNUE_ERR_UNSUPPORTED, "csr: slices need the chunked reduction (seg_chunk > 0)");
            NNUE_REQUIRE(tiles * row_groups <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "csr: grid too large");
            const unsigned grid = (unsigned)(tiles * row_groups);
            const int long_row = tuning().long_row;
            if (U == 1)
                k_segment_reduce<1><<<grid, kThreads, 0, s>>>(s4, W4, src_rows, plan.offsets, plan.entries,
                                                             o4, N, (int)row_groups, long_row, status);
            else if (U == 2)
                k_segment_reduce<2><<<grid, kThreads, 0, s>>>(s4, W4, src_rows, plan.offsets, plan.entries,
                                                             o4, N, (int)row_groups, long_row, status);
            else
                k_segment_reduce<4><<<grid, kThreads, 0, s>>>(s4, W4, src_rows, plan.offsets, plan.entries,
                                                             o4, N, (int)row_groups, long_row, status);
            note_launches(1);
        }
    } else {
        NNUE_REQUIRE(whole, NNUE_ERR_UNSUPPORTED, "csr: slices need 16-byte aligned rows");
        const int64_t tiles = (W + 31) / 32;
        NNUE_REQUIRE(tiles * row_groups <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "csr: grid too large");
        k_segment_reduce_scalar<<<(unsigned)(tiles * row_groups), kThreads, 0, s>>>(
            src, W, src_rows, plan.offsets, plan.entries, out, N, (int)row_groups, status);
        note_launches(1);
    }
    NNUE_CUDA_TRY(cudaGetLastError());
    return NNUE_OK;
}

// Per-device helper stream and events for overlapping the CSR build (atomics,
// latency bound) with DRAM-bound work on the caller's stream.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
static SideStream* side_stream() {
    static SideStream table[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    SideStream& t = table[dev];
    if (!t.stream) {
        if (cudaStreamCreateWithFlags(&t.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
        if (cudaEventCreateWithFlags(&t.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        if (cudaEventCreateWithFlags(&t.join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    }
    return &t;
}

bool side_stream_get(SideStreamView& out) {
    SideStream* side = side_stream();
    if (!side) return false;
    out.stream = side->stream;
    out.fork = side->fork;
    out.join = side->join;
    return true;
}

int csr_build_overlapped(const CsrPlan& plan, const int32_t* const* lists, cudaStream_t s,
                         CsrJoin& join) {
    join.pending = false;
    SideStream* side = tuning().overlap_csr ? side_stream() : nullptr;
    if (!side) return csr_build(plan, lists, s);
    NNUE_CUDA_TRY(cudaEventRecord(side->fork, s));
    NNUE_CUDA_TRY(cudaStreamWaitEvent(side->stream, side->fork, 0));
    const int rc = csr_build(plan, lists, side->stream);
    // always join, also after a failed launch, so the caller's stream stays ordered
    NNUE_CUDA_TRY(cudaEventRecord(side->join, side->stream));
    join.pending = true;
    join.event = side->join;
    return rc;
}

int csr_join(CsrJoin& join, cudaStream_t s) {
    if (join.pending) {
        NNUE_CUDA_TRY(cudaStreamWaitEvent(s, join.event, 0));
        join.pending = false;
    }
    return NNUE_OK;
}

}  // namespace nnue
