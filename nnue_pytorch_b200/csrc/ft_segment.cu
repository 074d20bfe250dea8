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

size_t csr_workspace_bytes(int64_t max_entries, int64_t n_rows) {
    size_t b = 0;
    b += align_up((size_t)(n_rows + 1) * sizeof(int32_t), 256);  // counts + long-row counter
    b += align_up((size_t)n_rows * sizeof(int32_t), 256);        // long-row list
    b += align_up((size_t)(n_rows + 1) * sizeof(int32_t), 256);  // offsets
    b += align_up((size_t)n_rows * sizeof(int32_t), 256);        // cursors
    b += align_up((size_t)(max_entries > 0 ? max_entries : 1) * sizeof(int32_t), 256);  // entries
    return b + 256;
}

// ---- pass 1 / pass 3: one warp per (position, list) ----------------------
template <bool FILL>
__global__ void __launch_bounds__(kThreads)
    k_csr_scan_lists(const int32_t* __restrict__ list0, const int32_t* __restrict__ list1,
                     int n_lists, int64_t B, int K, int64_t N, int32_t* __restrict__ counts_or_cursor,
                     int32_t* __restrict__ entries, unsigned long long* status) {
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
                if (FILL) {
                    const int pos = atomicAdd(counts_or_cursor + r, 1);
                    entries[pos] = e;
                } else {
                    atomicAdd(counts_or_cursor + r, 1);
                }
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
            gather_sum<U, 16 / U>(src, W4, src_rows, entries + beg, len, col, ok, acc, lane, status);
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
        gather_sum<U, 16 / U>(src, W4, src_rows, entries + beg + mb, me - mb, col, ok, acc, lane, status);
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

int csr_build_and_reduce(const int32_t* const* lists, int n_lists, int64_t B, int K, int64_t N,
                         const float* src, int W, float* out, void* ws, size_t ws_bytes,
                         cudaStream_t s) {
    NNUE_REQUIRE(n_lists == 1 || n_lists == 2, NNUE_ERR_ARG, "csr: n_lists must be 1 or 2");
    if (N == 0) return NNUE_OK;
    NNUE_REQUIRE(N < 0x7fffffffLL && B * n_lists < 0x7fffffffLL &&
                     B * (int64_t)n_lists * K < 0x7fffffffLL,
                 NNUE_ERR_UNSUPPORTED, "csr: sizes exceed 31-bit entry ids");
    const size_t need = csr_workspace_bytes(B * (int64_t)n_lists * K, N);
    NNUE_REQUIRE(ws && ws_bytes >= need, NNUE_ERR_WORKSPACE, "csr: workspace %zu < required %zu",
                 ws_bytes, need);
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "csr: no device status word");

    char* p = reinterpret_cast<char*>(align_up(reinterpret_cast<uintptr_t>(ws), 256));
    int32_t* counts = reinterpret_cast<int32_t*>(p);  // counts[N] is the long-row counter
    int32_t* n_long = counts + N;
    p += align_up((size_t)(N + 1) * sizeof(int32_t), 256);
    int32_t* long_list = reinterpret_cast<int32_t*>(p);
    p += align_up((size_t)N * sizeof(int32_t), 256);
    int32_t* offsets = reinterpret_cast<int32_t*>(p);
    p += align_up((size_t)(N + 1) * sizeof(int32_t), 256);
    int32_t* cursor = reinterpret_cast<int32_t*>(p);
    p += align_up((size_t)N * sizeof(int32_t), 256);
    int32_t* entries = reinterpret_cast<int32_t*>(p);

    NNUE_CUDA_TRY(cudaMemsetAsync(counts, 0, (size_t)(N + 1) * sizeof(int32_t), s));
    const int64_t warps = B * n_lists;
    const unsigned lgrid = (unsigned)((warps + kWarpsPerCta - 1) / kWarpsPerCta);
    const int32_t* l0 = lists[0];
    const int32_t* l1 = n_lists > 1 ? lists[1] : lists[0];
    if (warps > 0 && K > 0) {
        k_csr_scan_lists<false><<<lgrid, kThreads, 0, s>>>(l0, l1, n_lists, B, K, N, counts, entries,
                                                          status);
        note_launches(2);  // this pass and the fill pass below
    }
    k_csr_scan<<<1, 1024, 0, s>>>(counts, offsets, cursor, N, long_list, n_long, kWarpSortMax);
    note_launches(2);  // the scan and the segment gather-sum at the end
    if (warps > 0 && K > 0) {
        k_csr_scan_lists<true><<<lgrid, kThreads, 0, s>>>(l0, l1, n_lists, B, K, N, cursor, entries,
                                                         status);
    }
    const int64_t row_groups = (N + kWarpsPerCta - 1) / kWarpsPerCta;
    if (tuning().sort_segments && warps > 0 && K > 0) {
        k_csr_sort_short<<<(unsigned)row_groups, kThreads, 0, s>>>(offsets, entries, N);
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
            k_csr_sort_long<<<g, kThreads, smem, s>>>(offsets, entries, long_list, n_long, words,
                                                     status);
            note_launches(1);
        }
    }
    NNUE_CUDA_TRY(cudaGetLastError());

    const bool vec = (W % 4 == 0) && aligned16(src) && aligned16(out);
    if (vec) {
        const int64_t W4 = W / 4;
        int U = tuning().bwd_u;
        if (U != 1 && U != 2 && U != 4) U = 2;
        while (U > 1 && W4 <= 32 * (U / 2)) U /= 2;
        const int64_t tiles = (W4 + 32 * U - 1) / (32 * U);
        NNUE_REQUIRE(tiles * row_groups <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "csr: grid too large");
        const unsigned grid = (unsigned)(tiles * row_groups);
        const float4* s4 = reinterpret_cast<const float4*>(src);
        float4* o4 = reinterpret_cast<float4*>(out);
        const int long_row = tuning().long_row;
        if (U == 1)
            k_segment_reduce<1><<<grid, kThreads, 0, s>>>(s4, W4, B * n_lists, offsets, entries, o4, N,
                                                         (int)row_groups, long_row, status);
        else if (U == 2)
            k_segment_reduce<2><<<grid, kThreads, 0, s>>>(s4, W4, B * n_lists, offsets, entries, o4, N,
                                                         (int)row_groups, long_row, status);
        else
            k_segment_reduce<4><<<grid, kThreads, 0, s>>>(s4, W4, B * n_lists, offsets, entries, o4, N,
                                                         (int)row_groups, long_row, status);
    } else {
        const int64_t tiles = (W + 31) / 32;
        NNUE_REQUIRE(tiles * row_groups <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "csr: grid too large");
        k_segment_reduce_scalar<<<(unsigned)(tiles * row_groups), kThreads, 0, s>>>(
            src, W, B * n_lists, offsets, entries, out, N, (int)row_groups, status);
    }
    NNUE_CUDA_TRY(cudaGetLastError());
    return NNUE_OK;
}

}  // namespace nnue
