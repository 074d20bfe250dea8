// The bucketed layer stack behind the feature transformer, as a handful of
// kernels instead of three wide GEMMs plus ~150 small elementwise launches.
//
// The reference computes every layer for all 8 buckets and then keeps the
// slice of the position's own bucket (model/modules/stacked_linear.py:38-66 of
// the reference project): 8x the arithmetic that is used.  Here positions are
// grouped by bucket once per batch (k_ls_plan, this file: a stable counting
// sort into tiles of 64 positions of one bucket) and every kernel works tile
// by tile on the bucket's own 32-wide weight block, in fp32 FMA arithmetic
// (layer_stack_l1.cu: first layer forward / input gradient / weight gradient;
// layer_stack_tail.cu: activations, second and output layer, skip connection,
// output fake quantization and their gradient).  All sums run in a fixed
// order: results are reproducible.
// Shapes: L2 = L3 = 32 (one lane per output), L1 % 32 == 0, buckets <= 16.
#include "layer_stack.cuh"

namespace nnue {

// Single CTA: per-thread histograms over a contiguous slice of positions, a
// scan per bucket across threads, then an in-order fill (stable).
constexpr int kPlanThreads = 512;
constexpr int kMaxBuckets = 16;  // kMaxBuckets * kPlanThreads counters fit 48 KB of shared memory
__global__ void __launch_bounds__(kPlanThreads)
    k_ls_plan(const int64_t* __restrict__ bucket, int64_t B, int C, int32_t* __restrict__ plan,
              unsigned long long* status) {
    extern __shared__ int32_t s_cnt[];  // [C][kPlanThreads] then [C]
    int32_t* s_base = s_cnt + C * kPlanThreads;
    const int tid = threadIdx.x;
    const int64_t per = (B + kPlanThreads - 1) / kPlanThreads;
    const int64_t lo = min(B, tid * per), hi = min(B, lo + per);
    for (int c = 0; c < C; ++c) s_cnt[c * kPlanThreads + tid] = 0;
    for (int64_t p = lo; p < hi; ++p) {
        int64_t b = bucket[p];
        if (b < 0 || b >= C) { note_bad_index(status); b = 0; }
        s_cnt[(int)b * kPlanThreads + tid] += 1;
    }
    __syncthreads();
    if (tid < C) {  // exclusive scan over the threads, one bucket per scanning thread
        int run = 0;
        for (int t = 0; t < kPlanThreads; ++t) {
            const int v = s_cnt[tid * kPlanThreads + t];
            s_cnt[tid * kPlanThreads + t] = run;
            run += v;
        }
        s_base[tid] = run;  // bucket size for now
    }
    __syncthreads();
    const int64_t T = ls_max_tiles(B, C);
    int32_t* bucket_tile = plan + 4;
    int32_t* tile_start = bucket_tile + (C + 1 + 3) / 4 * 4;
    int32_t* tile_count = tile_start + T;
    int32_t* tile_bucket = tile_count + T;
    int32_t* perm = tile_bucket + T;
    if (tid == 0) {
        int pos = 0, tile = 0;
        for (int c = 0; c < C; ++c) {
            const int n = s_base[c];
            s_base[c] = pos;
            bucket_tile[c] = tile;
            for (int o = 0; o < n; o += kTP) {
                tile_start[tile] = pos + o;
                tile_count[tile] = min(kTP, n - o);
                tile_bucket[tile] = c;
                ++tile;
            }
            pos += n;
        }
        bucket_tile[C] = tile;
        plan[0] = tile;
    }
    __syncthreads();
    // s_cnt[c][tid] holds this thread's first slot inside bucket c; advance it in place
    for (int64_t p = lo; p < hi; ++p) {
        int64_t b = bucket[p];
        if (b < 0 || b >= C) b = 0;
        int32_t& cur = s_cnt[(int)b * kPlanThreads + tid];
        perm[s_base[(int)b] + cur] = (int32_t)p;
        cur += 1;
    }
}

}  // namespace nnue

using namespace nnue;

extern "C" size_t nnue_ls_plan_bytes(int64_t B, int32_t C) {
    if (B < 0 || C <= 0) return 0;
    return (size_t)ls_plan_ints(B, C) * sizeof(int32_t);
}

extern "C" int nnue_ls_plan(const int64_t* bucket, int64_t B, int32_t C, void* plan, size_t plan_bytes,
                            void* stream) {
    NNUE_REQUIRE(B >= 0 && C > 0 && C <= kMaxBuckets, NNUE_ERR_UNSUPPORTED,
                 "nnue_ls_plan: %d buckets outside 1..%d (or negative batch)", C, kMaxBuckets);
    NNUE_REQUIRE(B < 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "nnue_ls_plan: batch too large");
    NNUE_REQUIRE(plan && plan_bytes >= nnue_ls_plan_bytes(B, C) && aligned16(plan), NNUE_ERR_WORKSPACE,
                 "nnue_ls_plan: plan buffer too small or unaligned");
    NNUE_REQUIRE(B == 0 || bucket, NNUE_ERR_ARG, "nnue_ls_plan: null bucket list");
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "nnue_ls_plan: no device status word");
    const size_t smem = ((size_t)C * kPlanThreads + C) * sizeof(int32_t);
    k_ls_plan<<<1, kPlanThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        bucket, B, C, static_cast<int32_t*>(plan), status);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
