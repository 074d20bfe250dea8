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

// Single CTA: per-thread histograms over a contiguous slice of positions, one
// warp per bucket scans them across the threads, tiles are listed in parallel,
// then an in-order fill (stable).
constexpr int kPlanThreads = 1024;
constexpr int kMaxBuckets = 16;
// counters [C][kPlanThreads] live in dynamic shared memory (64 KB at 16 buckets)
__global__ void __launch_bounds__(kPlanThreads)
    k_ls_plan(const int64_t* __restrict__ bucket, int64_t B, int C, int32_t* __restrict__ plan,
              unsigned long long* status) {
    extern __shared__ int32_t s_cnt[];  // [C][kPlanThreads]
    __shared__ int32_t s_size[kMaxBuckets], s_base[kMaxBuckets], s_tile0[kMaxBuckets + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t per = (B + kPlanThreads - 1) / kPlanThreads;
    const int64_t lo = min(B, tid * per), hi = min(B, lo + per);
    for (int c = 0; c < C; ++c) s_cnt[c * kPlanThreads + tid] = 0;
    for (int64_t p = lo; p < hi; ++p) {
        int64_t b = bucket[p];
        if (b < 0 || b >= C) { note_bad_index(status); b = 0; }
        s_cnt[(int)b * kPlanThreads + tid] += 1;
    }
    __syncthreads();
    if (warp < C) {  // exclusive scan of bucket `warp` over the threads: 32 consecutive counters per lane
        int32_t* row = s_cnt + warp * kPlanThreads + lane * (kPlanThreads / 32);
        int sum = 0;
        for (int i = 0; i < kPlanThreads / 32; ++i) sum += row[i];
        int incl = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(kFullMask, incl, d);
            if (lane >= d) incl += v;
        }
        int run = incl - sum;
        for (int i = 0; i < kPlanThreads / 32; ++i) {
            const int v = row[i];
            row[i] = run;
            run += v;
        }
        if (lane == 31) s_size[warp] = incl;
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
            s_base[c] = pos;
            s_tile0[c] = tile;
            bucket_tile[c] = tile;
            pos += s_size[c];
            tile += (s_size[c] + kTP - 1) / kTP;
        }
        s_tile0[C] = tile;
        bucket_tile[C] = tile;
        plan[0] = tile;
    }
    __syncthreads();
    for (int t = tid; t < s_tile0[C]; t += kPlanThreads) {
        int c = 0;
        while (t >= s_tile0[c + 1]) ++c;
        const int o = (t - s_tile0[c]) * kTP;
        tile_start[t] = s_base[c] + o;
        tile_count[t] = min(kTP, s_size[c] - o);
        tile_bucket[t] = c;
    }
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
    const size_t smem = (size_t)C * kPlanThreads * sizeof(int32_t);
    static bool opted[64] = {};  // more than 48 KB of dynamic shared memory needs the opt-in, once per device
    int dev = 0;
    NNUE_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !opted[dev]) {
        NNUE_CUDA_TRY(cudaFuncSetAttribute(k_ls_plan, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kMaxBuckets * kPlanThreads * (int)sizeof(int32_t)));
        if (dev >= 0 && dev < 64) opted[dev] = true;
    }
    k_ls_plan<<<1, kPlanThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        bucket, B, C, static_cast<int32_t*>(plan), status);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
