// Data-parallel exchange of the feature-transformer table fused with the
// optimizer, over peer memory (NVLink / NVSwitch), one process per GPU.
//
// The reference wraps the model in DistributedDataParallel
// (trainer/engine.py:149-162 of the reference project): every rank receives
// the full averaged gradient (286 MB all-reduce) and every rank then updates
// the whole table.  Here each rank owns a contiguous shard of table rows:
//
//   k_ddp_reduce_shard   reads its shard of the gradient from EVERY rank's
//                        buffer with plain peer loads, adds in rank order,
//                        keeps the sum in its own buffer and accumulates the
//                        squared norm   (reduce-scatter + norm, one kernel)
//   k_ddp_update_shard   RangerLite on the shard (moments exist for the shard
//                        only) and stores the new rows into EVERY rank's
//                        table with plain peer stores
//                                          (optimizer + all-gather, one kernel)
//
// No kernel waits on another GPU: ordering between ranks comes from the tiny
// NCCL collectives the host issues between the phases (a collective cannot
// complete before every rank has reached it on its stream).  No multicast
// loads, no multimem: plain ld/st on peer pointers only.
#include <algorithm>

#include "ranger.cuh"

namespace nnue {

constexpr int kMaxRanks = 16;

struct PeerPtrs {
    float* p[kMaxRanks];
};

// Per-CTA partial norms of the reduce kernel (file scope: reduce launches of one device are ordered
// on one stream by the exchange).
constexpr int kReduceMaxGrid = 2048;
__device__ float g_reduce_partial[kReduceMaxGrid];
__device__ unsigned int g_reduce_arrived;

// UN float4 per thread and trip, every rank's copy of them loaded before the first add: with few
// ranks (few loads per float4) the unroll keeps enough bytes in flight to fill the links even when
// the grid is capped to leave SMs to a kernel running beside it.
// WMAX bounds the world size of the instantiation (registers: UN * WMAX float4).
template <int UN, int WMAX>
__global__ void __launch_bounds__(kThreads)
    k_ddp_reduce_shard(PeerPtrs grads, int world, int rank, int64_t beg4, int64_t end4,
                       float* __restrict__ sumsq) {
    __shared__ float s_w[kWarpsPerCta];
    __shared__ bool s_last;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    float acc = 0.f;
    for (int64_t i0 = beg4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < end4; i0 += stride * UN) {
        float4 v[UN][WMAX];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int64_t i = i0 + u * stride;
#pragma unroll
            for (int r = 0; r < WMAX; ++r)
                if (r < world && i < end4) v[u][r] = __ldcs(reinterpret_cast<const float4*>(grads.p[r]) + i);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int64_t i = i0 + u * stride;
            if (i >= end4) break;
            float4 s = v[u][0];
#pragma unroll
            for (int r = 1; r < WMAX; ++r)
                if (r < world) s = f4_add(s, v[u][r]);
            reinterpret_cast<float4*>(grads.p[rank])[i] = s;
            acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
        }
    }
    // reproducible norm: a slot per CTA, the CTA that arrives last adds the slots in index order
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(kFullMask, acc, d);
    if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < kWarpsPerCta; ++w) t += s_w[w];
        g_reduce_partial[blockIdx.x] = t;
        __threadfence();
        s_last = atomicAdd(&g_reduce_arrived, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float tot = 0.f;
    for (unsigned i = threadIdx.x; i < gridDim.x; i += kThreads) tot += __ldcg(&g_reduce_partial[i]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) tot += __shfl_xor_sync(kFullMask, tot, d);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = tot;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < kWarpsPerCta; ++w) t += s_w[w];
        *sumsq += t;
        g_reduce_arrived = 0;
    }
}

// Moment tensors are shard-sized: element i of the table is element i - beg4 of them.
__global__ void __launch_bounds__(kThreads)
    k_ddp_update_shard(PeerPtrs tables, int world, int rank, int64_t beg4, int64_t end4,
                       const float* __restrict__ grad, float* __restrict__ gm, float* __restrict__ ngm,
                       float* __restrict__ vm, float* __restrict__ slow,
                       const float* __restrict__ d_scale, RangerConst c) {
    const float scale = d_scale ? __ldg(d_scale) : 1.f;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const float4* g4 = reinterpret_cast<const float4*>(grad);
    float4* own = reinterpret_cast<float4*>(tables.p[rank]);
    float4* gm4 = reinterpret_cast<float4*>(gm);
    float4* ngm4 = reinterpret_cast<float4*>(ngm);
    float4* vm4 = reinterpret_cast<float4*>(vm);
    float4* slow4 = reinterpret_cast<float4*>(slow);
    for (int64_t i = beg4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < end4; i += stride) {
        const int64_t j = i - beg4;
        const float4 gv = __ldcs(g4 + i);
        float4 pv = own[i], gmv = gm4[j], vmv = vm4[j];
        float4 ngv = c.use_pnm ? ngm4[j] : f4_zero();
        float4 sv = c.do_merge ? slow4[j] : f4_zero();
        ranger_elem(c, scale, gv.x, pv.x, gmv.x, ngv.x, vmv.x, sv.x);
        ranger_elem(c, scale, gv.y, pv.y, gmv.y, ngv.y, vmv.y, sv.y);
        ranger_elem(c, scale, gv.z, pv.z, gmv.z, ngv.z, vmv.z, sv.z);
        ranger_elem(c, scale, gv.w, pv.w, gmv.w, ngv.w, vmv.w, sv.w);
        vm4[j] = vmv;
        if (!c.use_pnm || c.step_is_odd) gm4[j] = gmv;
        if (c.use_pnm && !c.step_is_odd) ngm4[j] = ngv;
        if (c.do_merge) slow4[j] = sv;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < world) reinterpret_cast<float4*>(tables.p[r])[i] = pv;
    }
}

}  // namespace nnue

using namespace nnue;

static int check_shard(const char* who, const void* const* ptrs, int world, int rank, int64_t beg,
                       int64_t end) {
    NNUE_REQUIRE(ptrs != nullptr, NNUE_ERR_ARG, "%s: null pointer table", who);
    NNUE_REQUIRE(world >= 1 && world <= kMaxRanks, NNUE_ERR_UNSUPPORTED, "%s: world size %d outside 1..%d",
                 who, world, kMaxRanks);
    NNUE_REQUIRE(rank >= 0 && rank < world, NNUE_ERR_ARG, "%s: rank %d outside the world", who, rank);
    NNUE_REQUIRE(beg >= 0 && end >= beg && beg % 4 == 0 && end % 4 == 0, NNUE_ERR_ARG,
                 "%s: shard [%lld, %lld) must be a non-negative range of whole float4", who, (long long)beg,
                 (long long)end);
    for (int r = 0; r < world; ++r)
        NNUE_REQUIRE(ptrs[r] != nullptr && aligned16(ptrs[r]), NNUE_ERR_ALIGN,
                     "%s: buffer of rank %d is null or not 16-byte aligned", who, r);
    return NNUE_OK;
}

extern "C" int nnue_ddp_reduce_shard(float* const* h_grad_ptrs, int32_t world, int32_t rank,
                                     int64_t elem_begin, int64_t elem_end, float* d_sumsq,
                                     void* stream) {
    int rc = check_shard("nnue_ddp_reduce_shard", reinterpret_cast<const void* const*>(h_grad_ptrs), world,
                         rank, elem_begin, elem_end);
    if (rc != NNUE_OK) return rc;
    NNUE_REQUIRE(d_sumsq != nullptr, NNUE_ERR_ARG, "nnue_ddp_reduce_shard: null norm accumulator");
    if (elem_end == elem_begin) return NNUE_OK;
    PeerPtrs pp{};
    for (int r = 0; r < world; ++r) pp.p[r] = h_grad_ptrs[r];
    const int64_t n4 = (elem_end - elem_begin) / 4;
    const int cap = std::min(kReduceMaxGrid, tuning().ddp_reduce_ctas > 0 ? tuning().ddp_reduce_ctas : sm_count() * 8);
    const unsigned grid = (unsigned)std::min<int64_t>((n4 + kThreads - 1) / kThreads, (int64_t)cap);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (world <= 2)
        k_ddp_reduce_shard<4, 2><<<grid, kThreads, 0, s>>>(pp, world, rank, elem_begin / 4, elem_end / 4, d_sumsq);
    else if (world <= 4)
        k_ddp_reduce_shard<2, 4><<<grid, kThreads, 0, s>>>(pp, world, rank, elem_begin / 4, elem_end / 4, d_sumsq);
    else if (world <= 8)
        k_ddp_reduce_shard<2, 8><<<grid, kThreads, 0, s>>>(pp, world, rank, elem_begin / 4, elem_end / 4, d_sumsq);
    else
        k_ddp_reduce_shard<1, kMaxRanks><<<grid, kThreads, 0, s>>>(pp, world, rank, elem_begin / 4, elem_end / 4,
                                                                  d_sumsq);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

extern "C" int nnue_ddp_update_shard(float* const* h_table_ptrs, int32_t world, int32_t rank,
                                     int64_t elem_begin, int64_t elem_end, const float* grad,
                                     float* grad_ma, float* neg_grad_ma, float* variance_ma, float* slow,
                                     const float* d_grad_scale, const nnue_ranger_hparams* hp,
                                     void* stream) {
    int rc = check_shard("nnue_ddp_update_shard", reinterpret_cast<const void* const*>(h_table_ptrs), world,
                         rank, elem_begin, elem_end);
    if (rc != NNUE_OK) return rc;
    NNUE_REQUIRE(hp != nullptr && hp->phase == 0, NNUE_ERR_ARG,
                 "nnue_ddp_update_shard: needs hyper-parameters of a full (phase 0) update");
    if (elem_end == elem_begin) return NNUE_OK;
    NNUE_REQUIRE(grad && grad_ma && variance_ma && aligned16(grad) && aligned16(grad_ma) &&
                     aligned16(variance_ma),
                 NNUE_ERR_ARG, "nnue_ddp_update_shard: null or unaligned tensor");
    NNUE_REQUIRE(!hp->use_pnm || (neg_grad_ma && aligned16(neg_grad_ma)), NNUE_ERR_ARG,
                 "nnue_ddp_update_shard: PNM needs neg_grad_ma");
    NNUE_REQUIRE(!hp->do_merge || (slow && aligned16(slow)), NNUE_ERR_ARG,
                 "nnue_ddp_update_shard: merge needs the slow copy");
    PeerPtrs pp{};
    for (int r = 0; r < world; ++r) pp.p[r] = h_table_ptrs[r];
    const int64_t n4 = (elem_end - elem_begin) / 4;
    const unsigned grid = (unsigned)std::min<int64_t>((n4 + kThreads - 1) / kThreads, (int64_t)sm_count() * 8);
    k_ddp_update_shard<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        pp, world, rank, elem_begin / 4, elem_end / 4, grad, grad_ma, neg_grad_ma, variance_ma, slow,
        d_grad_scale, *hp);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
