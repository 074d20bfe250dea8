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
//   k_ddp_reduce_block   the same over a column slice of its rows (the
//                        backward can deliver the gradient in column slices)
//   k_ddp_update_shard   RangerLite on the shard (moments exist for the shard
//                        only) and stores into EVERY rank's memory, with plain
//                        peer stores, what the ranks read next: the fp32 rows,
//                        or the int16 / PSQT rows of the table their forward
//                        gathers (half the bytes; the fp32 rows then stay home)
//                                          (optimizer + all-gather, one kernel)
//   k_ddp_publish_stats  this rank's range statistics of its int16 rows into
//                        a slot of every rank's statistics array
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

// The same reduce over a 2-D block of the [rows, W4] gradient: rows [row0, row0 + n_rows), float4 columns
// [c40, c40 + cols4) (a column slice of this rank's rows).  Linear index i of the block -> row i / cols4.
template <int UN, int WMAX>
__global__ void __launch_bounds__(kThreads)
    k_ddp_reduce_block(PeerPtrs grads, int world, int rank, unsigned row0, unsigned n4, unsigned cols4, unsigned c40,
                       unsigned W4, float* __restrict__ sumsq) {
    __shared__ float s_w[kWarpsPerCta];
    __shared__ bool s_last;
    const unsigned stride = gridDim.x * blockDim.x;
    float acc = 0.f;
    auto at = [&](unsigned i) -> int64_t {
        const unsigned r = i / cols4;
        return (int64_t)(row0 + r) * W4 + c40 + (i - r * cols4);
    };
    for (unsigned i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += stride * UN) {
        float4 v[UN][WMAX];
        int64_t idx[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const unsigned i = i0 + u * stride;
            idx[u] = i < n4 ? at(i) : -1;
#pragma unroll
            for (int r = 0; r < WMAX; ++r)
                if (r < world && idx[u] >= 0) v[u][r] = __ldcs(reinterpret_cast<const float4*>(grads.p[r]) + idx[u]);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            if (idx[u] < 0) break;
            float4 s = v[u][0];
#pragma unroll
            for (int r = 1; r < WMAX; ++r)
                if (r < world) s = f4_add(s, v[u][r]);
            reinterpret_cast<float4*>(grads.p[rank])[idx[u]] = s;
            acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
        }
    }
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

// What the update kernel sends to the other ranks besides (or instead of) the fp32 rows: the rows of the
// integer table their forward gathers (nnue_ft_quantize_table's format).  Half the bytes over NVLink when the
// fp32 rows stay with their owner.
struct PeerEmit {
    int16_t* q16[kMaxRanks];
    float* psqt[kMaxRanks];
    int* stats_local;      // this rank's [overflow count, max |k|] of its share, accumulated over the step
    long long pitch4;      // q16 row pitch in groups of four int16
    int w4, l4, p4;        // float4 per table row, of them L1 part and PSQT part
    float scale_main, scale_psqt;
};

// Moment tensors are shard-sized: element i of the table is element i - beg4 of them.
// FP32_TO_PEERS: the new rows go into every rank's table (else only into the owner's).  EMIT: see PeerEmit.
// IDX = unsigned when the float4 indices (plus one grid stride) fit 32 bits.  The other ranks' pointers sit in shared
// memory and the stores to them are short rolled loops: the kernel then needs as few registers as the single-GPU
// update (it measured a quarter slower with the pointers in unrolled, predicated loops: fewer warps per SM).
template <bool FP32_TO_PEERS, bool EMIT, typename IDX>
__global__ void __launch_bounds__(kThreads)
    k_ddp_update_shard(PeerPtrs tables, int world, int rank, int64_t beg4_, int64_t end4_,
                       const float* __restrict__ grad, float* __restrict__ gm, float* __restrict__ ngm,
                       float* __restrict__ vm, float* __restrict__ slow,
                       const float* __restrict__ d_scale, RangerConst c, PeerEmit pe) {
    __shared__ float4* s_tab[kMaxRanks];
    __shared__ int2* s_q16[kMaxRanks];
    __shared__ float4* s_psqt[kMaxRanks];
    if (threadIdx.x < kMaxRanks) {
        s_tab[threadIdx.x] = reinterpret_cast<float4*>(tables.p[threadIdx.x]);
        s_q16[threadIdx.x] = reinterpret_cast<int2*>(pe.q16[threadIdx.x]);
        s_psqt[threadIdx.x] = reinterpret_cast<float4*>(pe.psqt[threadIdx.x]);
    }
    __syncthreads();
    int bad = 0, max_abs = 0;
    const float scale = d_scale ? __ldg(d_scale) : 1.f;
    const IDX beg4 = (IDX)beg4_, end4 = (IDX)end4_;
    const IDX stride = (IDX)gridDim.x * blockDim.x;
    const float4* g4 = reinterpret_cast<const float4*>(grad);
    float4* own = s_tab[rank];
    float4* gm4 = reinterpret_cast<float4*>(gm);
    float4* ngm4 = reinterpret_cast<float4*>(ngm);
    float4* vm4 = reinterpret_cast<float4*>(vm);
    float4* slow4 = reinterpret_cast<float4*>(slow);
    for (IDX i = beg4 + (IDX)blockIdx.x * blockDim.x + threadIdx.x; i < end4; i += stride) {
        const IDX j = i - beg4;
        const float4 gv = __ldg(g4 + i);
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
        if (FP32_TO_PEERS) {
#pragma unroll 1
            for (int r = 0; r < world; ++r) s_tab[r][i] = pv;
        } else {
            own[i] = pv;
        }
        if (EMIT) {
            const unsigned row = (unsigned)i / (unsigned)pe.w4;  // the host checked that the index fits 31 bits
            const int c4 = (int)((unsigned)i - row * (unsigned)pe.w4);
            if (c4 < pe.l4) {
                const float x[4] = {pv.x, pv.y, pv.z, pv.w};
                int k[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float rr = rintf(__fmul_rn(x[q], pe.scale_main));
                    if (!(fabsf(rr) <= 32767.f)) {
                        ++bad;
                        rr = fminf(fmaxf(rr, -32767.f), 32767.f);
                        if (rr != rr) rr = 0.f;
                    }
                    k[q] = (int)rr;
                    max_abs = max(max_abs, abs(k[q]));
                }
                const int2 words = make_int2(k[1] * 65536 + k[0], k[3] * 65536 + k[2]);
                const long long at = (long long)row * pe.pitch4 + c4;
#pragma unroll 1
                for (int r = 0; r < world; ++r) s_q16[r][at] = words;
            } else {
                auto fq = [&](float a) { return __fdiv_rn(rintf(__fmul_rn(a, pe.scale_psqt)), pe.scale_psqt); };
                const float4 v = make_float4(fq(pv.x), fq(pv.y), fq(pv.z), fq(pv.w));
                const long long at = (long long)row * pe.p4 + (c4 - pe.l4);
#pragma unroll 1
                for (int r = 0; r < world; ++r) s_psqt[r][at] = v;
            }
        }
    }
    if (EMIT) {
        if (bad) atomicAdd(pe.stats_local, bad);
        max_abs = __reduce_max_sync(kFullMask, max_abs);
        if ((threadIdx.x & 31) == 0 && max_abs > 0) atomicMax(pe.stats_local + 1, max_abs);
    }
}

// This rank's range statistics into slot `rank` of every rank's statistics array.
struct StatPtrs {
    int* p[kMaxRanks];
};
__global__ void k_ddp_publish_stats(StatPtrs all, int world, int rank, const int* __restrict__ local) {
    const int r = threadIdx.x;
    if (r < world) {
        all.p[r][2 * rank] = local[0];
        all.p[r][2 * rank + 1] = local[1];
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
    const int u = tuning().ddp_reduce_u;
#define LAUNCH_RED(UU, WW) \
    k_ddp_reduce_shard<UU, WW><<<grid, kThreads, 0, s>>>(pp, world, rank, elem_begin / 4, elem_end / 4, d_sumsq)
    ProfScope prof("k_ddp_reduce_shard", s);
    if (world <= 2) {
        if (u == 8) LAUNCH_RED(8, 2);
        else if (u == 2) LAUNCH_RED(2, 2);
        else LAUNCH_RED(4, 2);
    } else if (world <= 4) {
        if (u == 4) LAUNCH_RED(4, 4);
        else if (u == 1) LAUNCH_RED(1, 4);
        else LAUNCH_RED(2, 4);
    } else if (world <= 8) {
        if (u == 4) LAUNCH_RED(4, 8);
        else if (u == 1) LAUNCH_RED(1, 8);
        else LAUNCH_RED(2, 8);
    } else {
        LAUNCH_RED(1, kMaxRanks);
    }
#undef LAUNCH_RED
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

extern "C" int nnue_ddp_reduce_block(float* const* h_grad_ptrs, int32_t world, int32_t rank, int64_t row_begin,
                                     int64_t row_end, int64_t col_begin, int64_t col_end, int64_t width,
                                     float* d_sumsq, void* stream) {
    int rc = check_shard("nnue_ddp_reduce_block", reinterpret_cast<const void* const*>(h_grad_ptrs), world, rank, 0, 0);
    if (rc != NNUE_OK) return rc;
    NNUE_REQUIRE(d_sumsq != nullptr, NNUE_ERR_ARG, "nnue_ddp_reduce_block: null norm accumulator");
    NNUE_REQUIRE(width > 0 && width % 4 == 0 && col_begin >= 0 && col_begin <= col_end && col_end <= width &&
                     col_begin % 4 == 0 && col_end % 4 == 0 && row_begin >= 0 && row_begin <= row_end,
                 NNUE_ERR_ARG, "nnue_ddp_reduce_block: bad block (whole float4 columns inside the row width)");
    const int64_t cols4 = (col_end - col_begin) / 4, n4 = (row_end - row_begin) * cols4;
    if (n4 == 0) return NNUE_OK;
    NNUE_REQUIRE(n4 < 0x7fffffffLL - (int64_t)kReduceMaxGrid * kThreads * 8 && row_end < 0x7fffffffLL && width / 4 < 0x7fffffffLL,
                 NNUE_ERR_UNSUPPORTED, "nnue_ddp_reduce_block: block too large for 32-bit indices");
    PeerPtrs pp{};
    for (int r = 0; r < world; ++r) pp.p[r] = h_grad_ptrs[r];
    const int cap = std::min(kReduceMaxGrid, tuning().ddp_reduce_ctas > 0 ? tuning().ddp_reduce_ctas : sm_count() * 8);
    const unsigned grid = (unsigned)std::min<int64_t>((n4 + kThreads - 1) / kThreads, (int64_t)cap);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int u = tuning().ddp_reduce_u;
#define LAUNCH_BLK(UU, WW)                                                                                          \
    k_ddp_reduce_block<UU, WW><<<grid, kThreads, 0, s>>>(pp, world, rank, (unsigned)row_begin, (unsigned)n4, (unsigned)cols4, \
                                                         (unsigned)(col_begin / 4), (unsigned)(width / 4), d_sumsq)
    ProfScope prof("k_ddp_reduce_block", s);
    if (world <= 2) {
        if (u == 8) LAUNCH_BLK(8, 2);
        else LAUNCH_BLK(4, 2);
    } else if (world <= 4) {
        if (u == 4) LAUNCH_BLK(4, 4);
        else LAUNCH_BLK(2, 4);
    } else if (world <= 8) {
        if (u == 4) LAUNCH_BLK(4, 8);
        else LAUNCH_BLK(2, 8);
    } else {
        LAUNCH_BLK(1, kMaxRanks);
    }
#undef LAUNCH_BLK
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

extern "C" int nnue_ddp_update_shard(float* const* h_table_ptrs, int32_t world, int32_t rank,
                                     int64_t elem_begin, int64_t elem_end, const float* grad,
                                     float* grad_ma, float* neg_grad_ma, float* variance_ma, float* slow,
                                     const float* d_grad_scale, const nnue_ranger_hparams* hp,
                                     void* stream) {
    return nnue_ddp_update_shard_emit(h_table_ptrs, world, rank, elem_begin, elem_end, grad, grad_ma, neg_grad_ma,
                                      variance_ma, slow, d_grad_scale, hp, nullptr, stream);
}

extern "C" int nnue_ddp_publish_stats(const nnue_ddp_emit* h_emit, int32_t world, int32_t rank, void* stream) {
    NNUE_REQUIRE(h_emit && h_emit->h_stats_ptrs && h_emit->d_stats_local, NNUE_ERR_ARG, "nnue_ddp_publish_stats: null pointer");
    NNUE_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, NNUE_ERR_ARG,
                 "nnue_ddp_publish_stats: bad world / rank");
    StatPtrs sp{};
    for (int r = 0; r < world; ++r) {
        NNUE_REQUIRE(h_emit->h_stats_ptrs[r] != nullptr, NNUE_ERR_ARG, "nnue_ddp_publish_stats: null statistics array");
        sp.p[r] = h_emit->h_stats_ptrs[r];
    }
    k_ddp_publish_stats<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(sp, world, rank, h_emit->d_stats_local);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

extern "C" int nnue_ddp_update_shard_emit(float* const* h_table_ptrs, int32_t world, int32_t rank,
                                          int64_t elem_begin, int64_t elem_end, const float* grad,
                                          float* grad_ma, float* neg_grad_ma, float* variance_ma, float* slow,
                                          const float* d_grad_scale, const nnue_ranger_hparams* hp,
                                          const nnue_ddp_emit* h_emit, void* stream) {
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
    PeerEmit pe{};
    bool fp32_to_peers = true;
    if (h_emit) {
        int e2 = 0;
        NNUE_REQUIRE(h_emit->h_q16_ptrs && h_emit->d_stats_local && (h_emit->h_psqt_ptrs || h_emit->P == 0), NNUE_ERR_ARG,
                     "nnue_ddp_update_shard_emit: null pointer");
        NNUE_REQUIRE(h_emit->L1 > 0 && h_emit->L1 % 8 == 0 && h_emit->P >= 0 && h_emit->P % 4 == 0 &&
                         h_emit->q16_pitch >= h_emit->L1 && h_emit->q16_pitch % 8 == 0,
                     NNUE_ERR_ARG, "nnue_ddp_update_shard_emit: bad table shape (L1 %% 8, P %% 4, pitch %% 8)");
        NNUE_REQUIRE(h_emit->scale_main > 0.f && frexpf(h_emit->scale_main, &e2) == 0.5f && h_emit->scale_psqt > 0.f,
                     NNUE_ERR_UNSUPPORTED, "nnue_ddp_update_shard_emit: the main scale must be a power of two");
        for (int r = 0; r < world; ++r) {
            NNUE_REQUIRE(h_emit->h_q16_ptrs[r] && aligned16(h_emit->h_q16_ptrs[r]) &&
                             (h_emit->P == 0 || (h_emit->h_psqt_ptrs[r] && aligned16(h_emit->h_psqt_ptrs[r]))),
                         NNUE_ERR_ALIGN, "nnue_ddp_update_shard_emit: table of rank %d is null or not 16-byte aligned", r);
            pe.q16[r] = h_emit->h_q16_ptrs[r];
            pe.psqt[r] = h_emit->P ? h_emit->h_psqt_ptrs[r] : nullptr;
        }
        NNUE_REQUIRE(elem_end / 4 < 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "nnue_ddp_update_shard_emit: table too large");
        pe.stats_local = h_emit->d_stats_local;
        pe.pitch4 = h_emit->q16_pitch / 4;
        pe.l4 = h_emit->L1 / 4;
        pe.p4 = h_emit->P / 4;
        pe.w4 = pe.l4 + pe.p4;
        pe.scale_main = h_emit->scale_main;
        pe.scale_psqt = h_emit->scale_psqt;
        fp32_to_peers = h_emit->fp32_to_peers != 0;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ProfScope prof("k_ddp_update_shard", s);
    const bool narrow = elem_end / 4 + (int64_t)grid * kThreads < 0x7fffffffLL;
#define LAUNCH_UPD(FF, EE)                                                                                        \
    do {                                                                                                          \
        if (narrow)                                                                                               \
            k_ddp_update_shard<FF, EE, unsigned><<<grid, kThreads, 0, s>>>(pp, world, rank, elem_begin / 4, elem_end / 4, grad, \
                                                                           grad_ma, neg_grad_ma, variance_ma, slow, d_grad_scale, *hp, pe); \
        else                                                                                                      \
            k_ddp_update_shard<FF, EE, int64_t><<<grid, kThreads, 0, s>>>(pp, world, rank, elem_begin / 4, elem_end / 4, grad,  \
                                                                          grad_ma, neg_grad_ma, variance_ma, slow, d_grad_scale, *hp, pe); \
    } while (0)
    if (!h_emit) LAUNCH_UPD(true, false);
    else if (fp32_to_peers) LAUNCH_UPD(true, true);
    else LAUNCH_UPD(false, true);
#undef LAUNCH_UPD
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
