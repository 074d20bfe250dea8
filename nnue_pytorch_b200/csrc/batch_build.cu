// Device-side construction of a training batch from packed positions.
//
// The reference builds `SparseBatch` on CPU worker threads
// (data_loader/cpp/training_data_loader.cpp:29-73: us/them, outcome, score,
// the two active-index lists, the piece-count bucket) and ships the expanded
// lists to the GPU (data_loader/_native.py:48-96).  Here the host ships
// 72 bytes per position and one warp per position expands them on the GPU
// with the HalfKAv2_hm index formula (model/modules/features/halfka_v2_hm.py:8-36):
// lane = piece slot, both perspectives, lists written in slot order and
// padded with -1 on the right, exactly the lists the feature-transformer
// kernels take.
#include "common.cuh"

namespace nnue {

static_assert(sizeof(nnue_packed_position) == 72, "packed position is 72 bytes");

constexpr int kPlanesNative = 12 * 64;  // 768 rows per king bucket, kings on planes 10 and 11
constexpr int kPlanesFlat = 11 * 64;    // 704 rows per king bucket, both kings on plane 10
constexpr int kRealFlat = 32 * kPlanesFlat;

// King bucket of the oriented king square (files e-h after the mirror).
__device__ __forceinline__ int king_bucket(int osq) { return (7 - (osq >> 3)) * 4 + (7 - (osq & 7)); }

__global__ void __launch_bounds__(kThreads)
    k_batch_build(const nnue_packed_position* __restrict__ pos, int64_t B, int layout, int K,
                  int32_t* __restrict__ white, int32_t* __restrict__ black, float* __restrict__ us,
                  float* __restrict__ them, float* __restrict__ outcome, float* __restrict__ score,
                  int64_t* __restrict__ piece_count, int64_t* __restrict__ bucket_idx,
                  unsigned long long* status) {
    const int lane = threadIdx.x & 31;
    const int64_t p = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (p >= B) return;
    const nnue_packed_position* rec = pos + p;
    // 72-byte records are 8-byte aligned: the tail is one 64-bit load
    const unsigned long long tail = __ldg(reinterpret_cast<const unsigned long long*>(rec) + 8);
    const int sc = (int)(short)(tail & 0xffff);
    const int outcome2 = (int)((tail >> 16) & 0xff);
    const int stm_white = (int)((tail >> 24) & 0xff);
    int count = (int)((tail >> 32) & 0xff);
    const unsigned v = __ldg(reinterpret_cast<const unsigned short*>(rec) + lane);
    const int sq = v & 63, type = (v >> 6) & 7, is_white = (v >> 9) & 1;

    bool good = count >= 2 && count <= 32 && outcome2 <= 2;
    const bool live = lane < count;
    good = good && !__any_sync(kFullMask, live && (type < 1 || type > 6));
    const unsigned wk = __ballot_sync(kFullMask, live && type == 6 && is_white);
    const unsigned bk = __ballot_sync(kFullMask, live && type == 6 && !is_white);
    good = good && __popc(wk) == 1 && __popc(bk) == 1;  // one king each
    if (!good) {
        if (lane == 0) note_bad_index(status);
        count = 0;  // the position keeps its targets but activates nothing
    }
    const int ksq_w = __shfl_sync(kFullMask, sq, good ? __ffs(wk) - 1 : 0);
    const int ksq_b = __shfl_sync(kFullMask, sq, good ? __ffs(bk) - 1 : 0);

#pragma unroll
    for (int persp = 0; persp < 2; ++persp) {  // 0 = white's point of view
        const int ksq = persp == 0 ? ksq_w : ksq_b;
        const int flip = ((ksq & 7) < 4 ? 7 : 0) ^ (persp == 0 ? 0 : 56);
        const int osq = sq ^ flip;
        const int kb = king_bucket(ksq ^ flip);
        const int theirs = (is_white != (persp == 0)) ? 1 : 0;
        int32_t* out = (persp == 0 ? white : black) + p * K;
        if (layout == NNUE_LAYOUT_NATIVE) {
            const int idx = osq + ((type - 1) * 2 + theirs) * 64 + kb * kPlanesNative;
            for (int j = lane; j < K; j += 32) out[j] = (j < count) ? idx : -1;
        } else {
            const int within = (type == 6 ? 10 : (type - 1) * 2 + theirs) * 64 + osq;
            const int real = within + kb * kPlanesFlat;
            const int virt = within + kRealFlat;
            // list = the count real rows, then the count matching factor rows
            for (int j0 = 0; j0 < K; j0 += 32) {
                const int j = j0 + lane;
                const int from_real = __shfl_sync(kFullMask, real, j & 31);
                const int from_virt = __shfl_sync(kFullMask, virt, (j - count) & 31);
                if (j < K) out[j] = (j < count) ? from_real : (j < 2 * count ? from_virt : -1);
            }
        }
    }
    if (lane == 0) {
        const float u = stm_white ? 1.f : 0.f;
        us[p] = u;
        them[p] = 1.f - u;
        outcome[p] = 0.5f * (float)min(outcome2, 2);
        score[p] = (float)sc;
        const int n = (int)((tail >> 32) & 0xff);
        if (piece_count) piece_count[p] = n;
        if (bucket_idx) bucket_idx[p] = n > 0 ? (n - 1) / 4 : 0;
    }
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_batch_build_halfka(const nnue_packed_position* positions, int64_t B, int32_t layout,
                                       int32_t K, int32_t* white_idx, int32_t* black_idx, float* us,
                                       float* them, float* outcome, float* score, int64_t* piece_count,
                                       int64_t* bucket_idx, void* stream) {
    NNUE_REQUIRE(layout == NNUE_LAYOUT_NATIVE || layout == NNUE_LAYOUT_FLAT, NNUE_ERR_ARG,
                 "nnue_batch_build_halfka: unknown layout %d", layout);
    const int need = layout == NNUE_LAYOUT_NATIVE ? 32 : 64;
    NNUE_REQUIRE(B >= 0 && K >= need, NNUE_ERR_ARG,
                 "nnue_batch_build_halfka: K=%d is too small for this layout (needs %d)", K, need);
    if (B == 0) return NNUE_OK;
    NNUE_REQUIRE(positions && white_idx && black_idx && us && them && outcome && score, NNUE_ERR_ARG,
                 "nnue_batch_build_halfka: null pointer");
    NNUE_REQUIRE((reinterpret_cast<uintptr_t>(positions) & 7u) == 0, NNUE_ERR_ALIGN,
                 "nnue_batch_build_halfka: positions must be 8-byte aligned");
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status != nullptr, NNUE_ERR_CUDA, "nnue_batch_build_halfka: no device status word");
    const unsigned grid = (unsigned)((B + kWarpsPerCta - 1) / kWarpsPerCta);
    k_batch_build<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        positions, B, layout, K, white_idx, black_idx, us, them, outcome, score, piece_count, bucket_idx,
        status);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
