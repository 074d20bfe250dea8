// First layer of the bucketed layer stack on the 5th-generation tensor cores:
//   o1[p, :] = W1[bucket(p)] . x[p] + b1[bucket(p)]         (32 outputs, K = L1)
// for inputs that TF32 holds exactly.  With fake quantization on, x is q / 128
// with q <= 127 and W1 is k / 128 (model/quantize.py:36-56 and
// model/modules/stacked_linear.py:96-127 of the reference project): both fit the
// 11 significant bits of TF32, every product is exact and so is every partial
// sum below 2^24 / 16384 = 1024, so one tcgen05.mma pass with fp32 accumulation in
// tensor memory returns the bits of the fp32 FMA kernel.  Other inputs would be
// truncated to TF32: the host side takes this path only for the quantized model.
//
// One CTA per tile of the batch plan (64 positions of one bucket, gathered rows
// of x).  The K loop walks chunks of 32 floats through a ring of shared-memory
// stages: all threads copy their 16-byte pieces with cp.async straight into the
// 128-byte-swizzled K-major layout the matrix descriptors name, one thread issues
// four tcgen05.mma (M = 128, N = 32, K = 8) per stage and commits them to the
// stage's mbarrier, which frees the stage for a later copy: the copy of chunk
// c + kTcAhead waits for the instructions of chunk c - kTcLag, issued kTcLag
// iterations earlier, so their latency stays off the loop's critical path.  The instruction is
// M = 128 (rows = TMEM lanes, one per position); rows 64..127 multiply whatever
// follows the tile in shared memory and are never read back.  The accumulator
// (128 lanes x 32 columns of tensor memory) comes back with tcgen05.ld, one
// position per thread.  Every wait is bounded: a wait that runs out raises the
// device status word, the CTA frees its tensor memory and leaves its tile unwritten.
#include "layer_stack.cuh"

namespace nnue {

constexpr int kTcStages = 8;                      // ring of shared-memory stages
constexpr int kTcLag = 3;                         // chunks whose tcgen05.mma may still be running when the next is issued
constexpr int kTcAhead = kTcStages - kTcLag;      // chunks whose copies are in flight
constexpr int kTcK = 32;                          // floats per stage along K: one 128-byte swizzle row
constexpr int kTcABytes = kTP * 128;              // 8 KiB: 64 positions x 128 B
constexpr int kTcBBytes = kLsOut * 128;           // 4 KiB: 32 outputs x 128 B
constexpr int kTcStageBytes = kTcABytes + kTcBBytes;
constexpr int kTcTailBytes = 128 * 128 - kTcStageBytes;  // what an M = 128 read of the last stage reaches beyond it
constexpr int kTcBarBytes = 16 * ((8 * (kTcStages + 1) + 15) / 16);  // one mbarrier per stage and one for the tile
constexpr int kTcSmemBytes = 1024 + kTcStages * kTcStageBytes + kTcTailBytes + kTcBarBytes;
constexpr int kTcThreads = 128;
constexpr int kTcCols = 32;                       // TMEM columns: the 32 outputs

__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    // K-major operand, 128-byte swizzle: rows of 128 B, groups of 8 rows 1024 B apart
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4)   // start address, 16-byte units
           | ((uint64_t)1 << 16)                    // leading byte offset: unused with this layout
           | ((uint64_t)(1024 >> 4) << 32)          // stride byte offset between 8-row groups
           | ((uint64_t)1 << 46)                    // descriptor version of this architecture
           | ((uint64_t)2 << 61);                   // layout type: 128-byte swizzle
}

// kind::tf32, D = F32, A and B TF32 and K-major, N = 32, M = 128
constexpr uint32_t kIdescTf32 = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kLsOut >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kIdescTf32), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__global__ void __launch_bounds__(kTcThreads)
    k_ls_l1_fwd_tc(const float* __restrict__ x, const float* __restrict__ W1, const float* __restrict__ b1,
                   LsPlanView plan, float* __restrict__ o1, int L1, unsigned long long* status) {
    extern __shared__ unsigned char smem_raw[];
    const int t = blockIdx.x;
    if (t >= *plan.n_tiles) return;
    const int cnt = plan.tile_count[t], bk = plan.tile_bucket[t];
    const int32_t* perm = plan.perm + plan.tile_start[t];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // stages at a 1024-byte boundary (the swizzle pattern repeats every 1024 B), barriers behind them
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* stage0 = smem_raw + (base - smem_u32(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(stage0 + kTcStages * kTcStageBytes + kTcTailBytes);
    uint64_t* bar_free = bars;               // [kTcStages]: the MMAs that read the stage have finished
    uint64_t* bar_done = bars + kTcStages;   // all MMAs of the tile have finished
    __shared__ uint32_t s_tmem;

    if (tid == 0) {
        for (int s = 0; s < kTcStages; ++s) mbar_init(bar_free + s, 1);
        mbar_init(bar_done, 1);
        fence_barrier_init();
    }
    if (warp == 0) {  // tensor memory for the accumulator: 32 columns, allocated by one whole warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(kTcCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    // copy plan: 16-byte piece q of row r lands at r * 128 + ((q ^ (r & 7)) * 16) inside its 1024-byte group
    // A: 64 rows x 8 pieces = 512 pieces, four per thread; B: 32 rows x 8 pieces, two per thread
    const float* a_src[4];
    uint32_t a_dst[4];
    bool a_live[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int piece = tid + kTcThreads * i, r = piece >> 3, q = piece & 7;
        a_live[i] = r < cnt;
        a_src[i] = x + (int64_t)(a_live[i] ? perm[r] : 0) * L1 + 4 * q;
        a_dst[i] = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((q ^ (r & 7)) << 4));
    }
    const float* b_src[2];
    uint32_t b_dst[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int piece = tid + kTcThreads * i, r = piece >> 3, q = piece & 7;
        b_src[i] = W1 + ((int64_t)bk * kLsOut + r) * L1 + 4 * q;
        b_dst[i] = (uint32_t)(kTcABytes + (r >> 3) * 1024 + (r & 7) * 128 + ((q ^ (r & 7)) << 4));
    }
    const int chunks = L1 / kTcK;
    auto issue = [&](int c) {  // chunk c into stage c % kTcStages; past the end: an empty group
        if (c < chunks) {
            unsigned char* st = stage0 + (c % kTcStages) * kTcStageBytes;
#pragma unroll
            for (int i = 0; i < 4; ++i) cp_async16(st + a_dst[i], a_src[i] + c * kTcK, a_live[i]);
#pragma unroll
            for (int i = 0; i < 2; ++i) cp_async16(st + b_dst[i], b_src[i] + c * kTcK, true);
        }
        cp_async_commit();
    };

    bool failed = false;
#pragma unroll
    for (int c = 0; c < kTcAhead; ++c) issue(c);
    for (int c = 0; c < chunks; ++c) {
        cp_async_wait<kTcAhead - 1>();                                    // this thread's pieces of chunk c are in
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // ... and visible to the tensor core's reads
        __syncthreads();                                                  // ... and so are everybody's
        if (tid == 0 && !failed) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = base + (uint32_t)((c % kTcStages) * kTcStageBytes);
            const uint64_t a_desc = umma_desc_k_sw128(a_addr), b_desc = umma_desc_k_sw128(a_addr + kTcABytes);
#pragma unroll
            for (int k = 0; k < kTcK / 8; ++k)  // 32 bytes along K per instruction: +2 in 16-byte units
                umma_tf32(tmem, a_desc + 2 * k, b_desc + 2 * k, (c | k) != 0);
            umma_commit(bar_free + c % kTcStages);
            if (c == chunks - 1) umma_commit(bar_done);
        }
        // the stage chunk c + kTcAhead goes into was read by the MMAs of chunk c - kTcLag
        const int next = c + kTcAhead;
        if (next < chunks && c >= kTcLag) {
            const int s = (c - kTcLag) % kTcStages;
            if (!mbar_wait_bounded(bar_free + s, (unsigned)(((c - kTcLag) / kTcStages) & 1))) failed = true;
        }
        if (__syncthreads_or(failed)) {  // one decision for the CTA
            failed = true;
            break;
        }
        issue(next);
    }
    cp_async_wait<0>();
    if (!failed && !mbar_wait_bounded(bar_done, 0)) failed = true;
    failed = __syncthreads_or(failed);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    if (!failed && warp < kTP / 32) {  // lanes 0..63 of the accumulator are the tile's positions
        uint32_t v[32];
        const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
              "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
              "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int pos = warp * 32 + lane;
        if (pos < cnt) {
            float4* dst = reinterpret_cast<float4*>(o1 + (int64_t)perm[pos] * kLsOut);
            const float4* bias = reinterpret_cast<const float4*>(b1 + bk * kLsOut);
#pragma unroll
            for (int j = 0; j < kLsOut / 4; ++j) {
                const float4 b = __ldg(bias + j);
                dst[j] = make_float4(__fadd_rn(__uint_as_float(v[4 * j]), b.x), __fadd_rn(__uint_as_float(v[4 * j + 1]), b.y),
                                     __fadd_rn(__uint_as_float(v[4 * j + 2]), b.z), __fadd_rn(__uint_as_float(v[4 * j + 3]), b.w));
            }
        }
    }
    if (failed && tid == 0) note_timeout(status);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTcCols) : "memory");
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_ls_l1_fwd_tc(const float* x, const float* W1, const float* b1, const void* plan, float* o1,
                                 int64_t B, int32_t L1, int32_t C, void* stream) {
    NNUE_REQUIRE(B >= 0 && L1 > 0 && L1 % kTcK == 0 && C > 0 && C <= 16, NNUE_ERR_UNSUPPORTED,
                 "nnue_ls_l1_fwd_tc: needs L1 %% 32 == 0 and 1..16 buckets (B=%lld L1=%d C=%d)", (long long)B, L1, C);
    NNUE_REQUIRE(plan != nullptr && aligned16(plan), NNUE_ERR_ARG, "nnue_ls_l1_fwd_tc: null or unaligned plan");
    if (B == 0) return NNUE_OK;
    NNUE_REQUIRE(x && W1 && b1 && o1 && aligned16(x) && aligned16(W1) && aligned16(o1) && aligned16(b1), NNUE_ERR_ARG,
                 "nnue_ls_l1_fwd_tc: null or unaligned tensor");
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "nnue_ls_l1_fwd_tc: no device status word");
    static bool done[64] = {false};
    int dev = -1;
    NNUE_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !done[dev]) {
        NNUE_CUDA_TRY(cudaFuncSetAttribute(k_ls_l1_fwd_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes));
        if (dev >= 0 && dev < 64) done[dev] = true;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ProfScope prof("k_ls_l1_fwd_tc", s);
    k_ls_l1_fwd_tc<<<(unsigned)ls_max_tiles(B, C), kTcThreads, kTcSmemBytes, s>>>(x, W1, b1, ls_view(plan, B, C), o1, L1,
                                                                                  status);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
