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
// of x).  The K loop walks chunks of 64 floats (two operand blocks of one
// 128-byte swizzle row each) through a ring of shared-memory stages: all threads
// copy their 16-byte pieces with cp.async straight into the 128-byte-swizzled
// K-major layout the matrix descriptors name, one thread issues eight
// tcgen05.mma (M = 128, N = 32, K = 8) per stage and commits them to the
// stage's mbarrier, which frees the stage for a later copy.  A trip of the loop
// costs about 0.5 us whatever it moves (copy wait, proxy fence, two CTA
// barriers), so a trip covers two blocks (0.061 ms with one).  The instruction is
// M = 128 (rows = TMEM lanes, one per position); rows 64..127 multiply whatever
// follows the tile in shared memory and are never read back.  The accumulator
// (128 lanes x 32 columns of tensor memory) comes back with tcgen05.ld, one
// position per thread.  Every wait is bounded: a wait that runs out raises the
// device status word, the CTA frees its tensor memory and leaves its tile unwritten.
#include "layer_stack.cuh"

namespace nnue {

constexpr int kTcStages = 4;                      // ring of shared-memory stages
constexpr int kTcLag = 1;                         // chunks whose tcgen05.mma may still be running when the next is issued
constexpr int kTcAhead = kTcStages - kTcLag;      // chunks whose copies are in flight
constexpr int kTcK = 32;                          // floats along K per operand block: one 128-byte swizzle row
constexpr int kTcSub = 2;                         // operand blocks per stage: a stage (one trip of the loop, with its
                                                  // proxy fence and CTA barriers) covers 64 floats of K
constexpr int kTcABytes = kTP * 128;              // 8 KiB: 64 positions x 128 B
constexpr int kTcBBytes = kLsOut * 128;           // 4 KiB: 32 outputs x 128 B
constexpr int kTcBlockBytes = kTcABytes + kTcBBytes;
constexpr int kTcStageBytes = kTcSub * kTcBlockBytes;
constexpr int kTcTailBytes = 128 * 128 - kTcBlockBytes;  // what an M = 128 read of the last block reaches beyond it
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
    const int blocks = L1 / kTcK;                         // operand blocks of 32 floats of K
    const int chunks = (blocks + kTcSub - 1) / kTcSub;    // stages; the last one may hold fewer blocks
    auto issue = [&](int c) {  // chunk c into stage c % kTcStages; past the end: an empty group
        if (c < chunks) {
#pragma unroll
            for (int u = 0; u < kTcSub; ++u) {
                const int blk = c * kTcSub + u;
                if (blk < blocks) {
                    unsigned char* st = stage0 + (c % kTcStages) * kTcStageBytes + u * kTcBlockBytes;
#pragma unroll
                    for (int i = 0; i < 4; ++i) cp_async16(st + a_dst[i], a_src[i] + blk * kTcK, a_live[i]);
#pragma unroll
                    for (int i = 0; i < 2; ++i) cp_async16(st + b_dst[i], b_src[i] + blk * kTcK, true);
                }
            }
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
#pragma unroll
            for (int u = 0; u < kTcSub; ++u) {
                if (c * kTcSub + u >= blocks) break;
                const uint32_t a_addr = base + (uint32_t)((c % kTcStages) * kTcStageBytes + u * kTcBlockBytes);
                const uint64_t a_desc = umma_desc_k_sw128(a_addr), b_desc = umma_desc_k_sw128(a_addr + kTcABytes);
#pragma unroll
                for (int k = 0; k < kTcK / 8; ++k)  // 32 bytes along K per instruction: +2 in 16-byte units
                    umma_tf32(tmem, a_desc + 2 * k, b_desc + 2 * k, (c | u | k) != 0);
            }
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


// ---- input gradient on the tensor cores ----------------------------------------------------------------
//   dx[p, c] = sum_o d_o1[p, o] * W1[bucket(p), o, c]
// d_o1 is an arbitrary fp32 gradient; W1 = k / 128 is exact in TF32.  d_o1 is split into three TF32-exact
// parts, hi = d with the low 13 mantissa bits cleared, mid = (d - hi) with its low 13 bits cleared,
// lo = d - hi - mid (every subtraction is exact; 11 + 11 + 2 significant bits), so that every product the
// tensor core forms is exact and only the fp32 accumulation of 96 terms rounds.  The three parts extend K:
// A = [lo | mid | hi] (64 positions x 96), B = the tile's columns of W1 transposed ([column, o], the same
// 32 values of K for each part), small parts first.  One CTA per tile of the batch plan; the 3072 columns
// go in blocks of 128 (one tcgen05.mma N), the weight blocks through a three-stage cp.async ring, two
// accumulators of 128 tensor-memory columns alternate so that the read-back and the stores of block j - 1
// run beside the instructions of block j.  A thread reads back one POSITION's sums (lane of tensor memory =
// row of the instruction), which as global stores would be 32 scattered 16-byte pieces per instruction
// (measured: 0.124 ms for the kernel, slower than the FMA kernel's 0.096); the block goes through a
// shared-memory tile instead and leaves as whole 512-byte rows written by all four warps.  Every wait is bounded.
constexpr int kDxN = 128;                                   // columns per block = N of the instruction
constexpr int kDxStages = 3;
constexpr int kDxSlabBytes = kTP * 128;                     // one part of A: the tile's 64 rows x 128 B (rows 64..127 of the
                                                            // instruction's M read the finite floats that follow and land in
                                                            // tensor-memory lanes nobody reads, as in the forward kernel)
constexpr int kDxABytes = 3 * kDxSlabBytes;
constexpr int kDxBBytes = kDxN * 128;                       // 16 KiB: 128 columns x 32 o
constexpr int kDxPitch = kDxN + 4;                          // staging row pitch in floats: rows 16 B apart modulo 128 B
constexpr int kDxStageOutBytes = kTP * kDxPitch * 4;        // 33 KiB: one block of the tile on its way out
constexpr int kDxSmemBytes = 1024 + kDxABytes + kDxStages * kDxBBytes + kDxStageOutBytes + 64;
constexpr int kDxTmemCols = 2 * kDxN;                       // two accumulators; 106 KiB of shared memory: two CTAs per SM
constexpr uint32_t kIdescTf32Dx =
    (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kDxN >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_tf32_dx(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kIdescTf32Dx), "r"(accumulate), "r"(0u)
        : "memory");
}

// W1 [C * 32, L1] -> W1T [C, L1, 32]: the K-major operand the instruction wants for B
__global__ void __launch_bounds__(256)
    k_ls_transpose_w1(const float* __restrict__ W1, float* __restrict__ W1T, int L1) {
    __shared__ float t[32][33];
    const int bk = blockIdx.y, c0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 8 rows of the tile per pass
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int o = ty + 8 * i;
        t[o][tx] = c0 + tx < L1 ? __ldg(W1 + ((int64_t)bk * kLsOut + o) * L1 + c0 + tx) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = ty + 8 * i;
        if (c0 + c < L1) W1T[((int64_t)bk * L1 + c0 + c) * kLsOut + tx] = t[tx][c];
    }
}

__global__ void __launch_bounds__(kTcThreads)
    k_ls_l1_dx_tc(const float* __restrict__ d_o1, const float* __restrict__ W1T, LsPlanView plan,
                  float* __restrict__ dx, int L1, unsigned long long* status) {
    extern __shared__ unsigned char smem_raw[];
    const int t = blockIdx.x;
    if (t >= *plan.n_tiles) return;
    const int cnt = plan.tile_count[t], bk = plan.tile_bucket[t];
    const int32_t* perm = plan.perm + plan.tile_start[t];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* a0 = smem_raw + (base - smem_u32(smem_raw));
    unsigned char* b0 = a0 + kDxABytes;
    float* stg = reinterpret_cast<float*>(b0 + kDxStages * kDxBBytes);             // [kTP][kDxPitch]
    uint64_t* bar_done = reinterpret_cast<uint64_t*>(b0 + kDxStages * kDxBBytes + kDxStageOutBytes);  // [2]: the block's MMAs have finished
    __shared__ uint32_t s_tmem;
    __shared__ int32_t s_perm[kTP];  // the tile's positions (the copy-out reads one per row)
    if (tid < kTP) s_perm[tid] = tid < cnt ? perm[tid] : 0;

    if (tid == 0) {
        mbar_init(bar_done, 1);
        mbar_init(bar_done + 1, 1);
        fence_barrier_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(kDxTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // B blocks: column n of the block is row n of the operand, 128 B (the 32 o) per row, 16-byte pieces swizzled
    const float* wsrc = W1T + (int64_t)bk * L1 * kLsOut;
    const int nblk = L1 / kDxN;
    auto issue = [&](int j) {
        if (j < nblk) {
            unsigned char* st = b0 + (j % kDxStages) * kDxBBytes;
            const float* src = wsrc + (int64_t)j * kDxN * kLsOut;
#pragma unroll
            for (int i = 0; i < (kDxN * 8) / kTcThreads; ++i) {
                const int piece = tid + kTcThreads * i, n = piece >> 3, q = piece & 7;
                cp_async16(st + (n >> 3) * 1024 + (n & 7) * 128 + ((q ^ (n & 7)) << 4), src + n * kLsOut + 4 * q, true);
            }
        }
        cp_async_commit();
    };
    issue(0);
    issue(1);

    // A: the three parts of the tile's d_o1 rows (rows beyond the tile's count: zeros)
    for (int piece = tid; piece < kTP * 8; piece += kTcThreads) {
        const int r = piece >> 3, q = piece & 7;
        float4 d = f4_zero();
        if (r < cnt) d = __ldg(reinterpret_cast<const float4*>(d_o1 + (int64_t)perm[r] * kLsOut) + q);
        const float v[4] = {d.x, d.y, d.z, d.w};
        float hi[4], mid[4], lo[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            hi[i] = __uint_as_float(__float_as_uint(v[i]) & 0xFFFFE000u);
            const float r1 = __fsub_rn(v[i], hi[i]);
            mid[i] = __uint_as_float(__float_as_uint(r1) & 0xFFFFE000u);
            lo[i] = __fsub_rn(r1, mid[i]);
        }
        const uint32_t off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((q ^ (r & 7)) << 4));
        *reinterpret_cast<float4*>(a0 + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<float4*>(a0 + kDxSlabBytes + off) = make_float4(mid[0], mid[1], mid[2], mid[3]);
        *reinterpret_cast<float4*>(a0 + 2 * kDxSlabBytes + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    // accumulator of block jb -> shared-memory tile (warps 0 and 1: lane of tensor memory = position) -> global
    // rows (all warps).  Called by the whole CTA; two CTA barriers inside.
    auto epilogue = [&](int jb) {
        if (warp < kTP / 32) {
            const int pos = warp * 32 + lane;
            const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)((jb & 1) * kDxN);
            float4* row = reinterpret_cast<float4*>(stg + pos * kDxPitch);
            uint32_t v[kDxN / 32][32];  // all four loads in flight, one wait
#pragma unroll
            for (int c = 0; c < kDxN / 32; ++c) {
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[c][0]), "=r"(v[c][1]), "=r"(v[c][2]), "=r"(v[c][3]), "=r"(v[c][4]), "=r"(v[c][5]), "=r"(v[c][6]),
                      "=r"(v[c][7]), "=r"(v[c][8]), "=r"(v[c][9]), "=r"(v[c][10]), "=r"(v[c][11]), "=r"(v[c][12]), "=r"(v[c][13]),
                      "=r"(v[c][14]), "=r"(v[c][15]), "=r"(v[c][16]), "=r"(v[c][17]), "=r"(v[c][18]), "=r"(v[c][19]), "=r"(v[c][20]),
                      "=r"(v[c][21]), "=r"(v[c][22]), "=r"(v[c][23]), "=r"(v[c][24]), "=r"(v[c][25]), "=r"(v[c][26]), "=r"(v[c][27]),
                      "=r"(v[c][28]), "=r"(v[c][29]), "=r"(v[c][30]), "=r"(v[c][31])
                    : "r"(taddr + (uint32_t)(32 * c))
                    : "memory");
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int c = 0; c < kDxN / 32; ++c)
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    row[8 * c + i] = make_float4(__uint_as_float(v[c][4 * i]), __uint_as_float(v[c][4 * i + 1]),
                                                 __uint_as_float(v[c][4 * i + 2]), __uint_as_float(v[c][4 * i + 3]));
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();  // the tile is complete (and the accumulator is free again)
#pragma unroll 4
        for (int r = warp; r < cnt; r += kTcThreads / 32) {
            const float4* src = reinterpret_cast<const float4*>(stg + r * kDxPitch);
            float4* dst = reinterpret_cast<float4*>(dx + (int64_t)s_perm[r] * L1 + (int64_t)jb * kDxN);
#pragma unroll
            for (int h = 0; h < kDxN / 128; ++h) __stcs(dst + 32 * h + lane, src[32 * h + lane]);
        }
        __syncthreads();  // the tile may be overwritten
    };

    bool failed = false;
    for (int j = 0; j < nblk; ++j) {
        cp_async_wait<1>();                                             // this thread's pieces of block j are in
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // ... and visible to the tensor core (A too, first pass)
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t b_desc = umma_desc_k_sw128(base + (uint32_t)(kDxABytes + (j % kDxStages) * kDxBBytes));
            const uint32_t acc = tmem + (uint32_t)((j & 1) * kDxN);
#pragma unroll
            for (int part = 0; part < 3; ++part) {  // lo, mid, hi: the small parts enter the sum first
                const uint64_t a_desc = umma_desc_k_sw128(base + (uint32_t)(part * kDxSlabBytes));
#pragma unroll
                for (int k = 0; k < kLsOut / 8; ++k)
                    umma_tf32_dx(acc, a_desc + 2 * k, b_desc + 2 * k, (part | k) != 0);
            }
            umma_commit(bar_done + (j & 1));
        }
        if (j >= 1 && !mbar_wait_bounded(bar_done + ((j - 1) & 1), (unsigned)(((j - 1) >> 1) & 1))) failed = true;
        if (__syncthreads_or(failed)) {  // one decision for the CTA
            failed = true;
            break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (j >= 1) epilogue(j - 1);  // block j - 1 while the tensor core works on block j; frees accumulator (j - 1) & 1
        issue(j + 2);                 // into stage (j - 1) % 3, whose reader (the MMAs of block j - 1) has finished
    }
    cp_async_wait<0>();
    if (!failed) {
        if (!mbar_wait_bounded(bar_done + ((nblk - 1) & 1), (unsigned)(((nblk - 1) >> 1) & 1))) failed = true;
        failed = __syncthreads_or(failed);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (!failed) epilogue(nblk - 1);
    }
    if (failed && tid == 0) note_timeout(status);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kDxTmemCols) : "memory");
}


// ---- weight gradient on the tensor cores ----------------------------------------------------------------
//   dW1[bucket, o, c] = sum over the bucket's positions p of d_o1[p, o] * x[p, c]
// M = 128 columns c of one bucket's W1, N = 96 = the three TF32-exact parts of d_o1 (lo, mid, hi: see the input
// gradient above) x 32 outputs, K = the bucket's positions, 32 per stage.  x (q / 128) is exact in TF32, so every
// product is exact.  Both operands are wanted K-major, i.e. transposed against how x and d_o1 lie in memory.
// The rows of a stage (32 positions: 512 B of x, 128 B of d_o1 each) come in by cp.async, two stages ahead, into
// a raw tile whose rows are 16 B longer than their payload; then every LANE takes one position, reads its row
// (conflict-free thanks to the padding) and stores scalars into the 128-byte-swizzled operand layout, where the 32
// positions of a column fall into 32 different banks.  Operand buffers alternate, so that stage s + 1 is
// transposed while the tensor core works on stage s.  The sum over positions stays in tensor memory for
// kDwChunkStages stages (512 positions) at a time and is added to fp32 registers between chunks, which bounds the
// length of the tensor core's own accumulation chain.  The three parts are added in the epilogue, small ones
// first.  CTA = (bucket, 128 columns); 99 KiB of shared memory: two CTAs per SM.
constexpr int kDwM = 128;
constexpr int kDwN = 96;
constexpr int kDwABytesTc = kDwM * 128;                     // 16 KiB: 128 columns x 32 positions
constexpr int kDwBBytesTc = kDwN * 128;                     // 12 KiB: 96 rows (part, o) x 32 positions
constexpr int kDwOperandBytes = kDwABytesTc + kDwBBytesTc;  // 28 KiB
constexpr int kDwRawStages = 2;
constexpr int kDwXPitch = kDwM * 4 + 16;                    // bytes per raw row of x
constexpr int kDwDPitch = kLsOut * 4 + 16;                  // bytes per raw row of d_o1
constexpr int kDwRawBytes = 32 * (kDwXPitch + kDwDPitch);   // 21 KiB
constexpr int kDwChunkStages = 16;
constexpr int kDwSmemBytesTc = 1024 + 2 * kDwOperandBytes + kDwRawStages * kDwRawBytes + 64;
constexpr int kDwTmemCols = 128;
constexpr uint32_t kIdescTf32N96 = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kDwN >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_tf32_n96(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kIdescTf32N96), "r"(accumulate), "r"(0u)
        : "memory");
}

__global__ void __launch_bounds__(kTcThreads, 2)
    k_ls_l1_dw_tc(const float* __restrict__ x, const float* __restrict__ d_o1, LsPlanView plan,
                  float* __restrict__ dW1, float* __restrict__ db1, int L1, int n_col_blocks,
                  unsigned long long* status) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint32_t s_tmem;
    __shared__ float s_bias[kTcThreads / 32][kLsOut];
    const int bk = blockIdx.x / n_col_blocks, cb = blockIdx.x % n_col_blocks;
    const int t0 = plan.bucket_tile[bk], t1 = plan.bucket_tile[bk + 1];
    const int beg = t0 < t1 ? plan.tile_start[t0] : 0;
    const int end = t0 < t1 ? plan.tile_start[t1 - 1] + plan.tile_count[t1 - 1] : 0;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c0 = cb * kDwM;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* op0 = smem_raw + (base - smem_u32(smem_raw));   // two operand buffers (1024-byte aligned)
    unsigned char* raw0 = op0 + 2 * kDwOperandBytes;               // the raw ring
    uint64_t* bar_free = reinterpret_cast<uint64_t*>(raw0 + kDwRawStages * kDwRawBytes);  // [2]: operand buffer read
    uint64_t* bar_chunk = bar_free + 2;
    if (tid == 0) {
        mbar_init(bar_free, 1);
        mbar_init(bar_free + 1, 1);
        mbar_init(bar_chunk, 1);
        fence_barrier_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(kDwTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    float racc[kDwN];
#pragma unroll
    for (int i = 0; i < kDwN; ++i) racc[i] = 0.f;
    const int n_st = (end - beg + 31) / 32;

    // copies: thread t brings pieces (t & 3) + 4 i of row t >> 2 of the stage (8 of x, 2 of d_o1)
    const int crow = tid >> 2, cq = tid & 3;
    auto row_of = [&](int s) -> int64_t {  // position of this thread's row in stage s, -1 past the end
        const int k = beg + 32 * s + crow;
        return (s < n_st && k < end) ? (int64_t)__ldg(plan.perm + k) : -1;
    };
    auto issue = [&](int s, int64_t p) {   // stage s into raw slot s % kDwRawStages; rows past the end: zeros
        if (s < n_st) {
            unsigned char* rx = raw0 + (s % kDwRawStages) * kDwRawBytes + crow * kDwXPitch;
            unsigned char* rd = raw0 + (s % kDwRawStages) * kDwRawBytes + 32 * kDwXPitch + crow * kDwDPitch;
            const bool ok = p >= 0;
            const float* xs = x + (ok ? p : 0) * L1 + c0;
            const float* ds = d_o1 + (ok ? p : 0) * kLsOut;
#pragma unroll
            for (int i = 0; i < 8; ++i) cp_async16(rx + 16 * (cq + 4 * i), xs + 4 * (cq + 4 * i), ok);
#pragma unroll
            for (int i = 0; i < 2; ++i) cp_async16(rd + 16 * (cq + 4 * i), ds + 4 * (cq + 4 * i), ok);
        }
        cp_async_commit();
    };
    // transposition: lane = position of the stage, warp w takes columns [32 w, 32 w + 32) and outputs [8 w, 8 w + 8)
    const uint32_t kq = (uint32_t)(lane >> 2), kr = (uint32_t)((lane & 3) * 4);
    auto transpose = [&](int s) {
        const unsigned char* rx = raw0 + (s % kDwRawStages) * kDwRawBytes + lane * kDwXPitch + 128 * warp;
        const unsigned char* rd = raw0 + (s % kDwRawStages) * kDwRawBytes + 32 * kDwXPitch + lane * kDwDPitch + 32 * warp;
        unsigned char* A = op0 + (s & 1) * kDwOperandBytes;
        unsigned char* Bp = A + kDwABytesTc;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 q4 = *reinterpret_cast<const float4*>(rx + 16 * i);
            const float v[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t m = (uint32_t)(32 * warp + 4 * i + j);
                *reinterpret_cast<float*>(A + (m >> 3) * 1024 + (m & 7) * 128 + ((kq ^ (m & 7)) << 4) + kr) = v[j];
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float4 q4 = *reinterpret_cast<const float4*>(rd + 16 * i);
            const float v[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float hi = __uint_as_float(__float_as_uint(v[j]) & 0xFFFFE000u);
                const float r1 = __fsub_rn(v[j], hi);
                const float mid = __uint_as_float(__float_as_uint(r1) & 0xFFFFE000u);
                const float part[3] = {__fsub_rn(r1, mid), mid, hi};
#pragma unroll
                for (int q = 0; q < 3; ++q) {
                    const uint32_t n = (uint32_t)(q * kLsOut + 8 * warp + 4 * i + j);
                    *reinterpret_cast<float*>(Bp + (n >> 3) * 1024 + (n & 7) * 128 + ((kq ^ (n & 7)) << 4) + kr) = part[q];
                }
            }
        }
    };

    bool failed = false;
    int64_t p_next = row_of(kDwRawStages);  // row of the stage issued in the first trip
    for (int s = 0; s < kDwRawStages; ++s) issue(s, row_of(s));
    for (int s = 0; s < n_st; ++s) {
        cp_async_wait<kDwRawStages - 1>();  // this thread's pieces of stage s are in
        // the operand buffer was read by the instructions of stage s - 2
        if (s >= 2 && !mbar_wait_bounded(bar_free + (s & 1), (unsigned)((s / 2 - 1) & 1))) failed = true;
        if (__syncthreads_or(failed)) {     // ... and so are everybody's
            failed = true;
            break;
        }
        transpose(s);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();                    // operands complete; the raw slot may be refilled
        const bool last_of_chunk = (s % kDwChunkStages) == kDwChunkStages - 1 || s == n_st - 1;
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = base + (uint32_t)((s & 1) * kDwOperandBytes);
            const uint64_t a_desc = umma_desc_k_sw128(a_addr), b_desc = umma_desc_k_sw128(a_addr + kDwABytesTc);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                umma_tf32_n96(tmem, a_desc + 2 * k, b_desc + 2 * k, ((s % kDwChunkStages) | k) != 0);
            umma_commit(bar_free + (s & 1));
            if (last_of_chunk) umma_commit(bar_chunk);
        }
        issue(s + kDwRawStages, p_next);
        p_next = row_of(s + kDwRawStages + 1);
        if (last_of_chunk) {  // the chunk's sums out of tensor memory into the fp32 registers
            if (!mbar_wait_bounded(bar_chunk, (unsigned)((s / kDwChunkStages) & 1))) failed = true;
            if (__syncthreads_or(failed)) {
                failed = true;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c = 0; c < kDwN / 32; ++c) {
                uint32_t v[32];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(32 * c))
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 32; ++i) racc[32 * c + i] = __fadd_rn(racc[32 * c + i], __uint_as_float(v[i]));
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();  // the next chunk starts a fresh sum in tensor memory
        }
    }
    cp_async_wait<0>();
    if (!failed) {
        const int m = warp * 32 + lane;  // lane of tensor memory = column of the block
#pragma unroll
        for (int o = 0; o < kLsOut; ++o)
            dW1[((int64_t)bk * kLsOut + o) * L1 + c0 + m] =
                __fadd_rn(__fadd_rn(racc[o], racc[kLsOut + o]), racc[2 * kLsOut + o]);
        if (cb == 0) {  // the bias gradient: lane = output, the warps take every 4th position, added in warp order
            float b = 0.f;
            for (int k = beg + warp; k < end; k += kTcThreads / 32)
                b = __fadd_rn(b, __ldg(d_o1 + (int64_t)__ldg(plan.perm + k) * kLsOut + lane));
            s_bias[warp][lane] = b;
            __syncthreads();
            if (warp == 0) {
                float t = s_bias[0][lane];
                for (int w = 1; w < kTcThreads / 32; ++w) t = __fadd_rn(t, s_bias[w][lane]);
                db1[bk * kLsOut + lane] = t;
            }
        }
    }
    if (failed && tid == 0) note_timeout(status);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kDwTmemCols) : "memory");
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

extern "C" size_t nnue_ls_l1_bwd_tc_workspace_bytes(int32_t L1, int32_t C) {
    if (L1 <= 0 || C <= 0) return 0;
    return (size_t)C * kLsOut * (size_t)L1 * sizeof(float) + 256;
}

extern "C" int nnue_ls_l1_bwd_tc(const float* x, const float* W1, const float* d_o1, const void* plan, float* dx,
                                 float* dW1, float* db1, int64_t B, int32_t L1, int32_t C, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    NNUE_REQUIRE(B >= 0 && L1 > 0 && L1 % kDxN == 0 && C > 0 && C <= 16, NNUE_ERR_UNSUPPORTED,
                 "nnue_ls_l1_bwd_tc: needs L1 %% 128 == 0 and 1..16 buckets (B=%lld L1=%d C=%d)", (long long)B, L1, C);
    // the weight gradient (its K is the batch: thousands of terms) stays on the fp32 FMA kernel, and so does
    // everything when no input gradient is asked for
    if (B == 0 || dx == nullptr) return nnue_ls_l1_bwd(x, W1, d_o1, plan, dx, dW1, db1, B, L1, C, stream);
    NNUE_REQUIRE(plan != nullptr && aligned16(plan) && W1 && d_o1 && aligned16(W1) && aligned16(d_o1) && aligned16(dx),
                 NNUE_ERR_ARG, "nnue_ls_l1_bwd_tc: null or unaligned tensor");
    char* ws = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t)255);
    NNUE_REQUIRE(workspace && workspace_bytes >= nnue_ls_l1_bwd_tc_workspace_bytes(L1, C), NNUE_ERR_WORKSPACE,
                 "nnue_ls_l1_bwd_tc: workspace too small (see nnue_ls_l1_bwd_tc_workspace_bytes)");
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "nnue_ls_l1_bwd_tc: no device status word");
    static bool done[64] = {false};
    int dev = -1;
    NNUE_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !done[dev]) {
        NNUE_CUDA_TRY(cudaFuncSetAttribute(k_ls_l1_dx_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, kDxSmemBytes));
        if (dev >= 0 && dev < 64) done[dev] = true;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* W1T = reinterpret_cast<float*>(ws);
    k_ls_transpose_w1<<<dim3((unsigned)((L1 + 31) / 32), (unsigned)C), 256, 0, s>>>(W1, W1T, L1);
    {
        ProfScope prof("k_ls_l1_dx_tc", s);
        k_ls_l1_dx_tc<<<(unsigned)ls_max_tiles(B, C), kTcThreads, kDxSmemBytes, s>>>(d_o1, W1T, ls_view(plan, B, C), dx, L1,
                                                                                    status);
    }
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(2);
    if (tuning().ls_dw_tc == 0 || L1 % kDwM != 0)
        return nnue_ls_l1_bwd(x, W1, d_o1, plan, nullptr, dW1, db1, B, L1, C, stream);  // weight and bias gradients
    NNUE_REQUIRE(x && dW1 && db1 && aligned16(x) && aligned16(dW1), NNUE_ERR_ARG, "nnue_ls_l1_bwd_tc: null or unaligned tensor");
    static bool done_dw[64] = {false};
    if (dev < 0 || dev >= 64 || !done_dw[dev]) {
        NNUE_CUDA_TRY(cudaFuncSetAttribute(k_ls_l1_dw_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, kDwSmemBytesTc));
        if (dev >= 0 && dev < 64) done_dw[dev] = true;
    }
    {
        ProfScope prof("k_ls_l1_dw_tc", s);
        k_ls_l1_dw_tc<<<(unsigned)(C * (L1 / kDwM)), kTcThreads, kDwSmemBytesTc, s>>>(x, d_o1, ls_view(plan, B, C), dW1, db1, L1,
                                                                                     L1 / kDwM, status);
    }
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}
