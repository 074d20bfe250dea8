// Shared device/host helpers for libnnue_b200 (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/nnue_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "libnnue_b200 is written for sm_100a (Blackwell B200) only"
#endif

namespace nnue {

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr unsigned kFullMask = 0xffffffffu;

// ---- host-side error plumbing ------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define NNUE_CUDA_TRY(expr)                                         \
    do {                                                            \
        cudaError_t e__ = (expr);                                   \
        if (e__ != cudaSuccess) return ::nnue::cuda_fail(e__, #expr); \
    } while (0)

#define NNUE_REQUIRE(cond, code, ...)      \
    do {                                   \
        if (!(cond)) {                     \
            ::nnue::set_error(__VA_ARGS__);\
            return (code);                 \
        }                                  \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Device status word: [0] = count of out-of-range indices skipped,
// [1] = count of bounded waits that ran out, [2] = segments with repeated entries too long to sort
// in shared memory (informational), [3] = forward warps that needed fp32 table rows and had none.
// One per device, lazily resolved.
unsigned long long* device_status_ptr();

struct Tuning {
    int fwd_u = 1;        // float4 per lane per half in the fused forward (1, 2 or 4)
    int bwd_u = 2;        // float4 per lane in the segment gather-sum (1, 2 or 4)
    int sparse_u = 2;     // float4 per lane in the sparse-linear forward
    int stage_idx = 1;    // 1 = bulk-copy index lists to shared memory when aligned
    int long_row = 256;   // rows with more hits are reduced by a whole CTA
    int prologue_pb = 32; // positions per CTA in the backward prologue
    int sort_segments = 1;// 1 = order every CSR segment (deterministic sums)
    int seg_chunk = 256;  // entries per warp in the chunked segment gather-sum; 0 = one warp per row
    int bwd_r = 0;        // compiled variant of the chunked gather-sum (see LAUNCH_CHUNKS)
    int fwd_variant = 0;  // compiled variant of the fused forward (see LAUNCH_FWD)
    int fwd_q16_variant = 0;  // compiled variant of the int16-table forward (see LAUNCH_Q16)
    int overlap_csr = 1;  // 1 = build the CSR on the helper stream, beside the backward prologue
    int ddp_reduce_ctas = 0;  // > 0: grid cap of the peer-load reduce (it runs beside the sliced backward)
    int ls_dw_tc = 0;           // 1: the first layer's weight gradient of the quantized model on the tensor cores too
                                // (correct, measured slower than the FMA kernel: 0.163 against 0.111 ms)
    int col_slice_streams = 1;  // 1: column slices of the backward alternate between two streams
    int ddp_reduce_u = 0;     // > 0: float4 per thread and rank in flight in the peer-load reduce (1, 2, 4 or 8)
};
Tuning& tuning();

int sm_count();

// Host-side tally of kernels this process has launched (for benchmarks).
void note_launches(int n);

// Brackets the launches enqueued on `s` during its lifetime with two timing
// events when nnue_b200_profile(1) is in effect; free otherwise.  `name` must
// be a string constant.
class ProfScope {
public:
    ProfScope(const char* name, cudaStream_t s);
    ~ProfScope();
    ProfScope(const ProfScope&) = delete;
    ProfScope& operator=(const ProfScope&) = delete;

private:
    int slot_;
    cudaStream_t stream_;
};

// ---- device helpers -----------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ float4 ldg4(const float4* p) { return __ldg(p); }

__device__ __forceinline__ void st_stream4(float4* p, float4 v) { __stcs(p, v); }

__device__ __forceinline__ float4 f4_zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }

// Blackwell's packed fp32 add (add.rn.f32x2: two IEEE round-to-nearest adds in
// one instruction).  The gather kernels are instruction-issue bound, and half
// of their instructions are these adds.
#ifndef NNUE_F32X2
#define NNUE_F32X2 1
#endif
__device__ __forceinline__ float4 f4_add(float4 a, float4 b) {
#if NNUE_F32X2
    unsigned long long a01, a23, b01, b23, r01, r23;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a01) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(a23) : "f"(a.z), "f"(a.w));
    asm("mov.b64 %0, {%1, %2};" : "=l"(b01) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(b23) : "f"(b.z), "f"(b.w));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r01) : "l"(a01), "l"(b01));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r23) : "l"(a23), "l"(b23));
    float4 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(r01));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.z), "=f"(r.w) : "l"(r23));
    return r;
#else
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z),
                       __fadd_rn(a.w, b.w));
#endif
}

// a*s + b*t with each product and the sum rounded separately, as the
// elementwise torch composition does (no FMA contraction).
__device__ __forceinline__ float mix(float s, float a, float t, float b) {
    return __fadd_rn(__fmul_rn(s, a), __fmul_rn(t, b));
}
__device__ __forceinline__ float4 f4_mix(float s, float4 a, float t, float4 b) {
    return make_float4(mix(s, a.x, t, b.x), mix(s, a.y, t, b.y), mix(s, a.z, t, b.z),
                       mix(s, a.w, t, b.w));
}

__device__ __forceinline__ void red_add_v4(float* addr, float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y),
                 "f"(v.z), "f"(v.w)
                 : "memory");
}

__device__ __forceinline__ void note_bad_index(unsigned long long* status) {
    atomicAdd(status, 1ULL);
}
__device__ __forceinline__ void note_timeout(unsigned long long* status) {
    atomicAdd(status + 1, 1ULL);
}

// Number of leading non-negative entries of list[0..K): the reference stops
// at the first -1 (sparse_linear_kernel.py:149, fused_ft_kernel.py:69).
// Whole-warp call; `list` may be shared or global memory.
__device__ __forceinline__ int count_active(const int32_t* list, int K, int lane) {
    int n = 0;
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int k = k0 + lane;
        const int v = (k < K) ? list[k] : -1;
        const unsigned neg = __ballot_sync(kFullMask, v < 0);
        if (neg) {
            n += __ffs(neg) - 1;
            return n;
        }
        n += 32;
    }
    return n < K ? n : K;
}

// ---- mbarrier + 1-D bulk copy (global -> shared), no multicast ----------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// 16-byte aligned src/dst, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, unsigned bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// Bounded wait on phase `parity`.  Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity) {
    const uint32_t a = smem_u32(bar);
    for (int it = 0; it < (1 << 16); ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// ---- per-thread 16-byte asynchronous copies (global -> shared) -------------
// `pred` false writes 16 zero bytes instead (nothing is read from `src`).
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem, bool pred) {
    const unsigned n = pred ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(n)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

#endif  // __CUDACC__

}  // namespace nnue
