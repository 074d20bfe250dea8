// Single-perspective sparse linear layer: forward gather-sum and backward.
// Replaces the CuPy kernels of
// model/modules/feature_transformer/sparse_linear_kernel.py:114-157 / :237-288
// (reference project paths).
#include "gather.cuh"
#include "segment.cuh"

namespace nnue {

// One warp per (position, column tile of 32*U float4); tiles are the slow grid
// dimension (see ft_fused.cu for why).
template <int U>
__global__ void __launch_bounds__(kThreads)
    k_sparse_fwd(const int32_t* __restrict__ idx, const float4* __restrict__ weight,
                 const float4* __restrict__ bias, float4* __restrict__ out, int64_t B, int K,
                 int64_t N, int64_t W4, int n_pos_groups, unsigned long long* status) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / n_pos_groups;
    const int64_t p = (int64_t)(blockIdx.x % n_pos_groups) * kWarpsPerCta + warp;
    if (p >= B) return;
    int col[U];
    bool ok[U];
    float4 acc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        col[u] = tile * (32 * U) + u * 32 + lane;
        ok[u] = col[u] < W4;
        acc[u] = ok[u] ? ldg4(bias + col[u]) : f4_zero();
    }
    const int32_t* list = idx + p * K;
    const int n = count_active(list, K, lane);
    gather_sum<U, 8 / U>(weight, W4, N, list, n, col, ok, acc, lane, status);
#pragma unroll
    for (int u = 0; u < U; ++u)
        if (ok[u]) st_stream4(out + p * W4 + col[u], acc[u]);
}

// Scalar twin: lane = one column.
__global__ void __launch_bounds__(kThreads)
    k_sparse_fwd_scalar(const int32_t* __restrict__ idx, const float* __restrict__ weight,
                        const float* __restrict__ bias, float* __restrict__ out, int64_t B, int K,
                        int64_t N, int W, int n_pos_groups, unsigned long long* status) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / n_pos_groups;
    const int64_t p = (int64_t)(blockIdx.x % n_pos_groups) * kWarpsPerCta + warp;
    const int c = tile * 32 + lane;
    if (p >= B || c >= W) return;
    float acc = bias[c];
    const int32_t* list = idx + p * K;
    for (int k = 0; k < K; ++k) {
        const int r = list[k];
        if (r < 0) break;
        if ((int64_t)r >= N) { if (c == 0) note_bad_index(status); continue; }
        acc = __fadd_rn(acc, weight[(int64_t)r * W + c]);
    }
    out[p * W + c] = acc;
}

// Atomic backward for comparison runs: vector reductions into a zeroed table.
template <int U>
__global__ void __launch_bounds__(kThreads)
    k_sparse_bwd_atomic(const int32_t* __restrict__ idx, const float4* __restrict__ grad_out,
                        float* __restrict__ grad_weight, int64_t B, int K, int64_t N, int64_t W4,
                        int n_pos_groups, unsigned long long* status) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / n_pos_groups;
    const int64_t p = (int64_t)(blockIdx.x % n_pos_groups) * kWarpsPerCta + warp;
    if (p >= B) return;
    int col[U];
    bool nz[U];
    float4 g[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        col[u] = tile * (32 * U) + u * 32 + lane;
        const bool ok = col[u] < W4;
        g[u] = ok ? __ldcs(grad_out + p * W4 + col[u]) : f4_zero();
        nz[u] = ok && (g[u].x != 0.f || g[u].y != 0.f || g[u].z != 0.f || g[u].w != 0.f);
    }
    const int32_t* list = idx + p * K;
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int k = k0 + lane;
        const int mine = (k < K) ? __ldg(list + k) : -1;
        const unsigned neg = __ballot_sync(kFullMask, mine < 0);
        const int m = neg ? (__ffs(neg) - 1) : 32;
        for (int j = 0; j < m; ++j) {
            const int r = __shfl_sync(kFullMask, mine, j);
            if ((int64_t)r >= N) {
                if (lane == 0 && tile == 0) note_bad_index(status);
                continue;
            }
            float* row = grad_weight + (int64_t)r * (W4 * 4);
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (nz[u]) red_add_v4(row + 4 * col[u], g[u]);
        }
        if (neg) break;
    }
}

}  // namespace nnue

using namespace nnue;

static size_t align_up_(size_t x, size_t a) { return (x + a - 1) / a * a; }

extern "C" int nnue_ft_sparse_fwd(const int32_t* idx, const float* weight, const float* bias,
                                  float* out, int64_t B, int32_t K, int64_t N, int32_t W,
                                  void* stream) {
    NNUE_REQUIRE(B >= 0 && K >= 0 && N >= 0 && W > 0, NNUE_ERR_ARG,
                 "nnue_ft_sparse_fwd: negative size (B=%lld K=%d N=%lld W=%d)", (long long)B, K,
                 (long long)N, W);
    if (B == 0) return NNUE_OK;
    NNUE_REQUIRE(idx && weight && bias && out, NNUE_ERR_ARG, "nnue_ft_sparse_fwd: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "nnue_ft_sparse_fwd: no device status word");
    const int64_t groups = (B + kWarpsPerCta - 1) / kWarpsPerCta;
    const bool vec = (W % 4 == 0) && aligned16(weight) && aligned16(bias) && aligned16(out);
    if (!vec) {
        const int64_t tiles = (W + 31) / 32;
        NNUE_REQUIRE(groups * tiles <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "grid too large");
        k_sparse_fwd_scalar<<<(unsigned)(groups * tiles), kThreads, 0, s>>>(
            idx, weight, bias, out, B, K, N, W, (int)groups, status);
        NNUE_CUDA_TRY(cudaGetLastError());
        note_launches(1);
        return NNUE_OK;
    }
    const int64_t W4 = W / 4;
    int U = tuning().sparse_u;
    if (U != 1 && U != 2 && U != 4) U = 2;
    while (U > 1 && W4 <= 32 * (U / 2)) U /= 2;
    const int64_t tiles = (W4 + 32 * U - 1) / (32 * U);
    NNUE_REQUIRE(groups * tiles <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "grid too large");
    const unsigned grid = (unsigned)(groups * tiles);
    const float4* w4 = reinterpret_cast<const float4*>(weight);
    const float4* b4 = reinterpret_cast<const float4*>(bias);
    float4* o4 = reinterpret_cast<float4*>(out);
    if (U == 1) k_sparse_fwd<1><<<grid, kThreads, 0, s>>>(idx, w4, b4, o4, B, K, N, W4, (int)groups, status);
    else if (U == 2) k_sparse_fwd<2><<<grid, kThreads, 0, s>>>(idx, w4, b4, o4, B, K, N, W4, (int)groups, status);
    else k_sparse_fwd<4><<<grid, kThreads, 0, s>>>(idx, w4, b4, o4, B, K, N, W4, (int)groups, status);
    NNUE_CUDA_TRY(cudaGetLastError());
    note_launches(1);
    return NNUE_OK;
}

// workspace: column-sum scratch [kColumnSumSlices, W] | CSR scratch
extern "C" size_t nnue_ft_sparse_bwd_workspace_bytes(int64_t B, int32_t K, int64_t N, int32_t W,
                                                     int32_t mode) {
    (void)mode;
    if (B < 0 || K < 0 || N < 0 || W <= 0) return 0;
    return align_up_((size_t)kColumnSumSlices * W * sizeof(float), 256) +
           csr_workspace_bytes(B * (int64_t)K, N, W) + 256;
}

extern "C" int nnue_ft_sparse_bwd(const int32_t* idx, const float* grad_out, float* grad_weight,
                                  float* grad_bias, int64_t B, int32_t K, int64_t N, int32_t W,
                                  void* workspace, size_t workspace_bytes, int32_t mode,
                                  void* stream) {
    NNUE_REQUIRE(B >= 0 && K >= 0 && N >= 0 && W > 0, NNUE_ERR_ARG, "nnue_ft_sparse_bwd: negative size");
    NNUE_REQUIRE(mode >= NNUE_BWD_AUTO && mode <= NNUE_BWD_SEGMENT, NNUE_ERR_ARG,
                 "nnue_ft_sparse_bwd: unknown mode %d", mode);
    NNUE_REQUIRE(grad_weight && grad_bias, NNUE_ERR_ARG, "nnue_ft_sparse_bwd: null output");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (B == 0) {
        if (N > 0) NNUE_CUDA_TRY(cudaMemsetAsync(grad_weight, 0, (size_t)N * W * sizeof(float), s));
        NNUE_CUDA_TRY(cudaMemsetAsync(grad_bias, 0, (size_t)W * sizeof(float), s));
        return NNUE_OK;
    }
    NNUE_REQUIRE(idx && grad_out, NNUE_ERR_ARG, "nnue_ft_sparse_bwd: null pointer");
    const size_t need = nnue_ft_sparse_bwd_workspace_bytes(B, K, N, W, mode);
    NNUE_REQUIRE(workspace && workspace_bytes >= need, NNUE_ERR_WORKSPACE,
                 "nnue_ft_sparse_bwd: workspace %zu bytes < required %zu", workspace_bytes, need);
    unsigned long long* status = device_status_ptr();
    NNUE_REQUIRE(status, NNUE_ERR_CUDA, "nnue_ft_sparse_bwd: no device status word");

    char* ws = reinterpret_cast<char*>(align_up_(reinterpret_cast<uintptr_t>(workspace), 256));
    float* scratch = reinterpret_cast<float*>(ws);
    ws += align_up_((size_t)kColumnSumSlices * W * sizeof(float), 256);
    int rc = column_sum(grad_out, B, W, grad_bias, s, scratch);
    if (rc != NNUE_OK) return rc;

    const bool vec = (W % 4 == 0) && aligned16(grad_out) && aligned16(grad_weight);
    if (mode == NNUE_BWD_ATOMIC && vec) {
        NNUE_CUDA_TRY(cudaMemsetAsync(grad_weight, 0, (size_t)N * W * sizeof(float), s));
        const int64_t W4 = W / 4;
        int U = tuning().bwd_u;
        if (U != 1 && U != 2 && U != 4) U = 2;
        while (U > 1 && W4 <= 32 * (U / 2)) U /= 2;
        const int64_t tiles = (W4 + 32 * U - 1) / (32 * U);
        const int64_t groups = (B + kWarpsPerCta - 1) / kWarpsPerCta;
        NNUE_REQUIRE(groups * tiles <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "grid too large");
        const unsigned grid = (unsigned)(groups * tiles);
        const float4* g4 = reinterpret_cast<const float4*>(grad_out);
        if (U == 1) k_sparse_bwd_atomic<1><<<grid, kThreads, 0, s>>>(idx, g4, grad_weight, B, K, N, W4, (int)groups, status);
        else if (U == 2) k_sparse_bwd_atomic<2><<<grid, kThreads, 0, s>>>(idx, g4, grad_weight, B, K, N, W4, (int)groups, status);
        else k_sparse_bwd_atomic<4><<<grid, kThreads, 0, s>>>(idx, g4, grad_weight, B, K, N, W4, (int)groups, status);
        NNUE_CUDA_TRY(cudaGetLastError());
        note_launches(1);
        return NNUE_OK;
    }
    const int32_t* lists[1] = {idx};
    CsrPlan plan;
    rc = csr_plan(plan, 1, B, K, N, W, ws, workspace_bytes - (size_t)(ws - static_cast<char*>(workspace)));
    if (rc != NNUE_OK) return rc;
    rc = csr_build(plan, lists, s);
    if (rc != NNUE_OK) return rc;
    return csr_reduce(plan, grad_out, W, grad_weight, s);
}
