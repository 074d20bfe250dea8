// Library-wide plumbing: error text, tuning table, the per-device status
// words and the two dense helpers (gradient norm, clip coefficient).
#include <stdarg.h>

#include <algorithm>

#include "common.cuh"

namespace nnue {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return NNUE_ERR_CUDA;
}

Tuning& tuning() {
    static Tuning t;
    return t;
}

// [0] out-of-range indices skipped, [1] bounded waits that ran out,
// [2] CSR segments left in fill order, [3] spare.
__device__ unsigned long long g_status[4];

unsigned long long* device_status_ptr() {
    static unsigned long long* cache[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cache[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status) != cudaSuccess) return nullptr;
        cache[dev] = static_cast<unsigned long long*>(p);
    }
    return cache[dev];
}

static unsigned long long g_launches = 0;
void note_launches(int n) { g_launches += (unsigned long long)n; }

int sm_count() {
    static int cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cache[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

// ---- gradient norm helpers ------------------------------------------------
// The gradients the norm was taken over are `prescale` times the true ones
// (data-parallel ranks sum before they average): the coefficient folds both.
__global__ void k_clip_coef(const float* __restrict__ sumsq, float max_norm, float prescale,
                            float* __restrict__ coef) {
    const float total = prescale * sqrtf(*sumsq);
    const float c = max_norm / (total + 1e-6f);
    *coef = prescale * (c < 1.f ? c : 1.f);
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_b200_abi_version(void) { return NNUE_B200_ABI_VERSION; }

extern "C" const char* nnue_b200_last_error(void) { return g_error; }

extern "C" int64_t nnue_b200_launch_count(void) { return (int64_t)g_launches; }

extern "C" int nnue_b200_tune(const char* key, int value) {
    NNUE_REQUIRE(key != nullptr, NNUE_ERR_ARG, "nnue_b200_tune: null key");
    Tuning& t = tuning();
    if (!strcmp(key, "fwd_u")) t.fwd_u = value;
    else if (!strcmp(key, "bwd_u")) t.bwd_u = value;
    else if (!strcmp(key, "sparse_u")) t.sparse_u = value;
    else if (!strcmp(key, "stage_idx")) t.stage_idx = value;
    else if (!strcmp(key, "long_row")) t.long_row = value > 0 ? value : 1;
    else if (!strcmp(key, "prologue_pb")) t.prologue_pb = value > 0 ? value : 1;
    else if (!strcmp(key, "sort_segments")) t.sort_segments = value;
    else if (!strcmp(key, "seg_chunk")) t.seg_chunk = value > 0 ? value : 0;
    else if (!strcmp(key, "bwd_r")) t.bwd_r = value;
    else if (!strcmp(key, "fwd_variant")) t.fwd_variant = value;
    else if (!strcmp(key, "ddp_reduce_ctas")) t.ddp_reduce_ctas = value;
    else if (!strcmp(key, "overlap_csr")) t.overlap_csr = value;
    else {
        set_error("nnue_b200_tune: unknown key '%s'", key);
        return NNUE_ERR_ARG;
    }
    return NNUE_OK;
}

extern "C" int nnue_b200_device_status(void* stream, int64_t* h_bad_index_count,
                                       int64_t* h_timeout_count) {
    unsigned long long* d = device_status_ptr();
    NNUE_REQUIRE(d, NNUE_ERR_CUDA, "nnue_b200_device_status: no device status word");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned long long h[4] = {0, 0, 0, 0};
    NNUE_CUDA_TRY(cudaMemcpyAsync(h, d, sizeof(h), cudaMemcpyDeviceToHost, s));
    NNUE_CUDA_TRY(cudaMemsetAsync(d, 0, sizeof(h), s));
    NNUE_CUDA_TRY(cudaStreamSynchronize(s));
    if (h_bad_index_count) *h_bad_index_count = (int64_t)h[0];
    if (h_timeout_count) *h_timeout_count = (int64_t)h[1];
    if (h[0]) {
        set_error("%llu feature indices were outside [0, N) and were skipped", h[0]);
        return NNUE_ERR_INDEX;
    }
    if (h[1]) {
        set_error("%llu bounded device-side waits ran out", h[1]);
        return NNUE_ERR_TIMEOUT;
    }
    return NNUE_OK;
}

extern "C" int nnue_grad_sumsq(const float* grad, int64_t n, float* d_out_sumsq, void* stream) {
    NNUE_REQUIRE(n >= 0 && d_out_sumsq, NNUE_ERR_ARG, "nnue_grad_sumsq: bad argument");
    if (n == 0) return NNUE_OK;
    NNUE_REQUIRE(grad, NNUE_ERR_ARG, "nnue_grad_sumsq: null gradient");
    const float* grads[1] = {grad};
    return nnue_grad_sumsq_multi(grads, &n, 1, d_out_sumsq, stream);  // one reproducible implementation
}

extern "C" int nnue_clip_coef(const float* d_sumsq, float max_norm, float prescale, float* d_coef,
                              void* stream) {
    NNUE_REQUIRE(d_sumsq && d_coef, NNUE_ERR_ARG, "nnue_clip_coef: null pointer");
    k_clip_coef<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(d_sumsq, max_norm, prescale, d_coef);
    note_launches(1);
    NNUE_CUDA_TRY(cudaGetLastError());
    return NNUE_OK;
}
