// Library-wide plumbing: error text, tuning table, the per-device status
// words and the two dense helpers (gradient norm, clip coefficient).
#include <stdarg.h>

#include <algorithm>
#include <vector>

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

// ---- per-kernel timing (nnue_b200_profile) ----------------------------------
struct ProfSpan {
    const char* name;
    cudaEvent_t a, b;
    bool closed;
};
static bool g_prof_on = false;
static std::vector<ProfSpan> g_prof_spans;   // used[0, g_prof_used) belong to the current record
static size_t g_prof_used = 0;
constexpr size_t kProfMaxSpans = 1 << 16;

ProfScope::ProfScope(const char* name, cudaStream_t s) : slot_(-1), stream_(s) {
    if (!g_prof_on || g_prof_used >= kProfMaxSpans) return;
    if (g_prof_used == g_prof_spans.size()) {
        ProfSpan sp{name, nullptr, nullptr, false};
        if (cudaEventCreate(&sp.a) != cudaSuccess || cudaEventCreate(&sp.b) != cudaSuccess) {
            cudaGetLastError();
            return;
        }
        g_prof_spans.push_back(sp);
    }
    ProfSpan& sp = g_prof_spans[g_prof_used];
    sp.name = name;
    sp.closed = false;
    if (cudaEventRecord(sp.a, s) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    slot_ = (int)g_prof_used++;
}

ProfScope::~ProfScope() {
    if (slot_ < 0) return;
    ProfSpan& sp = g_prof_spans[(size_t)slot_];
    if (cudaEventRecord(sp.b, stream_) == cudaSuccess) sp.closed = true;
    else cudaGetLastError();
}

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
    else if (!strcmp(key, "fwd_q16_variant")) t.fwd_q16_variant = value;
    else if (!strcmp(key, "ddp_reduce_ctas")) t.ddp_reduce_ctas = value;
    else if (!strcmp(key, "ddp_reduce_u")) t.ddp_reduce_u = value;
    else if (!strcmp(key, "col_slice_streams")) t.col_slice_streams = value;
    else if (!strcmp(key, "ls_dw_tc")) t.ls_dw_tc = value;
    else if (!strcmp(key, "overlap_csr")) t.overlap_csr = value;
    else {
        set_error("nnue_b200_tune: unknown key '%s'", key);
        return NNUE_ERR_ARG;
    }
    return NNUE_OK;
}

extern "C" int nnue_b200_profile(int32_t enable) {
    if (enable) g_prof_used = 0;
    g_prof_on = enable != 0;
    return NNUE_OK;
}

extern "C" int nnue_b200_profile_read(int32_t i, const char** h_name, double* h_total_ms,
                                      int64_t* h_launches) {
    NNUE_REQUIRE(i >= 0 && h_name && h_total_ms && h_launches, NNUE_ERR_ARG, "nnue_b200_profile_read: bad argument");
    NNUE_CUDA_TRY(cudaDeviceSynchronize());
    // group by name in order of first appearance
    std::vector<const char*> names;
    for (size_t k = 0; k < g_prof_used; ++k) {
        const char* n = g_prof_spans[k].name;
        bool seen = false;
        for (const char* m : names) seen = seen || !strcmp(m, n);
        if (!seen) names.push_back(n);
    }
    NNUE_REQUIRE((size_t)i < names.size(), NNUE_ERR_ARG, "nnue_b200_profile_read: entry %d of %zu", i, names.size());
    double total = 0.0;
    int64_t count = 0;
    for (size_t k = 0; k < g_prof_used; ++k) {
        const ProfSpan& sp = g_prof_spans[k];
        if (!sp.closed || strcmp(sp.name, names[(size_t)i])) continue;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, sp.a, sp.b) != cudaSuccess) {
            cudaGetLastError();
            continue;
        }
        total += ms;
        ++count;
    }
    *h_name = names[(size_t)i];
    *h_total_ms = total;
    *h_launches = count;
    return NNUE_OK;
}

// ---- L2 -> SM read probe ------------------------------------------------------
namespace nnue {
__global__ void __launch_bounds__(kThreads, 4)
    k_l2_read_probe(const float4* __restrict__ buf, long long rows, long long warps, int rows_per_warp,
                    int pattern, float4* __restrict__ sink) {
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (w >= warps) return;
    float4 acc0 = f4_zero(), acc1 = f4_zero();
    // 64 float4 per row; the lane's two pieces are the forward's "column c and column h + c"
    unsigned long long state = 0x9E3779B97F4A7C15ULL * (unsigned long long)(w + 1);
    long long r = (long long)(state % (unsigned long long)rows);
    for (int i = 0; i < rows_per_warp; i += 4) {
        float4 v[4][2];
        long long rr[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            if (pattern) {
                state = state * 6364136223846793005ULL + 1442695040888963407ULL;
                rr[t] = (long long)((state >> 33) % (unsigned long long)rows);
            } else {
                rr[t] = r;
                r = (r + 1 == rows) ? 0 : r + 1;
            }
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const bool live = i + t < rows_per_warp;
            const float4* row = buf + rr[t] * 64;
            v[t][0] = live ? ldg4(row + lane) : f4_zero();
            v[t][1] = live ? ldg4(row + 32 + lane) : f4_zero();
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            acc0 = f4_add(acc0, v[t][0]);
            acc1 = f4_add(acc1, v[t][1]);
        }
    }
    sink[w * 32 + lane] = f4_add(acc0, acc1);
}
}  // namespace nnue

extern "C" int nnue_l2_read_probe(const void* buf, int64_t rows, int64_t warps, int32_t rows_per_warp,
                                  int32_t pattern, void* sink, void* stream) {
    NNUE_REQUIRE(buf && sink && rows > 0 && warps > 0 && rows_per_warp > 0, NNUE_ERR_ARG,
                 "nnue_l2_read_probe: bad argument");
    NNUE_REQUIRE(aligned16(buf) && aligned16(sink), NNUE_ERR_ALIGN, "nnue_l2_read_probe: 16-byte aligned buffers");
    const int64_t ctas = (warps + kWarpsPerCta - 1) / kWarpsPerCta;
    NNUE_REQUIRE(ctas <= 0x7fffffffLL, NNUE_ERR_UNSUPPORTED, "nnue_l2_read_probe: grid too large");
    k_l2_read_probe<<<(unsigned)ctas, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float4*>(buf), rows, warps, rows_per_warp, pattern, static_cast<float4*>(sink));
    note_launches(1);
    NNUE_CUDA_TRY(cudaGetLastError());
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
    if (h[3]) {
        set_error("%llu forward warps needed the fp32 table rows (a weight left the packed int16 range) "
                  "and were given none", h[3]);
        return NNUE_ERR_UNSUPPORTED;
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
