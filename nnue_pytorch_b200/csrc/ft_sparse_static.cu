// Sparse-linear backward for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc (or anything that calls it
// for them) at the moment they need a gradient: a program that handed the
// whole device to its own memory pool at start-up and forbids later
// allocations, or a service with a no-allocation-after-initialisation rule.
// nnue_ft_sparse_bwd needs a
// caller-provided workspace, which such a host may have no way to obtain.
// This entry point brings its own: a fixed array in the library's device
// image.  It has no counterpart in the reference project.
#include "common.cuh"

namespace nnue {

// Every device that loads the library holds this array until the process
// exits.  256-byte alignment is what the workspace carving assumes.
constexpr size_t kStaticScratchBytes = NNUE_SPARSE_BWD_STATIC_SCRATCH_BYTES;  // 32 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a
// device address; the address comes from cudaGetSymbolAddress, once per
// device, with that device current.  The cache below is filled without a
// lock: concurrent first calls from several host threads would each do the
// same look-up and store the same value.
static int static_scratch_ptr(void** out) {
    static void* cache[64] = {nullptr};
    int dev = -1;
    NNUE_CUDA_TRY(cudaGetDevice(&dev));
    NNUE_REQUIRE(dev >= 0 && dev < 64, NNUE_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (!cache[dev]) {
        void* p = nullptr;
        NNUE_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        NNUE_REQUIRE(p != nullptr, NNUE_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        cache[dev] = p;
    }
    *out = cache[dev];
    return NNUE_OK;
}

}  // namespace nnue

using namespace nnue;

extern "C" int nnue_ft_sparse_bwd_static(const int32_t* idx, const float* grad_out,
                                         float* grad_weight, float* grad_bias, int64_t B, int32_t K,
                                         int64_t N, int32_t W, void* stream) {
    NNUE_REQUIRE(B >= 0 && K >= 0 && N >= 0 && W > 0, NNUE_ERR_ARG,
                 "nnue_ft_sparse_bwd_static: negative size");
    const size_t need = nnue_ft_sparse_bwd_workspace_bytes(B, K, N, W, NNUE_BWD_SEGMENT);
    NNUE_REQUIRE(need <= kStaticScratchBytes, NNUE_ERR_WORKSPACE,
                 "nnue_ft_sparse_bwd_static: B=%lld K=%d N=%lld W=%d needs %zu bytes of scratch, the "
                 "built-in array holds %zu; use nnue_ft_sparse_bwd with your own workspace",
                 (long long)B, K, (long long)N, W, need, kStaticScratchBytes);
    void* scratch = nullptr;
    const int rc = static_scratch_ptr(&scratch);
    if (rc != NNUE_OK) return rc;
    // The segment route zeroes its counters itself (cudaMemsetAsync on `stream`)
    // and overwrites everything else it reads, so stale contents from the
    // previous call are harmless.
    return nnue_ft_sparse_bwd(idx, grad_out, grad_weight, grad_bias, B, K, N, W, scratch,
                              kStaticScratchBytes, NNUE_BWD_SEGMENT, stream);
}
