// fp8_gemm for callers that cannot hand the library any scratch memory.
//
// dsv3_fp8_gemm splits K on small problems and parks the partial sums in a workspace the caller
// allocates.  Some hosts have nothing to allocate from at call time: a serving process that gave
// the whole device to its own arena when it started (weights, KV cache and activations planned to
// the last byte, so a cudaMalloc in the request path either fails or stalls every stream while the
// driver synchronises the device), or a plain C program that links this library without a framework
// allocator behind it.  For them the same tcgen05 kernel runs here with its scratch in a fixed array
// that is part of the library image.
//
// The array costs kStaticScratchBytes of device memory on every GPU that loads the library, for the
// life of the process.  All calls on a device share it: two calls that can overlap on the GPU (different
// streams without an ordering between them) race on it, and whatever the previous call left in it is
// still there, so the part that must start at zero (the split-K ticket header) is cleared on the
// caller's stream before every launch.
#include "gemm_plan.cuh"

namespace dsv3 {

namespace {

constexpr size_t kStaticScratchBytes = DSV3_STATIC_SCRATCH_BYTES;

// Device-resident scratch.  In host code this name is only a handle for the runtime's symbol
// table, not an address a kernel could use: the device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device, resolved on first use with that device
// current.  Returns nullptr (error recorded) if the lookup fails.
void* static_scratch_ptr() {
    static void* cached[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaGetDevice");
        return nullptr;
    }
    if (dev < 0 || dev >= 64) {
        set_last_error("fp8_gemm_static: device ordinal %d is outside the supported range", dev);
        return nullptr;
    }
    if (!cached[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) {
            cuda_fail(e, "cudaGetSymbolAddress(g_static_scratch)");
            return nullptr;
        }
        cached[dev] = ptr;
    }
    return cached[dev];
}

}  // namespace

}  // namespace dsv3

using namespace dsv3;

extern "C" {

size_t dsv3_fp8_gemm_static_scratch_bytes(void) { return kStaticScratchBytes; }

int dsv3_fp8_gemm_static(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N,
                         int64_t K, void* c, dsv3_stream_t stream) {
    if (M < 0 || N < 0 || K < 0) {
        set_last_error("fp8_gemm_static: negative size");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (M == 0 || N == 0) return DSV3_OK;
    if (!c || (K > 0 && (!a || !a_s || !b || !b_s))) {
        set_last_error("fp8_gemm_static: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (K == 0) {
        DSV3_CUDA_TRY(cudaMemsetAsync(c, 0, static_cast<size_t>(M) * N * 2, st));
        return DSV3_OK;
    }
    if (!tc_supported(a, b, c, M, N, K)) {
        set_last_error("fp8_gemm_static: needs K %% 16 == 0 and 16-byte aligned a, b, c (the tcgen05 kernels' limits)");
        return DSV3_ERR_UNSUPPORTED;
    }
    const int forced = gemm_policy_kernel();
    if (forced == 1) {
        set_last_error("fp8_gemm_static: gemm policy 1 (CUDA-core kernel) is not offered here; it needs no scratch, "
                       "call dsv3_fp8_gemm");
        return DSV3_ERR_UNSUPPORTED;
    }
    TcPlan pl = tc_plan(M, N, K, forced, gemm_policy_split());
    if (pl.error != DSV3_OK) return pl.error;
    // The automatic plan may want more partial tiles than the array holds: fall back to the largest split factor
    // of the same tile shape that fits (a pinned split factor is honoured or refused, never changed).
    if (gemm_policy_split() == 0 && tc_workspace_bytes(pl, M, N) > kStaticScratchBytes) {
        const int kernel = pl.swap ? 3 : 2;
        for (int sfac = pl.splits - 1; sfac >= 1; --sfac) {
            const TcPlan alt = tc_plan(M, N, K, kernel, sfac);
            if (alt.error == DSV3_OK && tc_workspace_bytes(alt, M, N) <= kStaticScratchBytes) {
                pl = alt;
                break;
            }
        }
    }
    const size_t need = tc_workspace_bytes(pl, M, N);
    if (need > kStaticScratchBytes) {
        set_last_error("fp8_gemm_static: this problem (M=%lld N=%lld K=%lld, split-K %d) needs %zu bytes of scratch, "
                       "the built-in array holds %zu; use dsv3_fp8_gemm with a caller-provided workspace",
                       static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(K), pl.splits, need,
                       kStaticScratchBytes);
        return DSV3_ERR_WORKSPACE;
    }
    void* scratch = nullptr;
    if (need > 0) {
        scratch = static_scratch_ptr();
        if (!scratch) return DSV3_ERR_CUDA;
        // the ticket header must read zero when the kernel starts; an earlier call that was cut short
        // may have left it dirty
        DSV3_CUDA_TRY(cudaMemsetAsync(scratch, 0, DSV3_WORKSPACE_HEADER_BYTES, st));
    }
    return launch_fp8_gemm_tc(a, a_s, b, b_s, M, N, K, c, scratch, need > 0 ? kStaticScratchBytes : 0, pl, st);
}

}  // extern "C"
