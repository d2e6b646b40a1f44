// extern "C" surface of libdsv3_b200.so: argument checks, kernel selection, status plumbing.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include <stdlib.h>

#include "common.cuh"
#include "gemm_plan.cuh"

namespace dsv3 {

// kernels (one translation unit each)
int launch_act_quant(const void* x, int64_t rows, int64_t K, int block_size, int scale_fmt, void* y, float* s,
                     cudaStream_t stream);
int launch_swiglu_quant(const void* a, const void* b, int64_t rows, int64_t K, int scale_fmt, void* y, float* s,
                        cudaStream_t stream);
int launch_weight_dequant(const void* w, const float* s, int64_t N, int64_t K, int block, void* y, cudaStream_t stream);
int launch_weight_quant(const void* w, int64_t N, int64_t K, void* q, float* s, cudaStream_t stream);
int launch_fp8_gemm_simple(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N,
                           int64_t K, void* c, cudaStream_t stream);

// ------------------------------------------------------------------ errors
static thread_local char t_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_last_error, sizeof(t_last_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_last_error("%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
    return DSV3_ERR_CUDA;
}

static int g_sm_budget = 0;   // dsv3_set_num_sms: SMs the persistent GEMM kernels may occupy (0 = all)

int num_sms() {
    static int cached[64] = {};
    int dev = 0;
    int n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
        if (cached[dev] == 0) {
            int q = 0;
            if (cudaDeviceGetAttribute(&q, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || q <= 0) q = 148;
            cached[dev] = q;
        }
        n = cached[dev];
    }
    return (g_sm_budget > 0 && g_sm_budget < n) ? g_sm_budget : n;
}

bool pdl_enabled() {
    static const bool on = (getenv("DSV3_DISABLE_PDL") == nullptr);
    return on;
}

// ------------------------------------------------------------------ status words
__device__ unsigned int g_status[4];

unsigned int* status_device_ptr() {
    static unsigned int* cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        set_last_error("status word: no current device");
        return nullptr;
    }
    if (!cached[dev]) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_status);
        if (e != cudaSuccess) {
            cuda_fail(e, "cudaGetSymbolAddress(g_status)");
            return nullptr;
        }
        cached[dev] = static_cast<unsigned int*>(ptr);
    }
    return cached[dev];
}

static int g_force_kernel = 0;
static int g_force_split = 0;
int gemm_policy_kernel() { return g_force_kernel; }
int gemm_policy_split() { return g_force_split; }

static bool is_null(const void* p) { return p == nullptr; }

}  // namespace dsv3

using namespace dsv3;

extern "C" {

int dsv3_version(void) { return 100; }

const char* dsv3_strerror(int status) {
    switch (status) {
        case DSV3_OK: return "ok";
        case DSV3_ERR_INVALID_ARGUMENT: return "invalid argument";
        case DSV3_ERR_UNSUPPORTED: return "unsupported shape or option";
        case DSV3_ERR_CUDA: return "CUDA call failed";
        case DSV3_ERR_WORKSPACE: return "workspace missing or too small";
        case DSV3_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
        default: return "unknown status";
    }
}

const char* dsv3_last_error(void) { return t_last_error; }

int dsv3_act_quant(const void* x, int64_t rows, int64_t K, int block_size, int scale_fmt, void* y, float* s,
                   dsv3_stream_t stream) {
    if (rows < 0 || K < 0 || block_size <= 0) {
        set_last_error("act_quant: negative size or block_size <= 0");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (K % block_size != 0) {
        set_last_error("act_quant: last dimension %lld is not divisible by block_size %d", (long long)K, block_size);
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (scale_fmt != DSV3_SCALE_FMT_FP32 && scale_fmt != DSV3_SCALE_FMT_UE8M0) {
        set_last_error("act_quant: unknown scale_fmt %d", scale_fmt);
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (rows == 0 || K == 0) return DSV3_OK;
    if (is_null(x) || is_null(y) || is_null(s)) {
        set_last_error("act_quant: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (block_size % 8 != 0 || block_size > 1024) {
        set_last_error("act_quant: block_size %d must be a multiple of 8 and at most 1024", block_size);
        return DSV3_ERR_UNSUPPORTED;
    }
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(y) % 8 != 0) {
        set_last_error("act_quant: x must be 16-byte and y 8-byte aligned");
        return DSV3_ERR_UNSUPPORTED;
    }
    return launch_act_quant(x, rows, K, block_size, scale_fmt, y, s, static_cast<cudaStream_t>(stream));
}

int dsv3_swiglu_quant(const void* a, const void* b, int64_t rows, int64_t K, int scale_fmt, void* y, float* s,
                      dsv3_stream_t stream) {
    if (rows < 0 || K < 0) {
        set_last_error("swiglu_quant: negative size");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (K % 128 != 0) {
        set_last_error("swiglu_quant: last dimension %lld is not divisible by 128", (long long)K);
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (scale_fmt != DSV3_SCALE_FMT_FP32 && scale_fmt != DSV3_SCALE_FMT_UE8M0) {
        set_last_error("swiglu_quant: unknown scale_fmt %d", scale_fmt);
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (rows == 0 || K == 0) return DSV3_OK;
    if (is_null(a) || is_null(b) || is_null(y) || is_null(s)) {
        set_last_error("swiglu_quant: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (reinterpret_cast<uintptr_t>(a) % 16 != 0 || reinterpret_cast<uintptr_t>(b) % 16 != 0 || reinterpret_cast<uintptr_t>(y) % 8 != 0) {
        set_last_error("swiglu_quant: a and b must be 16-byte and y 8-byte aligned");
        return DSV3_ERR_UNSUPPORTED;
    }
    return launch_swiglu_quant(a, b, rows, K, scale_fmt, y, s, static_cast<cudaStream_t>(stream));
}

int dsv3_weight_dequant(const void* w, const float* s, int64_t N, int64_t K, int block_size, void* y,
                        dsv3_stream_t stream) {
    if (N < 0 || K < 0 || block_size <= 0) {
        set_last_error("weight_dequant: negative size or block_size <= 0");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (N == 0 || K == 0) return DSV3_OK;
    if (is_null(w) || is_null(s) || is_null(y)) {
        set_last_error("weight_dequant: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    return launch_weight_dequant(w, s, N, K, block_size, y, static_cast<cudaStream_t>(stream));
}

int dsv3_weight_quant(const void* w, int64_t N, int64_t K, void* q, float* s, dsv3_stream_t stream) {
    if (N < 0 || K < 0) {
        set_last_error("weight_quant: negative size");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (N == 0 || K == 0) return DSV3_OK;
    if (is_null(w) || is_null(q) || is_null(s)) {
        set_last_error("weight_quant: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    return launch_weight_quant(w, N, K, q, s, static_cast<cudaStream_t>(stream));
}

int dsv3_set_gemm_policy(int kernel, int split_k) {
    if (kernel < 0 || kernel > 6 || split_k < 0 || split_k > 64) {
        set_last_error("set_gemm_policy: kernel must be 0..6 and split_k 0..64");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    g_force_kernel = kernel;
    g_force_split = split_k;
    return DSV3_OK;
}

int dsv3_set_num_sms(int n) {
    if (n < 0 || (n > 0 && n < 2)) {
        set_last_error("set_num_sms: 0 (all SMs) or at least 2");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    g_sm_budget = n;
    return DSV3_OK;
}

size_t dsv3_fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0 || g_force_kernel == 1 || g_force_kernel == 5 || (K % 16) != 0) return 0;
    if (g_force_kernel == 0 && g_force_split == 0 && M <= 8 && N >= 2048 && K >= 1024 && N * K <= (6ll << 20)) return 0;   // decode kernel
    const TcPlan pl = tc_plan(M, N, K, g_force_kernel, g_force_split);
    if (pl.error != DSV3_OK) return 0;     // dsv3_fp8_gemm reports the reason
    return tc_workspace_bytes(pl, M, N);
}

int dsv3_fp8_gemm(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N, int64_t K,
                  void* c, void* workspace, size_t workspace_bytes, dsv3_stream_t stream) {
    if (M < 0 || N < 0 || K < 0) {
        set_last_error("fp8_gemm: negative size");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (M == 0 || N == 0) return DSV3_OK;
    if (is_null(c) || (K > 0 && (is_null(a) || is_null(a_s) || is_null(b) || is_null(b_s)))) {
        set_last_error("fp8_gemm: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (K == 0) {
        DSV3_CUDA_TRY(cudaMemsetAsync(c, 0, static_cast<size_t>(M) * N * 2, st));
        return DSV3_OK;
    }
    if (g_force_kernel == 5) {
        if (!small_linear_supported(a, b, c, M, N, K, false)) {
            set_last_error("fp8_gemm: the decode kernel needs M <= 16, K %% 16 == 0 and 16-byte aligned a and b");
            return DSV3_ERR_UNSUPPORTED;
        }
        return launch_fp8_linear_small(nullptr, a, a_s, b, b_s, M, N, K, DSV3_SCALE_FMT_FP32, c, st);
    }
    // Automatic choice, decode-sized problems with a few megabytes of weights in many rows and at least eight K
    // chunks: the register-streaming kernel has less to set up than the tcgen05 pipeline (measured on B200 at
    // M = 1..8: N 3072 x K 1536: 4.5-4.6 vs 4.8-4.9 us; with shorter K the tcgen05 kernel is level or ahead -- N 4096 x
    // K 512: 3.2 vs 3.2 us, N 7168 x K 256: 3.3-3.6 vs 2.9-3.0 us -- as it is at 11 MB and more: 7.4 vs 6.1 us).
    if (g_force_kernel == 0 && g_force_split == 0 && M <= 8 && N >= 2048 && K >= 1024 && N * K <= (6ll << 20) &&
        small_linear_supported(a, b, c, M, N, K, false))
        return launch_fp8_linear_small(nullptr, a, a_s, b, b_s, M, N, K, DSV3_SCALE_FMT_FP32, c, st);
    const bool tc_ok = tc_supported(a, b, c, M, N, K);
    if (g_force_kernel == 1 || (!tc_ok && g_force_kernel == 0))
        return launch_fp8_gemm_simple(a, a_s, b, b_s, M, N, K, c, st);
    if (!tc_ok) {
        set_last_error("fp8_gemm: the tcgen05 kernels need K %% 16 == 0 and 16-byte aligned a, b, c");
        return DSV3_ERR_UNSUPPORTED;
    }
    const TcPlan pl = tc_plan(M, N, K, g_force_kernel, g_force_split);
    if (pl.error != DSV3_OK) return pl.error;
    return launch_fp8_gemm_tc(a, a_s, b, b_s, M, N, K, c, workspace, workspace_bytes, pl, st);
}

int dsv3_fp8_linear(const void* x, int64_t M, int64_t K, const void* w, const float* w_s, int64_t N, int scale_fmt, void* c,
                    dsv3_stream_t stream) {
    if (M < 0 || N < 0 || K < 0) {
        set_last_error("fp8_linear: negative size");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (scale_fmt != DSV3_SCALE_FMT_FP32 && scale_fmt != DSV3_SCALE_FMT_UE8M0) {
        set_last_error("fp8_linear: unknown scale_fmt %d", scale_fmt);
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (M == 0 || N == 0) return DSV3_OK;
    if (is_null(x) || is_null(w) || is_null(w_s) || is_null(c)) {
        set_last_error("fp8_linear: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (!small_linear_supported(x, w, c, M, N, K, true)) {
        set_last_error("fp8_linear: takes 1..16 rows, K %% 128 == 0 and 16-byte aligned x and w (M=%lld K=%lld); use "
                       "dsv3_act_quant + dsv3_fp8_gemm otherwise", (long long)M, (long long)K);
        return DSV3_ERR_UNSUPPORTED;
    }
    return launch_fp8_linear_small(x, nullptr, nullptr, w, w_s, M, N, K, scale_fmt, c, static_cast<cudaStream_t>(stream));
}

int dsv3_selftest_bounded_wait(uint64_t limit_ns, dsv3_stream_t stream) {
    if (limit_ns == 0 || limit_ns > 1000ull * 1000ull * 1000ull) {
        set_last_error("selftest_bounded_wait: the limit must be between 1 ns and 1 s");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    return launch_bounded_wait_selftest(limit_ns, static_cast<cudaStream_t>(stream));
}

int dsv3_check_device_status(dsv3_stream_t stream, uint32_t detail[4]) {
    DSV3_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    unsigned int* dptr = status_device_ptr();
    if (!dptr) return DSV3_ERR_CUDA;
    unsigned int host[4] = {0, 0, 0, 0};
    DSV3_CUDA_TRY(cudaMemcpy(host, dptr, sizeof(host), cudaMemcpyDeviceToHost));
    if (detail) memcpy(detail, host, sizeof(host));
    if (host[0] == 0) return DSV3_OK;
    const unsigned int zero[4] = {0, 0, 0, 0};
    DSV3_CUDA_TRY(cudaMemcpy(dptr, zero, sizeof(zero), cudaMemcpyHostToDevice));
    set_last_error("device wait gave up: kind=%u (1 smem-empty, 2 smem-full, 3 tmem-empty, 4 tmem-full, 7/8 scale table, "
                   "9 self-test, 10 all-reduce peer signal) counter=%u cta=%u",
                   host[1], host[2], host[3]);
    return DSV3_ERR_DEVICE_TIMEOUT;
}

}  // extern "C"
