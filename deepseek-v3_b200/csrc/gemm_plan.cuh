// Internal interface of the tcgen05 fp8_gemm kernels: problem geometry ("plan") and launcher.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace dsv3 {

// Geometry chosen for a problem; shared by the workspace query and the launch.
struct TcPlan {
    int error;  // DSV3_OK, or the status to return (detail recorded): a pinned kernel / split factor that cannot be honoured
    bool swap;  // true: weights on the MMA M axis (small M)
    bool pair;  // token-major tiles on CTA pairs (fp8_gemm_tm.cu); never with split-K
    bool wide;  // with pair: 256 x 256 tiles (fp8_gemm_tw.cu)
    int bn;     // rows of the second operand tile
    int tiles_p, tiles_q, splits, kc;
};

bool tc_supported(const void* a, const void* b, const void* c, int64_t M, int64_t N, int64_t K);
TcPlan tc_plan(int64_t M, int64_t N, int64_t K, int force_kernel, int force_split);
// 0 when the plan does not split K; otherwise ticket header + splits * M * N fp32 partial sums.
size_t tc_workspace_bytes(const TcPlan& pl, int64_t M, int64_t N);
int launch_fp8_gemm_tc(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N,
                       int64_t K, void* c, void* workspace, size_t workspace_bytes, const TcPlan& pl,
                       cudaStream_t stream);

// Tensor maps over the operands as they lie in memory.  Operand: [rows, K] bytes, row-major; box = 128 bytes x
// box_rows, 128-byte swizzle, zero fill outside.  Result: [M, N] bf16, row-major; box = 64 columns x 128 rows,
// 128-byte swizzle (N % 8 == 0).
int make_tmap(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int box_rows);
int make_tmap_out(CUtensorMap* map, void* base, int64_t M, int64_t N);

// Token-major kernel on CTA pairs (256 x 128 tiles, tcgen05 cta_group::2, no split-K): fp8_gemm_tm.cu.
// `forced`: the kernel was pinned, so only its hard limit applies, not the speed heuristic.
bool tm_pair_supported(int64_t M, int64_t N, int64_t K, bool forced);
int launch_fp8_gemm_tm(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N,
                       int64_t K, void* c, cudaStream_t stream);

// Token-major kernel on CTA pairs with 256-wide accumulators (256 x 256 tiles, no split-K): fp8_gemm_tw.cu.
bool tw_pair_supported(int64_t M, int64_t N, int64_t K, bool forced);
int launch_fp8_gemm_tw(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N,
                       int64_t K, void* c, cudaStream_t stream);

// Decode-sized Linear without tcgen05 set-up (fp8_linear_small.cu): M <= 16; x != nullptr quantises bf16 activations
// in the kernel's prologue (K % 128 == 0), otherwise (a, a_s) are the quantised activations (K % 16 == 0).
bool small_linear_supported(const void* act, const void* w, const void* c, int64_t M, int64_t N, int64_t K, bool fused);
int launch_fp8_linear_small(const void* x, const void* a, const float* a_s, const void* w, const float* w_s, int64_t M,
                            int64_t N, int64_t K, int scale_fmt, void* c, cudaStream_t stream);

// Grouped GEMM over per-group weights (MoE experts).
size_t group_table_bytes(int n);
int build_group_table(void* table_dev, const void* const* weights, const float* const* scales, int n, int64_t N,
                      int64_t K, cudaStream_t stream);
int launch_fp8_gemm_grouped(const void* table_dev, int n, const void* a, const float* a_s, const int* seg_dev,
                            int64_t rows_total, int64_t rows_hint, int64_t N, int64_t K, void* c, cudaStream_t stream);

// One thread waits for an mbarrier phase that never completes; the bounded wait gives up after limit_ns.
int launch_bounded_wait_selftest(uint64_t limit_ns, cudaStream_t stream);

// Kernel / split-K override set through dsv3_set_gemm_policy (0 = automatic).
int gemm_policy_kernel();
int gemm_policy_split();

}  // namespace dsv3
