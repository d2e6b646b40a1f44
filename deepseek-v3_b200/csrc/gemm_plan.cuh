// Internal interface of the tcgen05 fp8_gemm kernels: problem geometry ("plan") and launcher.
#pragma once

#include "common.cuh"

namespace dsv3 {

// Geometry chosen for a problem; shared by the workspace query and the launch.
struct TcPlan {
    bool swap;  // true: weights on the MMA M axis (small M)
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

// Grouped GEMM over per-group weights (MoE experts).
size_t group_table_bytes(int n);
int build_group_table(void* table_dev, const void* const* weights, const float* const* scales, int n, int64_t N,
                      int64_t K, cudaStream_t stream);
int launch_fp8_gemm_grouped(const void* table_dev, int n, const void* a, const float* a_s, const int* seg_dev,
                            int64_t rows_total, int64_t N, int64_t K, void* c, cudaStream_t stream);

// Kernel / split-K override set through dsv3_set_gemm_policy (0 = automatic).
int gemm_policy_kernel();
int gemm_policy_split();

}  // namespace dsv3
