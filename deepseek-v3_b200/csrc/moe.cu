// MoE expert loop as grouped GEMMs: C entry points and the combine kernel.
//
// Replaces the Python loop of MoE.forward (inference/model.py:683-689): per local expert i,
//   idx, top = where(indices == i) ; y[idx] += expert(x[idx]) * weights[idx, top, None]
// with bf16 rounding after the product and after every accumulation, in ascending expert order.
#include "gemm_plan.cuh"

namespace dsv3 {

namespace {

constexpr int kThreads = 256;

// y[t, :] = sum over the token's experts, in ascending expert order, of bf16(o[pos, :] * w), each
// partial sum rounded to bf16 (the arithmetic of `y[idx] += ...` on bf16 tensors).
//   pos [T, topk] int32: row of `o` holding expert output for the j-th smallest expert id of token t, or -1
//   w   [T, topk] bf16 : routing weight of that pair
__global__ void __launch_bounds__(kThreads) moe_combine_kernel(const __nv_bfloat16* __restrict__ o,
                                                                const int* __restrict__ pos,
                                                                const __nv_bfloat16* __restrict__ w,
                                                                __nv_bfloat16* __restrict__ y, int64_t T, int topk,
                                                                int64_t dim) {
    const int64_t groups_per_row = dim >> 3;                       // 8 bf16 = 16 bytes per thread
    const int64_t total = T * groups_per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
        const int64_t t = i / groups_per_row;
        const int64_t d = (i - t * groups_per_row) << 3;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
        for (int j = 0; j < topk; ++j) {
            const int r = __ldg(pos + t * topk + j);
            if (r < 0) continue;
            const float wf = __bfloat162float(w[t * topk + j]);
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(o + static_cast<int64_t>(r) * dim + d));
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(words[e] << 16), hi = __uint_as_float(words[e] & 0xFFFF0000u);
                const float pl = __bfloat162float(__float2bfloat16_rn(lo * wf));       // bf16 product
                const float ph = __bfloat162float(__float2bfloat16_rn(hi * wf));
                acc[2 * e] = __bfloat162float(__float2bfloat16_rn(acc[2 * e] + pl));    // bf16 accumulate
                acc[2 * e + 1] = __bfloat162float(__float2bfloat16_rn(acc[2 * e + 1] + ph));
            }
        }
        uint4 out = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                               pack_bf16x2(acc[6], acc[7]));
        *reinterpret_cast<uint4*>(y + t * dim + d) = out;
    }
}

}  // namespace

}  // namespace dsv3

using namespace dsv3;

extern "C" {

size_t dsv3_group_table_bytes(int n_groups) { return n_groups > 0 ? group_table_bytes(n_groups) : 0; }

int dsv3_group_table_build(void* table, const void* const* weights, const float* const* scales, int n_groups,
                           int64_t N, int64_t K, dsv3_stream_t stream) {
    if (!table || !weights || !scales || N <= 0 || K <= 0) {
        set_last_error("group_table_build: null pointer or non-positive size");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    return build_group_table(table, weights, scales, n_groups, N, K, static_cast<cudaStream_t>(stream));
}

int dsv3_fp8_gemm_grouped(const void* table, int n_groups, const void* a, const float* a_s, const int32_t* seg,
                          int64_t rows_total, int64_t N, int64_t K, void* c, dsv3_stream_t stream) {
    if (rows_total < 0 || N < 0 || K <= 0) {
        set_last_error("fp8_gemm_grouped: negative size");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (rows_total == 0 || N == 0) return DSV3_OK;
    if (!table || !a || !a_s || !seg || !c) {
        set_last_error("fp8_gemm_grouped: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    return launch_fp8_gemm_grouped(table, n_groups, a, a_s, seg, rows_total, N, K, c, static_cast<cudaStream_t>(stream));
}

int dsv3_moe_combine(const void* o, const int32_t* pos, const void* w, int64_t T, int topk, int64_t dim, void* y,
                     dsv3_stream_t stream) {
    if (T < 0 || topk < 0 || dim < 0) {
        set_last_error("moe_combine: negative size");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (T == 0 || dim == 0) return DSV3_OK;
    if (!pos || !w || !y || (topk > 0 && !o)) {
        set_last_error("moe_combine: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (dim % 8 != 0 || reinterpret_cast<uintptr_t>(o) % 16 != 0 || reinterpret_cast<uintptr_t>(y) % 16 != 0) {
        set_last_error("moe_combine: dim must be a multiple of 8 and o, y 16-byte aligned");
        return DSV3_ERR_UNSUPPORTED;
    }
    const int64_t total = T * (dim >> 3);
    int64_t grid = (total + kThreads - 1) / kThreads;
    const int64_t cap = static_cast<int64_t>(num_sms()) * 8;
    if (grid > cap) grid = cap;
    moe_combine_kernel<<<static_cast<unsigned>(grid), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(o), pos, static_cast<const __nv_bfloat16*>(w),
        static_cast<__nv_bfloat16*>(y), T, topk, dim);
    DSV3_CUDA_TRY(cudaGetLastError());
    return DSV3_OK;
}

}  // extern "C"
