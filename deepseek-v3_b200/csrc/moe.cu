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

// Bookkeeping of the expert loop in one launch (one CTA): groups the (token, expert) pairs by local expert and
// orders every token's pairs by expert id.  Replaces `counts = bincount(indices)`, the per-expert
// `where(indices == i)` (model.py:680-686) and the sort / scan / gather chain a framework needs for the same.
//   seg [n + 1]        : seg[e] = first row of expert e in the grouped order, seg[n] = number of local pairs
//   tok [P]            : token of the pair placed at each row (pairs of other ranks' experts follow seg[n])
//   pair_row [P]       : scratch; row given to pair p, or -1 when its expert is not local
//   pos_sorted, w_sorted [T, topk]: per token, rows and routing weights in ascending expert order
// The order of an expert's rows is whatever the atomics give; every row's result depends on that row alone, so
// the outputs do not depend on it.
constexpr int kRouteThreads = 1024;
constexpr int kRouteMaxExperts = 256;
constexpr int kRouteMaxTopk = 32;

__global__ void __launch_bounds__(kRouteThreads) moe_route_kernel(const int64_t* __restrict__ indices,
                                                                  const float* __restrict__ weights, int64_t T, int topk,
                                                                  int start, int n, int* __restrict__ seg,
                                                                  int* __restrict__ tok, int* __restrict__ pair_row,
                                                                  int* __restrict__ pos_sorted,
                                                                  __nv_bfloat16* __restrict__ w_sorted) {
    __shared__ int cnt[kRouteMaxExperts + 1];
    __shared__ int cursor[kRouteMaxExperts + 1];
    const int64_t P = T * topk;
    for (int i = threadIdx.x; i <= n; i += kRouteThreads) cnt[i] = 0;
    __syncthreads();
    for (int64_t pr = threadIdx.x; pr < P; pr += kRouteThreads) {
        const int64_t e = indices[pr] - start;
        atomicAdd(&cnt[(e >= 0 && e < n) ? static_cast<int>(e) : n], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i <= n; ++i) {
            cursor[i] = run;
            if (i <= n) seg[i] = run;
            run += cnt[i];
        }
    }
    __syncthreads();
    for (int64_t pr = threadIdx.x; pr < P; pr += kRouteThreads) {
        const int64_t e = indices[pr] - start;
        const bool local = (e >= 0 && e < n);
        const int row = atomicAdd(&cursor[local ? static_cast<int>(e) : n], 1);
        tok[row] = static_cast<int>(pr / topk);
        pair_row[pr] = local ? row : -1;
    }
    __syncthreads();   // pair_row is read below by other threads of this CTA
    for (int64_t t = threadIdx.x; t < T; t += kRouteThreads) {
        int64_t e[kRouteMaxTopk];
        int order[kRouteMaxTopk];
        for (int j = 0; j < topk; ++j) {          // insertion sort of the token's experts, ascending
            const int64_t ej = indices[t * topk + j];
            int k = j;
            while (k > 0 && e[k - 1] > ej) {
                e[k] = e[k - 1];
                order[k] = order[k - 1];
                --k;
            }
            e[k] = ej;
            order[k] = j;
        }
        for (int j = 0; j < topk; ++j) {
            pos_sorted[t * topk + j] = pair_row[t * topk + order[j]];
            w_sorted[t * topk + j] = __float2bfloat16_rn(weights[t * topk + order[j]]);
        }
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
                          int64_t rows_total, int64_t rows_hint, int64_t N, int64_t K, void* c, dsv3_stream_t stream) {
    if (rows_total < 0 || rows_hint < 0 || N < 0 || K <= 0) {
        set_last_error("fp8_gemm_grouped: negative size");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (rows_total == 0 || N == 0) return DSV3_OK;
    if (!table || !a || !a_s || !seg || !c) {
        set_last_error("fp8_gemm_grouped: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    return launch_fp8_gemm_grouped(table, n_groups, a, a_s, seg, rows_total, rows_hint, N, K, c,
                                   static_cast<cudaStream_t>(stream));
}

int dsv3_moe_route(const int64_t* indices, const float* weights, int64_t T, int topk, int start, int n_local,
                   int32_t* seg, int32_t* tok, int32_t* pair_row, int32_t* pos_sorted, void* w_sorted,
                   dsv3_stream_t stream) {
    if (T < 0 || topk < 0 || n_local < 0) {
        set_last_error("moe_route: negative size");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (n_local > kRouteMaxExperts || topk > kRouteMaxTopk || T * topk >= (1ll << 31)) {
        set_last_error("moe_route: at most %d local experts, top-%d and 2^31 pairs", kRouteMaxExperts, kRouteMaxTopk);
        return DSV3_ERR_UNSUPPORTED;
    }
    if (!seg || (T * topk > 0 && (!indices || !weights || !tok || !pair_row || !pos_sorted || !w_sorted))) {
        set_last_error("moe_route: null pointer");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    moe_route_kernel<<<1, kRouteThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        indices, weights, T, topk, start, n_local, seg, tok, pair_row, pos_sorted, static_cast<__nv_bfloat16*>(w_sorted));
    DSV3_CUDA_TRY(cudaGetLastError());
    return DSV3_OK;
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
