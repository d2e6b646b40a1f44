// fp8_gemm, CUDA-core tiled kernel: accepts every shape (any M, N, K, any alignment).
//
// Same arithmetic as inference/kernel.py:145-172: per 128-wide K chunk an fp32 dot of
// the decoded FP8 operands, scaled by a_s[m, chunk] * b_s[n/128, chunk], accumulated in
// fp32, cast to bf16.  It serves the shapes the tensor-core kernels cannot take
// (K not a multiple of 16, unaligned pointers) and is the on-device cross-check for them.
#include "common.cuh"

namespace dsv3 {

namespace {

constexpr int kTile = 64;   // output tile is kTile x kTile
constexpr int kSub = 32;    // K elements staged per step
constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads) fp8_gemm_simple_kernel(const uint8_t* __restrict__ a,
                                                                    const float* __restrict__ a_s,
                                                                    const uint8_t* __restrict__ b,
                                                                    const float* __restrict__ b_s,
                                                                    __nv_bfloat16* __restrict__ c, int64_t M, int64_t N,
                                                                    int64_t K) {
    __shared__ float As[kSub][kTile + 4];
    __shared__ float Bs[kSub][kTile + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTile, n0 = static_cast<int64_t>(blockIdx.x) * kTile;
    const int64_t kc = (K + 127) / 128;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int64_t ch = 0; ch < kc; ++ch) {
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.0f;

        for (int sub = 0; sub < 128 / kSub; ++sub) {
            const int64_t kbase = ch * 128 + sub * kSub;
            // stage 64 x 32 bytes of each operand, decoded to fp32, transposed to [k][row]
            for (int e = threadIdx.x; e < kTile * kSub; e += kThreads) {
                const int r = e / kSub, kk = e % kSub;
                const int64_t k = kbase + kk;
                float av = 0.0f, bv = 0.0f;
                if (k < K) {
                    if (m0 + r < M) av = e4m3x2_to_float2(static_cast<uint16_t>(a[(m0 + r) * K + k])).x;
                    if (n0 + r < N) bv = e4m3x2_to_float2(static_cast<uint16_t>(b[(n0 + r) * K + k])).x;
                }
                As[kk][r] = av;
                Bs[kk][r] = bv;
            }
            __syncthreads();
#pragma unroll 8
            for (int kk = 0; kk < kSub; ++kk) {
                float av[4], bv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) part[i][j] = fmaf(av[i], bv[j], part[i][j]);
            }
            __syncthreads();
        }
        // promotion: acc += (part * a_s[m]) * b_s[n/128]   (kernel.py:162)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t m = m0 + ty * 4 + i;
            const float as = (m < M) ? a_s[m * kc + ch] : 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int64_t n = n0 + tx * 4 + j;
                const float bs = (n < N) ? b_s[(n / 128) * kc + ch] : 0.0f;
                acc[i][j] = fmaf(part[i][j] * as, bs, acc[i][j]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t n = n0 + tx * 4 + j;
            if (n < N) c[m * N + n] = __float2bfloat16_rn(acc[i][j]);
        }
    }
}

}  // namespace

int launch_fp8_gemm_simple(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N,
                           int64_t K, void* c, cudaStream_t stream) {
    const int64_t gm = (M + kTile - 1) / kTile, gn = (N + kTile - 1) / kTile;
    if (gm > 65535) {
        set_last_error("fp8_gemm (CUDA-core kernel): M=%lld exceeds the grid limit", static_cast<long long>(M));
        return DSV3_ERR_UNSUPPORTED;
    }
    dim3 grid(static_cast<unsigned>(gn), static_cast<unsigned>(gm));
    fp8_gemm_simple_kernel<<<grid, kThreads, 0, stream>>>(static_cast<const uint8_t*>(a), a_s,
                                                          static_cast<const uint8_t*>(b), b_s,
                                                          static_cast<__nv_bfloat16*>(c), M, N, K);
    DSV3_CUDA_TRY(cudaGetLastError());
    return DSV3_OK;
}

}  // namespace dsv3
