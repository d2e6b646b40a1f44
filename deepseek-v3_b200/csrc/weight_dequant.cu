// weight_dequant / weight_quant for sm_100a.
//
// weight_dequant replaces inference/kernel.py:60-86 (weight_dequant_kernel) and its
// launch at :108-109: y[n,k] = bf16_rn(float(w[n,k]) * s[n/block, k/block]).  The
// reference moves one byte per load; here a thread converts 8 FP8 bytes (one 8-byte load)
// into 8 bf16 values (one 16-byte store) and every CTA owns one contiguous tile.
//
// weight_quant is the harness-side inverse (the reference ships none): per 128x128
// block s = max(amax,1e-4)/448 with IEEE division, q = e4m3_rn(w / s).
#include "common.cuh"

namespace dsv3 {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ uint4 dequant8(uint32_t lo, uint32_t hi, float s) {
    const float2 a = e4m3x2_to_float2(static_cast<uint16_t>(lo & 0xFFFFu));
    const float2 b = e4m3x2_to_float2(static_cast<uint16_t>(lo >> 16));
    const float2 c = e4m3x2_to_float2(static_cast<uint16_t>(hi & 0xFFFFu));
    const float2 d = e4m3x2_to_float2(static_cast<uint16_t>(hi >> 16));
    return make_uint4(pack_bf16x2(__fmul_rn(a.x, s), __fmul_rn(a.y, s)), pack_bf16x2(__fmul_rn(b.x, s), __fmul_rn(b.y, s)),
                      pack_bf16x2(__fmul_rn(c.x, s), __fmul_rn(c.y, s)), pack_bf16x2(__fmul_rn(d.x, s), __fmul_rn(d.y, s)));
}

constexpr int kVecUnroll = 4;   // independent 8-byte loads in flight per thread

// K % 8 == 0 and a power-of-two block size >= 8: an 8-element group never straddles a scale block.
// A thread converts 8 FP8 bytes (one 8-byte load) into 8 bf16 values (one 16-byte store), so a warp reads
// 256 and writes 512 contiguous bytes per instruction.  A CTA owns one contiguous tile of
// kThreads * kVecUnroll groups (8 KB in, 16 KB out): measured on B200, contiguous tiles run at 6.3 TB/s
// where a grid-stride sweep of the same accesses (every CTA touching addresses megabytes apart) reached 4.7.
__global__ void __launch_bounds__(kThreads, 8) weight_dequant_vec_kernel(const uint2* __restrict__ w,
                                                                       const float* __restrict__ s,
                                                                       uint4* __restrict__ y, uint32_t total,
                                                                       FastDiv row_div, uint32_t block_shift,
                                                                       uint32_t kb) {
    const uint32_t base = blockIdx.x * (kThreads * kVecUnroll) + threadIdx.x;
    uint2 v[kVecUnroll];
    float sc[kVecUnroll];
#pragma unroll
    for (int u = 0; u < kVecUnroll; ++u) {
        const uint32_t g = base + u * kThreads;
        if (g < total) {
            v[u] = __ldg(w + g);
            const uint32_t n = fast_div(g, row_div);
            const uint32_t k = (g - n * row_div.d) << 3;
            sc[u] = __ldg(s + static_cast<size_t>(n >> block_shift) * kb + (k >> block_shift));
        }
    }
#pragma unroll
    for (int u = 0; u < kVecUnroll; ++u) {
        const uint32_t g = base + u * kThreads;
        if (g < total) y[g] = dequant8(v[u].x, v[u].y, sc[u]);
    }
}

// Any K / alignment / block size: one element per thread.
__global__ void __launch_bounds__(kThreads) weight_dequant_scalar_kernel(const uint8_t* __restrict__ w,
                                                                          const float* __restrict__ s,
                                                                          __nv_bfloat16* __restrict__ y, int64_t N,
                                                                          int64_t K, int block, int64_t kb) {
    const int64_t total = N * K;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
        const int64_t n = i / K, k = i - n * K;
        const float2 f = e4m3x2_to_float2(static_cast<uint16_t>(w[i]));
        y[i] = __float2bfloat16_rn(__fmul_rn(f.x, s[(n / block) * kb + (k / block)]));
    }
}

// One CTA per 128x128 block; thread t owns 16-byte column segment (t % 8) of rows t/8, t/8+32, ...
__global__ void __launch_bounds__(kThreads) weight_quant_kernel(const __nv_bfloat16* __restrict__ w,
                                                                 uint8_t* __restrict__ q, float* __restrict__ s,
                                                                 int64_t N, int64_t K, int64_t kb) {
    __shared__ float red[kThreads / 32];
    const int64_t n0 = static_cast<int64_t>(blockIdx.y) * 128, k0 = static_cast<int64_t>(blockIdx.x) * 128;
    float m = 0.0f;
    for (int e = threadIdx.x; e < 128 * 128; e += kThreads) {
        const int64_t n = n0 + (e >> 7), k = k0 + (e & 127);
        if (n < N && k < K) m = fmaxf(m, fabsf(__bfloat162float(w[n * K + k])));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, red[i]);
    const float sc = __fdiv_rn(fmaxf(m, 1e-4f), 448.0f);
    for (int e = threadIdx.x; e < 128 * 128; e += kThreads) {
        const int64_t n = n0 + (e >> 7), k = k0 + (e & 127);
        if (n < N && k < K) {
            const float v = __fdiv_rn(__bfloat162float(w[n * K + k]), sc);
            q[n * K + k] = static_cast<uint8_t>(cvt_e4m3x2(v, 0.0f) & 0xFFu);
        }
    }
    if (threadIdx.x == 0) s[static_cast<int64_t>(blockIdx.y) * kb + blockIdx.x] = sc;
}

}  // namespace

int launch_weight_dequant(const void* w, const float* s, int64_t N, int64_t K, int block, void* y,
                          cudaStream_t stream) {
    if (N == 0 || K == 0) return DSV3_OK;
    const int64_t kb = (K + block - 1) / block;
    const int64_t cap = static_cast<int64_t>(num_sms()) * 8;
    const bool pow2 = (block & (block - 1)) == 0;
    const int64_t total = N * (K >> 3);
    const bool vec = (K % 8 == 0) && pow2 && block >= 8 && (reinterpret_cast<uintptr_t>(w) % 8 == 0) &&
                     (reinterpret_cast<uintptr_t>(y) % 16 == 0) && total < (1ll << 32) - (1ll << 20) && kb < (1ll << 31);
    if (vec) {
        const int64_t per_cta = static_cast<int64_t>(kThreads) * kVecUnroll;
        const int64_t grid = (total + per_cta - 1) / per_cta;
        const FastDiv fd = make_fast_div(static_cast<uint32_t>(K >> 3));
        uint32_t bshift = 0;
        while ((1 << bshift) < block) ++bshift;
        weight_dequant_vec_kernel<<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
            static_cast<const uint2*>(w), s, static_cast<uint4*>(y), static_cast<uint32_t>(total), fd, bshift,
            static_cast<uint32_t>(kb));
    } else {
        int64_t grid = (N * K + kThreads - 1) / kThreads;
        if (grid > cap) grid = cap;
        weight_dequant_scalar_kernel<<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
            static_cast<const uint8_t*>(w), s, static_cast<__nv_bfloat16*>(y), N, K, block, kb);
    }
    DSV3_CUDA_TRY(cudaGetLastError());
    return DSV3_OK;
}

int launch_weight_quant(const void* w, int64_t N, int64_t K, void* q, float* s, cudaStream_t stream) {
    if (N == 0 || K == 0) return DSV3_OK;
    const int64_t nb = (N + 127) / 128, kb = (K + 127) / 128;
    if (nb > 65535) {
        set_last_error("weight_quant: N=%lld exceeds the grid limit", static_cast<long long>(N));
        return DSV3_ERR_UNSUPPORTED;
    }
    dim3 grid(static_cast<unsigned>(kb), static_cast<unsigned>(nb));
    weight_quant_kernel<<<grid, kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(w),
                                                       static_cast<uint8_t*>(q), s, N, K, kb);
    DSV3_CUDA_TRY(cudaGetLastError());
    return DSV3_OK;
}

}  // namespace dsv3
