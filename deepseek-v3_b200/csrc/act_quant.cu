// act_quant for sm_100a: per-(1 x block) FP8 e4m3 quantisation of bf16 activations.
//
// Replaces inference/kernel.py:9-35 (act_quant_kernel) and its launch at :55-56.
// The reference runs one 128-thread program per 128-element block with one element
// per thread; here a half-warp owns a block (16 lanes x 16 bytes), every thread keeps
// several independent blocks in flight, and a CTA owns a contiguous 16 KB tile of the input.
//
// Bit-exactness contract (what the reference's kernel computes when compiled for a GPU):
//   amax = max|x| (NaN operands dropped) ; amax = max(amax, 1e-4f)
//   s = div.full.f32(amax, 448) ; [ue8m0: s = exp2(ceil(log2(s)))]
//   y = cvt.rn.satfinite.e4m3(div.full.f32(x, s))
// For the fp32 scale format the quotient is formed as x * rcp.approx.f32(s): on sm_100 this is
// bit-identical to div.full.f32(x, s) for every bf16 x and every scale a bf16 block maximum can
// produce (checked exhaustively on a B200: 5.3e8 (amax, x) pairs, no mismatch), and it needs one
// reciprocal per block instead of one division per element.
#include "common.cuh"
#include "quant_math.cuh"

namespace dsv3 {

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;  // blocks in flight per half-warp per loop trip

// block_size == 128.  nblk = rows * K / 128; block b covers elements [128 b, 128 b + 128).
// A CTA owns kBlocksPerCta consecutive blocks (16 KB of input): in trip u its sixteen half-warps take
// sixteen consecutive blocks, so every load instruction of the CTA covers 4 KB of contiguous memory
// and the four trips are in flight together.  (Contiguous tiles matter: a grid-stride sweep of the same
// accesses, with every CTA touching addresses megabytes apart, ran 20-30 % slower on B200.)
constexpr int kBlocksPerCta = (kThreads / 16) * kUnroll;

__global__ void __launch_bounds__(kThreads, 4) act_quant128_kernel(const uint4* __restrict__ x, uint2* __restrict__ y,
                                                                 float* __restrict__ s, int64_t nblk, int scale_fmt) {
    griddep_launch_dependents();   // a dependent launch (the GEMM) may set itself up while this kernel runs
    griddep_wait();
    const int lane16 = threadIdx.x & 15;
    const int64_t b0 = static_cast<int64_t>(blockIdx.x) * kBlocksPerCta + (threadIdx.x >> 4);
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t b = b0 + u * (kThreads / 16);
        v[u] = (b < nblk) ? __ldcs(x + b * 16 + lane16) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t b = b0 + u * (kThreads / 16);
        float m = amax8(v[u]);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        const float sc = scale_from_amax(m, scale_fmt);
        if (b < nblk) {
            y[b * 16 + lane16] = (scale_fmt == DSV3_SCALE_FMT_FP32) ? quant8<true>(v[u], sc) : quant8<false>(v[u], sc);
            if (lane16 == 0) s[b] = sc;
        }
    }
}

// Any block size that is a multiple of 8 and at most 1024: one warp per block.
__global__ void __launch_bounds__(kThreads) act_quant_generic_kernel(const uint4* __restrict__ x,
                                                                      uint2* __restrict__ y, float* __restrict__ s,
                                                                      int64_t nblk, int groups, int scale_fmt) {
    griddep_launch_dependents();
    griddep_wait();
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * kThreads) >> 5;
    for (int64_t b = warp; b < nblk; b += nwarps) {
        uint4 v[4];
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int g = lane + 32 * i;
            v[i] = (g < groups) ? x[b * groups + g] : make_uint4(0, 0, 0, 0);
            m = fmaxf(m, amax8(v[i]));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float sc = scale_from_amax(m, scale_fmt);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int g = lane + 32 * i;
            if (g < groups) y[b * groups + g] = quant8<false>(v[i], sc);
        }
        if (lane == 0) s[b] = sc;
    }
}

// SwiGLU followed by act_quant in one pass: h = bf16(bf16(silu(a)) * b), then h is quantised per 128 values.
// Replaces the three launches `F.silu(w1(x)) * w3(x)` + act_quant in front of w2 (model.py:532, 633 and 158-159) and
// keeps their rounding points: silu is evaluated in fp32 as a / (1 + exp(-a)) and rounded to bf16, the product is
// formed in fp32 and rounded to bf16 (what the framework's bf16 kernels do), and the quantisation of h is the
// arithmetic of act_quant128_kernel.  h itself is never written.
__device__ __forceinline__ uint32_t swiglu2(uint32_t a2, uint32_t b2) {
    const float al = bf16_bits_to_float(a2 & 0xFFFFu), ah = __uint_as_float(a2 & 0xFFFF0000u);
    const float bl = bf16_bits_to_float(b2 & 0xFFFFu), bh = __uint_as_float(b2 & 0xFFFF0000u);
    const float sl = __bfloat162float(__float2bfloat16_rn(al / (1.0f + expf(-al))));
    const float sh = __bfloat162float(__float2bfloat16_rn(ah / (1.0f + expf(-ah))));
    return pack_bf16x2(sl * bl, sh * bh);
}

__global__ void __launch_bounds__(kThreads, 4) swiglu_quant128_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b,
                                                                    uint2* __restrict__ y, float* __restrict__ s, int64_t nblk,
                                                                    int scale_fmt) {
    griddep_launch_dependents();
    griddep_wait();
    const int lane16 = threadIdx.x & 15;
    const int64_t b0 = static_cast<int64_t>(blockIdx.x) * kBlocksPerCta + (threadIdx.x >> 4);
    uint4 va[kUnroll], vb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t blk = b0 + u * (kThreads / 16);
        va[u] = (blk < nblk) ? __ldcs(a + blk * 16 + lane16) : make_uint4(0, 0, 0, 0);
        vb[u] = (blk < nblk) ? __ldcs(b + blk * 16 + lane16) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t blk = b0 + u * (kThreads / 16);
        const uint4 h = make_uint4(swiglu2(va[u].x, vb[u].x), swiglu2(va[u].y, vb[u].y), swiglu2(va[u].z, vb[u].z),
                                   swiglu2(va[u].w, vb[u].w));
        float m = amax8(h);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        const float sc = scale_from_amax(m, scale_fmt);
        if (blk < nblk) {
            y[blk * 16 + lane16] = (scale_fmt == DSV3_SCALE_FMT_FP32) ? quant8<true>(h, sc) : quant8<false>(h, sc);
            if (lane16 == 0) s[blk] = sc;
        }
    }
}

}  // namespace

int launch_act_quant(const void* x, int64_t rows, int64_t K, int block_size, int scale_fmt, void* y, float* s,
                     cudaStream_t stream) {
    const int64_t nblk = rows * (K / block_size);
    if (nblk == 0) return DSV3_OK;
    const int64_t cap = static_cast<int64_t>(num_sms()) * 8;  // 8 resident CTAs of 256 threads per SM
    if (block_size == 128) {
        const int64_t grid = (nblk + kBlocksPerCta - 1) / kBlocksPerCta;
        if (grid >= (1ll << 31)) {
            set_last_error("act_quant: too many blocks (%lld)", static_cast<long long>(nblk));
            return DSV3_ERR_UNSUPPORTED;
        }
        DSV3_CUDA_TRY(launch_dependent(act_quant128_kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0, stream,
                                       static_cast<const uint4*>(x), static_cast<uint2*>(y), s, nblk, scale_fmt));
    } else {
        const int64_t per_cta = kThreads / 32;
        int64_t grid = (nblk + per_cta - 1) / per_cta;
        if (grid > cap) grid = cap;
        DSV3_CUDA_TRY(launch_dependent(act_quant_generic_kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0, stream,
                                       static_cast<const uint4*>(x), static_cast<uint2*>(y), s, nblk, block_size / 8,
                                       scale_fmt));
    }
    DSV3_CUDA_TRY(cudaGetLastError());
    return DSV3_OK;
}

int launch_swiglu_quant(const void* a, const void* b, int64_t rows, int64_t K, int scale_fmt, void* y, float* s,
                        cudaStream_t stream) {
    const int64_t nblk = rows * (K / 128);
    if (nblk == 0) return DSV3_OK;
    const int64_t grid = (nblk + kBlocksPerCta - 1) / kBlocksPerCta;
    if (grid >= (1ll << 31)) {
        set_last_error("swiglu_quant: too many blocks (%lld)", static_cast<long long>(nblk));
        return DSV3_ERR_UNSUPPORTED;
    }
    DSV3_CUDA_TRY(launch_dependent(swiglu_quant128_kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0, stream,
                                   static_cast<const uint4*>(a), static_cast<const uint4*>(b), static_cast<uint2*>(y), s, nblk,
                                   scale_fmt));
    return DSV3_OK;
}

}  // namespace dsv3
