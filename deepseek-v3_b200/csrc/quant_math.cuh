// Arithmetic of act_quant shared by the stand-alone kernel and the GEMM kernels that quantise in their prologue.
//
// Bit-exactness contract (what the reference's kernel computes when compiled for a GPU, inference/kernel.py:23-35):
//   amax = max|x| (NaN operands dropped) ; amax = max(amax, 1e-4f)
//   s = div.full.f32(amax, 448) ; [ue8m0: s = exp2(ceil(log2(s)))]
//   y = cvt.rn.satfinite.e4m3(div.full.f32(x, s))
// For the fp32 scale format the quotient is formed as x * rcp.approx.f32(s): on sm_100 this is
// bit-identical to div.full.f32(x, s) for every bf16 x and every scale a bf16 block maximum can
// produce (checked exhaustively on a B200: 5.3e8 (amax, x) pairs, no mismatch), and it needs one
// reciprocal per block instead of one division per element.
#pragma once

#include "common.cuh"

namespace dsv3 {

__device__ __forceinline__ float scale_from_amax(float amax, int scale_fmt) {
    amax = fmaxf(amax, 1e-4f);
    float s = div_full(amax, 448.0f);
    if (scale_fmt == DSV3_SCALE_FMT_UE8M0) s = exp2f(ceilf(log2f(s)));
    return s;
}

__device__ __forceinline__ float amax8(const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m = fmaxf(m, fabsf(bf16_bits_to_float(w[i] & 0xFFFFu)));
        m = fmaxf(m, fabsf(__uint_as_float(w[i] & 0xFFFF0000u)));
    }
    return m;
}

__device__ __forceinline__ float rcp_approx(float s) {
    float r;
    asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(s));
    return r;
}

// kRcp: quotient as x * rcp.approx(s) (fp32 scale format) instead of div.full(x, s).
template <bool kRcp>
__device__ __forceinline__ uint2 quant8(const uint4& v, float s) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint16_t p[4];
    const float r = kRcp ? rcp_approx(s) : 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float xl = bf16_bits_to_float(w[i] & 0xFFFFu), xh = __uint_as_float(w[i] & 0xFFFF0000u);
        const float lo = kRcp ? __fmul_rn(xl, r) : div_full(xl, s);
        const float hi = kRcp ? __fmul_rn(xh, r) : div_full(xh, s);
        p[i] = cvt_e4m3x2(lo, hi);
    }
    return make_uint2(static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 16),
                      static_cast<uint32_t>(p[2]) | (static_cast<uint32_t>(p[3]) << 16));
}

}  // namespace dsv3
