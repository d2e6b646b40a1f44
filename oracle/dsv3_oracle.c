/*
 * CPU restatement of DeepSeek-V3's FP8 inference GEMM path (inference/kernel.py).
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against and the timed CPU baseline; nothing in the product path may
 * link, load or call it.
 *
 * Numerics follow what the reference's Triton kernels compute on a GPU:
 *   - fp32 arithmetic throughout, IEEE division (the GPU uses `div.full.f32`,
 *     which may differ from IEEE by <= 2 ulp; tests bound that difference),
 *   - fp32 -> e4m3 is round-to-nearest-even, saturating to +-448,
 *   - fp32 -> bf16 is round-to-nearest-even.
 * Each function cites the reference lines it restates.
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC (see oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* scalar format helpers                                               */
/* ------------------------------------------------------------------ */

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* fp32 -> bf16, round to nearest even; NaN stays a quiet NaN. */
static inline uint16_t f32_to_bf16_rne(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/* e4m3fn (1-4-3, bias 7, no inf, 0x7f/0xff = NaN) -> fp32, exact. */
static float e4m3_lut[256];
static int e4m3_lut_ready = 0;

static void e4m3_lut_init(void) {
    if (e4m3_lut_ready) return;
    for (int b = 0; b < 256; ++b) {
        int sign = b >> 7, e = (b >> 3) & 0xf, m = b & 7;
        float v;
        if (e == 0xf && m == 7) v = NAN;
        else if (e == 0) v = ldexpf((float)m, -9);            /* subnormal: m * 2^-9 */
        else v = ldexpf((float)(8 + m), e - 10);               /* (1 + m/8) * 2^(e-7) */
        e4m3_lut[b] = sign ? -v : v;
    }
    e4m3_lut_ready = 1;
}

/* fp32 -> e4m3fn, round to nearest even, saturate finite overflow to +-448
 * (the behaviour of PTX `cvt.rn.satfinite.e4m3x2.f32`; NaN -> 0x7f). */
static inline uint8_t f32_to_e4m3_rne_sat(float f) {
    uint32_t u = f32_bits(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return 0x7f;                          /* NaN */
    float x = bits_f32(a);
    if (x >= 448.0f) return sign | 0x7e;                       /* saturate (inf too) */
    if (x < 0.015625f) {                                       /* below 2^-6: subnormal grid 2^-9 */
        /* x * 512 is exact; rintf rounds to nearest even in the default mode */
        int q = (int)rintf(x * 512.0f);                        /* 0..8 ; 8 -> smallest normal */
        return sign | (uint8_t)q;
    }
    /* normal range: keep 3 mantissa bits */
    uint32_t mant = a & 0x7fffffu;
    int32_t e = (int32_t)(a >> 23) - 127;                      /* -6 .. 8 */
    uint32_t keep = mant >> 20;
    uint32_t rest = mant & 0xfffffu;
    uint32_t half = 0x80000u;
    if (rest > half || (rest == half && (keep & 1u))) {
        keep += 1;
        if (keep == 8) { keep = 0; e += 1; }
    }
    uint32_t code = ((uint32_t)(e + 7) << 3) | keep;
    if (code > 0x7e) code = 0x7e;                              /* 464+ rounds past 448 -> saturate */
    return sign | (uint8_t)code;
}

ORC_API float orc_e4m3_to_f32(uint8_t b) { e4m3_lut_init(); return e4m3_lut[b]; }
ORC_API uint8_t orc_f32_to_e4m3(float f) { return f32_to_e4m3_rne_sat(f); }
ORC_API uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16_rne(f); }

ORC_API void orc_f32_to_e4m3_array(const float* x, int64_t n, uint8_t* y) {
    for (int64_t i = 0; i < n; ++i) y[i] = f32_to_e4m3_rne_sat(x[i]);
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------ */
/* act_quant: inference/kernel.py:9-35 (kernel), :38-57 (wrapper)      */
/* ------------------------------------------------------------------ */
/*
 * x      : [rows, K] bf16 bit patterns, K % block == 0      (kernel.py:51-52)
 * y      : [rows, K] e4m3 bytes                              (kernel.py:53)
 * s      : [rows, K/block] fp32                              (kernel.py:54)
 * Per block of `block` consecutive elements (kernel.py:23-35):
 *   amax = max|x| ; amax = max(amax, 1e-4) ; s = amax / 448
 *   ue8m0: s = exp2(ceil(log2(s)))                            (kernel.py:29-31)
 *   y = e4m3(x / s)
 * A NaN element does not raise amax (the GPU's max.f32 drops NaN operands).
 */
ORC_API int orc_act_quant(const uint16_t* x, int64_t rows, int64_t K, int block, int ue8m0,
                          uint8_t* y, float* s) {
    if (block <= 0 || K % block != 0) return -1;
    const int64_t nb = K / block;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t b = 0; b < nb; ++b) {
            const uint16_t* xp = x + r * K + b * block;
            float amax = 0.0f;
            for (int i = 0; i < block; ++i) {
                float v = fabsf(bf16_to_f32(xp[i]));
                if (v > amax) amax = v;                        /* NaN compares false: dropped */
            }
            if (!(amax > 1e-4f)) amax = 1e-4f;
            float sc = amax / 448.0f;
            if (ue8m0) sc = exp2f(ceilf(log2f(sc)));
            uint8_t* yp = y + r * K + b * block;
            for (int i = 0; i < block; ++i) yp[i] = f32_to_e4m3_rne_sat(bf16_to_f32(xp[i]) / sc);
            s[r * nb + b] = sc;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ */
/* weight_dequant: inference/kernel.py:60-86 (kernel), :89-110         */
/* ------------------------------------------------------------------ */
/*
 * w : [N, K] e4m3 bytes ; s : [ceil(N/block), ceil(K/block)] fp32
 * y : [N, K] bf16 bits  ; y = bf16_rne(float(w) * s[n/block, k/block]) (kernel.py:83-86)
 */
ORC_API int orc_weight_dequant(const uint8_t* w, const float* s, int64_t N, int64_t K, int block,
                               uint16_t* y) {
    if (block <= 0) return -1;
    e4m3_lut_init();
    const int64_t kb = (K + block - 1) / block;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const float* srow = s + (n / block) * kb;
        for (int64_t k = 0; k < K; ++k)
            y[n * K + k] = f32_to_bf16_rne(e4m3_lut[w[n * K + k]] * srow[k / block]);
    }
    return 0;
}

/* ------------------------------------------------------------------ */
/* fp8_gemm: inference/kernel.py:118-172 (kernel), :175-196            */
/* ------------------------------------------------------------------ */
/*
 * a   : [M, K] e4m3 ; a_s : [M, ceil(K/128)] fp32
 * b   : [N, K] e4m3 ; b_s : [ceil(N/128), ceil(K/128)] fp32
 * c   : [M, N] bf16 bits
 * Per 128-wide K chunk i (kernel.py:157-166):
 *   p   = sum_k a[m, i*128+k] * b[n, i*128+k]        (exact products; summed in
 *         double and rounded once to fp32 -- the hardware's summation order is
 *         unspecified, so the exactly rounded dot is the reference point)
 *   acc = fma(p * a_s[m, i], b_s[n/128, i], acc)     (fp32)
 * c = bf16_rne(acc)                                   (kernel.py:167)
 */
ORC_API int orc_fp8_gemm(const uint8_t* a, const float* a_s, const uint8_t* b, const float* b_s,
                         int64_t M, int64_t N, int64_t K, uint16_t* c) {
    e4m3_lut_init();
    const int64_t kc = (K + 127) / 128;
    int failed = 0;
#pragma omp parallel
    {
        /* per-thread decoded copies of one A row and one B row */
        float* af = (float*)malloc((size_t)(K > 0 ? K : 1) * sizeof(float));
        float* bf = (float*)malloc((size_t)(K > 0 ? K : 1) * sizeof(float));
        if (!af || !bf) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for schedule(static)
            for (int64_t n = 0; n < N; ++n) {
                for (int64_t k = 0; k < K; ++k) bf[k] = e4m3_lut[b[n * K + k]];
                const float* bs = b_s + (n / 128) * kc;
                for (int64_t m = 0; m < M; ++m) {
                    for (int64_t k = 0; k < K; ++k) af[k] = e4m3_lut[a[m * K + k]];
                    float acc = 0.0f;
                    for (int64_t i = 0; i < kc; ++i) {
                        const int64_t k0 = i * 128;
                        const int len = (int)((K - k0) < 128 ? (K - k0) : 128);
                        double p = 0.0;   /* exact: every partial sum fits in 53 bits */
#pragma omp simd reduction(+ : p)
                        for (int k = 0; k < len; ++k) p += (double)(af[k0 + k] * bf[k0 + k]);
                        const float t = (float)p * a_s[m * kc + i];
                        acc = fmaf(t, bs[i], acc);
                    }
                    c[m * N + n] = f32_to_bf16_rne(acc);
                }
            }
        }
        free(af);
        free(bf);
    }
    return failed ? -2 : 0;
}

/* ------------------------------------------------------------------ */
/* Harness weight quantiser (the reference ships none)                 */
/* ------------------------------------------------------------------ */
/*
 * Inverse of weight_dequant in the checkpoint format (README_WEIGHTS.md:60-92):
 * per 128x128 block (edge blocks are partial), s = max(amax, 1e-4) / 448,
 * q = e4m3_rne(w / s).  w : [N, K] bf16 bits.
 */
ORC_API int orc_weight_quant(const uint16_t* w, int64_t N, int64_t K, int block,
                             uint8_t* q, float* s) {
    if (block <= 0) return -1;
    const int64_t nb = (N + block - 1) / block, kb = (K + block - 1) / block;
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t bn = 0; bn < nb; ++bn) {
        for (int64_t bk = 0; bk < kb; ++bk) {
            const int64_t n1 = (bn + 1) * block < N ? (bn + 1) * block : N;
            const int64_t k1 = (bk + 1) * block < K ? (bk + 1) * block : K;
            float amax = 0.0f;
            for (int64_t n = bn * block; n < n1; ++n)
                for (int64_t k = bk * block; k < k1; ++k) {
                    float v = fabsf(bf16_to_f32(w[n * K + k]));
                    if (v > amax) amax = v;
                }
            if (!(amax > 1e-4f)) amax = 1e-4f;
            const float sc = amax / 448.0f;
            for (int64_t n = bn * block; n < n1; ++n)
                for (int64_t k = bk * block; k < k1; ++k)
                    q[n * K + k] = f32_to_e4m3_rne_sat(bf16_to_f32(w[n * K + k]) / sc);
            s[bn * kb + bk] = sc;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ */
/* linear(): inference/model.py:131-163, FP8 branch (:158-163)         */
/* ------------------------------------------------------------------ */
/* x bf16 [M,K] -> act_quant -> fp8_gemm with (w, w_s) -> bf16 [M,N].
 * scratch_q: M*K bytes, scratch_s: M*(K/128) floats. */
ORC_API int orc_linear_fp8(const uint16_t* x, const uint8_t* w, const float* w_s,
                           int64_t M, int64_t N, int64_t K,
                           uint8_t* scratch_q, float* scratch_s, uint16_t* y) {
    int rc = orc_act_quant(x, M, K, 128, 0, scratch_q, scratch_s);
    if (rc) return rc;
    return orc_fp8_gemm(scratch_q, scratch_s, w, w_s, M, N, K, y);
}
