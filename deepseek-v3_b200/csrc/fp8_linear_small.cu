// Decode-sized Linear for sm_100a (at most 16 token rows): act_quant folded into the GEMM, one launch.
//
// Replaces the FP8 branch of linear(), inference/model.py:158-160 (act_quant, kernel.py:38-57, followed by
// fp8_gemm, kernel.py:175-196), for the rows of one decode step.  With a handful of tokens the Linear is a stream
// of weight bytes; what it costs beyond that stream is fixed overhead, and the two-launch form pays it twice and
// sends the FP8 activations through HBM in between.  The tcgen05 kernels also carry set-up this regime cannot
// amortise over 2-15 MB of weights (TMEM allocation, tensor maps, mbarrier rings, a split-K workspace with
// tickets).  This kernel has none of it:
//
//   * a warp owns 16 weight rows and a range of 128-wide K chunks; every lane fetches 16 contiguous bytes of a
//     row straight into registers (ld.global, four chunks in flight per warp), which IS the A fragment of
//     mma.sync.m16n8k32 (e4m3 x e4m3 -> fp32) once the K positions inside a 64-byte slab are permuted the same way
//     for both operands (lane t of a quad holds bytes 16t..16t+15: the first mma takes bytes 0-7, the second 8-15);
//   * the token rows (8 or 16, zero-padded) are the N side of the mma.  The CTA quantises its K range of the
//     activations once, bit-identically to act_quant (same arithmetic, quant_math.cuh), into shared memory, or
//     copies already quantised activations there; the fragments are 16-byte shared-memory loads;
//   * every chunk's product is scaled as the reference does, acc = fma(p * a_s, b_s, acc) (kernel.py:162);
//   * K is split over the warps of a CTA and over the CTAs of a cluster (at most 8); partial sums meet in the
//     shared memory of the cluster's first CTA (st.shared::cluster), which adds them in a fixed order, so the
//     result is deterministic and no global scratch or atomics are involved.
//
// No wait in this kernel can hang: the only synchronisation is __syncthreads and the cluster barrier, which every
// thread reaches unconditionally.
#include <cuda.h>

#include "common.cuh"
#include "gemm_plan.cuh"
#include "quant_math.cuh"

namespace dsv3 {

namespace {

constexpr int kChunkK = 128;    // K elements (= bytes) per scale block
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kRing = 4;        // weight chunks in flight per warp (16 x 16-byte loads per lane)
constexpr int kRowPad = 64;     // bytes between the staged token rows beyond the K range: the 8 lanes of one
                                // shared-memory phase (two token rows x four 16-byte pieces) then hit 8 different bank groups

struct SmallParams {
    const uint4* x;          // bf16 [M, K], 8 values per uint4 (quantised here)       -- or nullptr
    const uint8_t* a;        // e4m3 [M, K], already quantised                         -- used when x is null
    const float* a_s;        // fp32 [M, kc]
    const uint8_t* w;        // e4m3 [N, K]
    const float* w_s;        // fp32 [ceil(N/128), kc]
    __nv_bfloat16* c;        // bf16 [M, N]
    int M, N, K, kc;
    int cpc;                 // K chunks per CTA of a cluster
    int csize;               // CTAs per cluster (K splits across CTAs)
    int scale_fmt;
};

__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void prefetch_l2(const void* ptr) { asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr)); }

__device__ __forceinline__ void st_cluster_f32(uint32_t addr_cluster, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr_cluster), "f"(v) : "memory");
}

constexpr size_t align16(size_t v) { return (v + 15) & ~static_cast<size_t>(15); }

// WR x WK = kWarps: WR row tiles of 16 weight rows per CTA, WK warps share a row tile and split the CTA's K range.
// MT: token groups of 8 (1 or 2).  kFused: activations arrive as bf16 and are quantised here.
template <int WR, int WK, int MT, bool kFused>
__global__ void __launch_bounds__(kThreads) fp8_linear_small_kernel(const SmallParams p) {
    static_assert(WR * WK == kWarps, "warp layout");
    constexpr int TOK = 8 * MT;
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t rank = cluster_ctarank();
    const int rowgroup = static_cast<int>(blockIdx.x) / p.csize;
    const int wr = warp / WK, wk = warp % WK;
    const int r0 = (rowgroup * WR + wr) * 16;
    const int N = p.N, K = p.K, kc = p.kc, cpc = p.cpc;
    const int c0 = static_cast<int>(rank) * cpc;
    const int c1 = min(kc, c0 + cpc);
    const int n_cta = max(c1 - c0, 0);                   // chunks of this CTA
    const int seg = (n_cta + WK - 1) / WK;
    const int w0 = c0 + wk * seg;
    const int n_w = max(min(c1, w0 + seg) - w0, 0);      // chunks of this warp: [w0, w0 + n_w)

    const int row_bytes = cpc * kChunkK + kRowPad;
    uint8_t* xq_s = smem;                                                        // [TOK][row_bytes]
    float* xs_s = reinterpret_cast<float*>(smem + align16(static_cast<size_t>(TOK) * row_bytes));   // [TOK][cpc]
    float* bs_s = xs_s + TOK * cpc;                                              // [WR][cpc]
    float* slots = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bs_s) + align16(static_cast<size_t>(WR) * cpc * 4));
    // slots: [csize * WK][WR][16][TOK] partial sums, used in the cluster's first CTA

    // rows of this lane (clamped at the edge: the loads stay inside the matrix, the results are masked)
    const uint8_t* wa = p.w + static_cast<int64_t>(min(r0 + g, N - 1)) * K + 16 * t;
    const uint8_t* wb = p.w + static_cast<int64_t>(min(r0 + g + 8, N - 1)) * K + 16 * t;
    // Programmatic dependent launch: the weights are constants of the model, so pulling this warp's first chunks
    // into L2 may overlap the tail of the kernel that produces the activations (L2 is the point of coherence: if
    // that kernel were still writing the weights, the loads after the wait would see its data all the same).
    griddep_launch_dependents();
    if (t == 0) {
        for (int s = 0; s < kRing && s < n_w; ++s) {
            prefetch_l2(wa + static_cast<int64_t>(w0 + s) * kChunkK);
            prefetch_l2(wb + static_cast<int64_t>(w0 + s) * kChunkK);
        }
    }
    griddep_wait();

    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    auto load_chunk = [&](uint4 (&buf)[4], int c) {
        const int64_t off = static_cast<int64_t>(c) * kChunkK;
        const int k = c * kChunkK + 16 * t;                  // K % 16 == 0: a 16-byte piece is inside or outside
        const bool in0 = k + 16 <= K, in1 = k + 64 + 16 <= K;
        buf[0] = in0 ? __ldcs(reinterpret_cast<const uint4*>(wa + off)) : zero4;
        buf[1] = in0 ? __ldcs(reinterpret_cast<const uint4*>(wb + off)) : zero4;
        buf[2] = in1 ? __ldcs(reinterpret_cast<const uint4*>(wa + off + 64)) : zero4;
        buf[3] = in1 ? __ldcs(reinterpret_cast<const uint4*>(wb + off + 64)) : zero4;
    };
    uint4 ring[kRing][4];
#pragma unroll
    for (int s = 0; s < kRing; ++s)
        if (s < n_w) load_chunk(ring[s], w0 + s);

    // ---- the CTA's K range of the activations: FP8 bytes and scales into shared memory
    if constexpr (kFused) {
        // a half-warp per (token, chunk) block: 16 lanes x 8 bf16, as in the stand-alone act_quant kernel.  (Measured
        // on B200: fetching several blocks per half-warp at once, or staging the bf16 rows with asynchronous copies
        // first, helps at 8 tokens but costs registers or shared memory that the single-token case pays for; with
        // more than a few tokens the per-CTA quantisation is the wrong trade anyway, see dsv3_fp8_linear's callers.)
        const int l16 = threadIdx.x & 15;
        const int nblk = p.M * n_cta;
        for (int b0 = (threadIdx.x >> 5) * 2; b0 < nblk; b0 += kThreads / 16) {     // warp-uniform trip count
            const int b = b0 + ((threadIdx.x >> 4) & 1);
            const bool valid = b < nblk;
            const int m = valid ? b / n_cta : 0;
            const int cl = valid ? b - m * n_cta : 0;
            const uint4 v = valid ? __ldg(p.x + (static_cast<int64_t>(m) * K + static_cast<int64_t>(c0 + cl) * kChunkK) / 8 + l16)
                                  : zero4;
            float mx = amax8(v);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            const float sc = scale_from_amax(mx, p.scale_fmt);
            if (valid) {
                const uint2 q = (p.scale_fmt == DSV3_SCALE_FMT_FP32) ? quant8<true>(v, sc) : quant8<false>(v, sc);
                *reinterpret_cast<uint2*>(xq_s + m * row_bytes + cl * kChunkK + l16 * 8) = q;
                if (l16 == 0) xs_s[m * cpc + cl] = sc;
            }
        }
    } else {
        // already quantised activations: asynchronous 16-byte copies, all in flight at once
        const int pieces = n_cta * (kChunkK / 16);               // 16-byte pieces per token row
        const uint32_t xq0 = smem_u32(xq_s);
        for (int idx = threadIdx.x; idx < p.M * pieces; idx += kThreads) {
            const int m = idx / pieces, pc = idx - m * pieces;
            const int k = c0 * kChunkK + pc * 16;
            if (k + 16 <= K) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(xq0 + m * row_bytes + pc * 16),
                             "l"(p.a + static_cast<int64_t>(m) * K + k)
                             : "memory");
            } else {
                *reinterpret_cast<uint4*>(xq_s + m * row_bytes + pc * 16) = zero4;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        for (int idx = threadIdx.x; idx < p.M * n_cta; idx += kThreads) {
            const int m = idx / n_cta, cl = idx - m * n_cta;
            xs_s[m * cpc + cl] = __ldg(p.a_s + static_cast<int64_t>(m) * kc + c0 + cl);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    // token rows beyond M multiply as zeros
    {
        const int pieces = n_cta * (kChunkK / 16);
        for (int idx = threadIdx.x; idx < (TOK - p.M) * pieces; idx += kThreads) {
            const int m = p.M + idx / pieces, pc = idx % pieces;
            *reinterpret_cast<uint4*>(xq_s + m * row_bytes + pc * 16) = zero4;
        }
        for (int idx = threadIdx.x; idx < (TOK - p.M) * n_cta; idx += kThreads)
            xs_s[(p.M + idx / n_cta) * cpc + idx % n_cta] = 0.0f;
    }
    // weight scales of the CTA's row tiles (a 16-row tile lies inside one 128-row scale block)
    for (int idx = threadIdx.x; idx < WR * n_cta; idx += kThreads) {
        const int w_ = idx / n_cta, cl = idx - w_ * n_cta;
        const int rb = min((rowgroup * WR + w_) * 16, N - 1) / 128;
        bs_s[w_ * cpc + cl] = __ldg(p.w_s + static_cast<int64_t>(rb) * kc + c0 + cl);
    }
    __syncthreads();

    // ---- stream the weights
    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;
    for (int i0 = 0; i0 < n_w; i0 += kRing) {
#pragma unroll
        for (int s = 0; s < kRing; ++s) {
            if (i0 + s < n_w) {
                const int c = w0 + i0 + s;
                const int cl = c - c0;
                const float bs = bs_s[wr * cpc + cl];
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    const uint8_t* xr = xq_s + (8 * j + g) * row_bytes + cl * kChunkK + 16 * t;
                    const uint4 f0 = *reinterpret_cast<const uint4*>(xr);
                    const uint4 f1 = *reinterpret_cast<const uint4*>(xr + 64);
                    float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    mma_e4m3(part, ring[s][0].x, ring[s][1].x, ring[s][0].y, ring[s][1].y, f0.x, f0.y);
                    mma_e4m3(part, ring[s][0].z, ring[s][1].z, ring[s][0].w, ring[s][1].w, f0.z, f0.w);
                    mma_e4m3(part, ring[s][2].x, ring[s][3].x, ring[s][2].y, ring[s][3].y, f1.x, f1.y);
                    mma_e4m3(part, ring[s][2].z, ring[s][3].z, ring[s][2].w, ring[s][3].w, f1.z, f1.w);
                    // part[0..1]: weight row g, tokens 8j+2t, 8j+2t+1; part[2..3]: weight row g+8, same tokens
                    const float as0 = xs_s[(8 * j + 2 * t) * cpc + cl], as1 = xs_s[(8 * j + 2 * t + 1) * cpc + cl];
                    acc[j][0] = fmaf(part[0] * as0, bs, acc[j][0]);
                    acc[j][1] = fmaf(part[1] * as1, bs, acc[j][1]);
                    acc[j][2] = fmaf(part[2] * as0, bs, acc[j][2]);
                    acc[j][3] = fmaf(part[3] * as1, bs, acc[j][3]);
                }
                if (i0 + s + kRing < n_w) load_chunk(ring[s], c + kRing);
            }
        }
    }

    // ---- partial sums of all K splits meet in the first CTA of the cluster
    {
        const uint32_t base = mapa_shared(smem_u32(slots), 0);
        const int slot = static_cast<int>(rank) * WK + wk;
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = g + ((i & 2) ? 8 : 0), tok = 8 * j + 2 * t + (i & 1);
                st_cluster_f32(base + 4u * static_cast<uint32_t>(((slot * WR + wr) * 16 + row) * TOK + tok), acc[j][i]);
            }
    }
    if (p.csize > 1) {
        cluster_arrive();
        cluster_wait();
    } else {
        __syncthreads();      // launched without a cluster: the slots are this CTA's own
    }
    if (rank == 0) {
        const int n_slots = p.csize * WK;
        constexpr int ROWS = WR * 16;
        for (int idx = threadIdx.x; idx < ROWS * p.M; idx += kThreads) {
            const int tok = idx / ROWS, rw = idx - tok * ROWS;
            const int n = rowgroup * ROWS + rw;
            if (n >= N) continue;
            float sum = 0.0f;
            for (int s = 0; s < n_slots; ++s) sum += slots[(s * ROWS + rw) * TOK + tok];
            p.c[static_cast<int64_t>(tok) * N + n] = __float2bfloat16_rn(sum);
        }
    }
}

template <int WR, int WK, int MT, bool kFused>
int launch_variant(const SmallParams& prm, int rowgroups, size_t smem_bytes, cudaStream_t stream) {
    auto kern = fp8_linear_small_kernel<WR, WK, MT, kFused>;
    static size_t configured[64] = {};
    int dev = 0;
    DSV3_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_last_error("fp8_linear: device ordinal %d is outside the supported range", dev);
        return DSV3_ERR_UNSUPPORTED;
    }
    if (smem_bytes > 48 * 1024 && configured[dev] < smem_bytes) {
        DSV3_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes)));
        configured[dev] = smem_bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(rowgroups * prm.csize));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    // attributes: dependent launch first, the cluster dimension only when K is split over more than one CTA (a
    // cluster launch, even of one CTA, takes a slower path through the launch machinery)
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (prm.csize > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = static_cast<unsigned>(prm.csize);
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    DSV3_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, prm));
    return DSV3_OK;
}

}  // namespace

bool small_linear_supported(const void* act, const void* w, const void* c, int64_t M, int64_t N, int64_t K, bool fused) {
    const bool aligned = (reinterpret_cast<uintptr_t>(act) % 16) == 0 && (reinterpret_cast<uintptr_t>(w) % 16) == 0 &&
                         (reinterpret_cast<uintptr_t>(c) % 2) == 0;
    return aligned && M >= 1 && M <= 16 && N >= 1 && N < (1ll << 31) && K >= 16 && K < (1ll << 24) &&
           (K % (fused ? 128 : 16)) == 0;
}

// x != nullptr: fused (bf16 activations); otherwise (a, a_s) are the quantised activations.
int launch_fp8_linear_small(const void* x, const void* a, const float* a_s, const void* w, const float* w_s, int64_t M,
                            int64_t N, int64_t K, int scale_fmt, void* c, cudaStream_t stream) {
    SmallParams prm;
    prm.x = static_cast<const uint4*>(x);
    prm.a = static_cast<const uint8_t*>(a);
    prm.a_s = a_s;
    prm.w = static_cast<const uint8_t*>(w);
    prm.w_s = w_s;
    prm.c = static_cast<__nv_bfloat16*>(c);
    prm.M = static_cast<int>(M);
    prm.N = static_cast<int>(N);
    prm.K = static_cast<int>(K);
    prm.kc = static_cast<int>((K + kChunkK - 1) / kChunkK);
    prm.scale_fmt = scale_fmt;
    // Layout: few weight rows -> a CTA takes one 16-row tile and its four warps split K (more CTAs, and every CTA
    // quantises only its own K range); many rows -> a CTA takes four row tiles that share the staged activations.
    const bool narrow = N <= 4096;
    const int wr = narrow ? 1 : 4, wk = narrow ? 4 : 1;
    const int rowgroups = static_cast<int>((N + 16 * wr - 1) / (16 * wr));
    // K splits across the CTAs of a cluster: enough CTAs for two per SM, at least 1.5 chunks per warp
    int csize = 1;
    while (csize < 8 && rowgroups * csize < 2 * num_sms() && prm.kc >= 3 * csize * wk) csize *= 2;
    prm.csize = csize;
    prm.cpc = (prm.kc + csize - 1) / csize;
    const int mt = M <= 8 ? 1 : 2;
    const int tok = 8 * mt;
    const size_t smem = align16(static_cast<size_t>(tok) * (prm.cpc * kChunkK + kRowPad)) + static_cast<size_t>(tok) * prm.cpc * 4 +
                        align16(static_cast<size_t>(wr) * prm.cpc * 4) + align16(static_cast<size_t>(csize) * wk * wr * 16 * tok * 4) + 16;
    if (smem > 200 * 1024) {
        set_last_error("fp8_linear: K=%lld is too long for the decode kernel's staging buffer", static_cast<long long>(K));
        return DSV3_ERR_UNSUPPORTED;
    }
    const bool fused = x != nullptr;
#define DSV3_SMALL_CASE(WR_, WK_, MT_, F_) return launch_variant<WR_, WK_, MT_, F_>(prm, rowgroups, smem, stream)
    if (narrow) {
        if (mt == 1) { if (fused) DSV3_SMALL_CASE(1, 4, 1, true); else DSV3_SMALL_CASE(1, 4, 1, false); }
        else         { if (fused) DSV3_SMALL_CASE(1, 4, 2, true); else DSV3_SMALL_CASE(1, 4, 2, false); }
    } else {
        if (mt == 1) { if (fused) DSV3_SMALL_CASE(4, 1, 1, true); else DSV3_SMALL_CASE(4, 1, 1, false); }
        else         { if (fused) DSV3_SMALL_CASE(4, 1, 2, true); else DSV3_SMALL_CASE(4, 1, 2, false); }
    }
#undef DSV3_SMALL_CASE
}

}  // namespace dsv3
