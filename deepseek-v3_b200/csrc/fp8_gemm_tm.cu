// fp8_gemm for sm_100a, token-major tiles (M > 128): TMA-fed, warp-specialised, persistent tcgen05 kernel in
// which two CTAs (a cluster of two SMs) work on one 256 x 128 tile, with software promotion of every 128-wide
// K chunk.
//
// Replaces inference/kernel.py:118-172 (fp8_gemm_kernel) and its launch at :194-195 for prefill-sized M.
//
// Why pairs.  The scales are fp32 (a_s per token per chunk, b_s per 128 x 128 weight block), so every chunk's
// product has to leave the tensor core's accumulator memory and be folded into fp32 registers as
// acc += dot * (a_s * b_s) (kernel.py:162).  That fixes the accumulator tile of one SM at 128 x 128: TMEM holds
// four such chunk products and the register file one fp32 accumulator tile plus the read-back buffers.  With
// one SM per tile every 256 tensor-core cycles need 32 KB of operands, and what the kernel then runs into is the
// operand stream: shared memory holds about six chunks, the load latency from L2 is over a microsecond, and the
// measured time follows the bytes in flight (three 64 KB stages: 560 us on M 4096, N 18432, K 7168; two stages:
// 664 us; no MMAs, read-back or FMAs at all: 415 us).  A pair of SMs running tcgen05.mma.cta_group::2 (M = 256)
// shares the weight tile: each CTA loads its own 128 token rows and HALF of the 128 weight rows, 24 KB per chunk
// instead of 32, so the same shared memory holds eight chunks and a quarter of the L2 traffic is gone, while
// the promotion work per SM is unchanged.
//
// Roles, per CTA (r = rank in the pair; the even CTA is the leader):
//   warp 0 (1 lane)          TMA producer: stage = two K chunks = 2 x (16 KB tokens + 8 KB weight half), four stages.
//                            Both producers' loads complete on the LEADER's full[] barrier (ordinary, non-multicast
//                            loads; only the completion signal crosses to the peer), each waits on its own empty[].
//   warps 1,2 (1 lane each)  leader only: MMA issuers; the issuer of unit g (= chunks 2g, 2g+1) is g % 2 and owns
//                            TMEM slots 2*(g%2), 2*(g%2)+1 (in both CTAs).  Per chunk: wait tempty[slot] (16 arrivals:
//                            the promotion warps of both CTAs), 4 x tcgen05.mma.cta_group::2 kind::f8f6f4 (M256 N128
//                            K32), commit -> tfull[slot] of both CTAs; per unit: commit -> empty[stage] of both CTAs.
//   warps 4..11              promotion of this CTA's 128 x 128 half: TMEM is four slots of one chunk product each,
//                            handed over chunk by chunk.  A thread owns one accumulator row and 64 columns and keeps
//                            two 64-register read-back buffers: while the tcgen05.ld of chunk i is in flight the FMAs
//                            of chunk i-1 issue from the other buffer, and the slot goes back to the leader's issuer
//                            as soon as the load has landed.  Result tile: bf16 through shared memory and a TMA store.
//
// A K range with an odd number of chunks ends in a unit whose second chunk has no MMAs; issuers and promotion
// warps still exchange that slot's barriers so that the phase of every barrier is a function of the unit
// counter alone.
//
// Every mbarrier wait is bounded: after about a second the waiting thread records what it was waiting for in
// the status word, raises a CTA-wide abort flag and all roles fall through to the common teardown.  Before a
// CTA leaves, its producer waits for the last commits onto its empty[] barriers (nothing else would), and the
// pair meets at a cluster barrier, so that no signal is in flight towards a CTA that has gone.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "gemm_plan.cuh"
#include "tc_wait.cuh"

namespace dsv3 {

namespace {

constexpr int kNumThreads = 384;          // warp 0: TMA producer, warps 1-2: MMA issuers (leader), 3 idle, 4..11: promotion
constexpr int kFirstPromoWarp = 4;
constexpr int kPromoThreads = 256;
constexpr int kRegsControl = 40;
constexpr int kRegsPromo = 232;
static_assert(128 * kRegsControl + 256 * kRegsPromo <= 384 * 168, "register pool");

constexpr int kBN = 128;                              // tile width (one b_s value per tile and chunk)
constexpr int kBHalf = kBN / 2;                       // weight rows each CTA of the pair loads
constexpr int kChunkBytes = (kPRows + kBHalf) * kChunk;   // per CTA: token tile + half weight tile of one chunk
constexpr int kUC = 2;                                // chunks per shared-memory stage ("unit")
constexpr int kStageBytes = kUC * kChunkBytes;
constexpr int kStages = 4;
constexpr int kSlots = 4;                             // TMEM slots of one chunk product each
constexpr int kTmemCols = kSlots * kBN;
constexpr int kStoreBytes = kPRows * 128 * 2;         // bf16 result tile, two 128-byte-swizzled 128 x 64 boxes
constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 1024;
static_assert(kSmemBytes <= 232448, "shared memory per CTA");
static_assert(kSmemBytes > 116 * 1024, "one CTA per SM (it allocates all of TMEM)");
static_assert(kTmemCols == 512, "all of TMEM");
static_assert((kPRows * kChunk) % 1024 == 0 && kChunkBytes % 1024 == 0, "operand tiles keep the swizzle atom's alignment");
// An issuer probes the tempty barriers of its next unit.  That is exact only because the slots of a unit
// depend on the unit's parity alone, i.e. a slot always belongs to the same issuer, which itself waited for
// the slot's previous phase.
static_assert(kSlots == 2 * kUC, "two issuers, each owning kUC slots");

struct TmParams {
    const float* a_s;
    const float* b_s;
    __nv_bfloat16* c;
    unsigned int* status;
    int64_t M, N;
    int kc;                 // K chunks
    int tiles_pp, tiles_q;  // pairs of token tiles, weight tiles
    int raster;             // token-tile pairs that share consecutive weight tiles in the work order
    FastDiv div_per_group, div_raster;
    int tma_store;          // results leave through shared memory and a TMA store (needs N % 8 == 0)
    int num_tiles;          // tiles_pp * tiles_q
};

struct Tile {
    int pp, q;
};

// Work order: `raster` token-tile pairs share consecutive weight tiles so that a wave re-uses both operands in L2.
__device__ __forceinline__ Tile decode_tile(int tile, const TmParams& p) {
    const int per_group = p.raster * p.tiles_q;
    const int grp = static_cast<int>(fast_div(static_cast<uint32_t>(tile), p.div_per_group));
    const int first = grp * p.raster;
    const int gsz = min(p.raster, p.tiles_pp - first);
    const int r = tile - grp * per_group;
    Tile t;
    t.q = (gsz == p.raster) ? static_cast<int>(fast_div(static_cast<uint32_t>(r), p.div_raster)) : r / gsz;   // the last group may be shorter
    t.pp = first + (r - t.q * gsz);
    return t;
}

__global__ void __launch_bounds__(kNumThreads, 1)
fp8_gemm_tm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_c, const TmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;     // the same offset in both CTAs of the pair
    uint8_t* gen_tiles = smem_raw + (tiles - raw);
    uint8_t* store_buf = gen_tiles + kStages * kStageBytes;                       // 1024-byte aligned (swizzle atom)
    uint64_t* bars = reinterpret_cast<uint64_t*>(store_buf + kStoreBytes);
    Control* ctl = reinterpret_cast<Control*>(bars + 2 * kStages + 2 * kSlots);
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };                        // used in the leader only
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto tfull_bar = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
    auto tempty_bar = [&](int s) { return bar0 + 8u * (2 * kStages + kSlots + s); };   // used in the leader only

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);   // uniform, and known to be
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0: leader (issues the MMAs), 1: peer
    const int pair = static_cast<int>(blockIdx.x >> 1);
    const int n_pairs = static_cast<int>(gridDim.x >> 1);
    const int kc = p.kc;
    const int n_units = (kc + kUC - 1) / kUC;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < kSlots; ++s) {
            mbar_init(tfull_bar(s), 1);
            mbar_init(tempty_bar(s), 2 * kPromoThreads / 32);   // every promotion warp of both CTAs reads its half of every slot
        }
        ctl->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        if (p.tma_store) tma_prefetch_desc(&tmap_c);
    }
    if (warp == 1) tc_alloc_pair(smem_u32(&ctl->tmem_base), kTmemCols);
    // Programmatic dependent launch: nothing above touches global memory, so it may overlap the tail of
    // the kernel before this one in the stream.  While waiting for that kernel, the producer thread pulls
    // the first weight boxes of this CTA's first tile into L2 (L2 is the point of coherence: should the
    // predecessor still be writing those weights, the later TMA loads see its data all the same).
    if (threadIdx.x == 0 && pair < p.num_tiles) {
        const Tile t = decode_tile(pair, p);
        const int n_pre = min(kc, kStages * kUC);
        for (int j = 0; j < n_pre; ++j) tma_prefetch_l2_2d(&tmap_b, j * kChunk, t.q * kBN + static_cast<int>(rank) * kBHalf);
    }
    griddep_launch_dependents();
    // the peer's barriers must be initialised before anything is signalled across the pair
    tc_fence_before();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    tc_fence_after();
    griddep_wait();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp < kFirstPromoWarp) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsControl));
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsPromo));
    }

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        // The whole warp walks the loop (waits included) and one elected lane issues: control flow, addresses and
        // descriptors then stay warp-uniform, which is what makes TMA and tcgen05 instructions cheap to issue.
        {
            uint32_t g = 0;
            uint32_t probe = 0;   // result of test_wait on empty[] for unit g, issued one unit earlier
            bool ok = true;
            for (int tile = pair; ok && tile < p.num_tiles; tile += n_pairs) {
                const Tile t = decode_tile(tile, p);
                const int a_row = (2 * t.pp + static_cast<int>(rank)) * kPRows;
                const int b_row = t.q * kBN + static_cast<int>(rank) * kBHalf;
                for (int u = 0; u < n_units; ++u, ++g) {
                    const int s = g % kStages;
                    ok = __all_sync(0xffffffffu, wait_probed(probe, empty_bar(s), ((g / kStages) & 1u) ^ 1u, ctl, p.status, 1, g));
                    if (!ok) break;
                    probe = mbar_test_wait(empty_bar((g + 1) % kStages), (((g + 1) / kStages) & 1u) ^ 1u) ? 1u : 0u;
                    const int k0 = u * kUC;
                    const int nch = min(kUC, kc - k0);
                    const uint32_t lead_full = mapa_shared(full_bar(s), 0);
                    // the leader's barrier expects the bytes of both CTAs; the peer's loads may complete on it
                    // before this arrive has been made (the phase cannot complete without it)
                    if (elect_one()) {
                        if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * nch * kChunkBytes);
                        for (int j = 0; j < nch; ++j) {
                            const uint32_t dst = tiles + s * kStageBytes + j * kChunkBytes;
                            tma_load_2d_pair(dst, &tmap_a, (k0 + j) * kChunk, a_row, lead_full);
                            tma_load_2d_pair(dst + kPRows * kChunk, &tmap_b, (k0 + j) * kChunk, b_row, lead_full);
                        }
                    }
                    __syncwarp();
                }
            }
            // Nothing waits for the commits onto the empty[] barriers of the last units; wait for them here so
            // that none is in flight when the CTA leaves (it would land in whatever CTA gets this shared memory next).
            for (uint32_t d = (g > kStages ? g - kStages : 0u); ok && d < g; ++d)
                ok = __all_sync(0xffffffffu, bounded_wait(empty_bar(d % kStages), (d / kStages) & 1u, ctl, p.status, 1, d));
        }
    } else if (warp <= 2) {
        // ------------------------------------------------------------ MMA issuers (leader CTA; unit g -> issuer g % 2)
        // (converged warp, elected lane: see the producer)
        if (rank == 0) {
            constexpr uint32_t idesc = umma_idesc_e4m3_f32(2 * kPRows, kBN);
            const uint32_t me = static_cast<uint32_t>(warp - 1);
            const int slot0 = static_cast<int>(me) * kUC;
            uint32_t probe_t[kUC] = {0u, 0u};   // probes of this issuer's tempty[] barriers for its next unit
            bool ok = true;
            uint32_t g = 0;
            for (int tile = pair; ok && tile < p.num_tiles; tile += n_pairs) {
                for (int u = 0; ok && u < n_units; ++u, ++g) {
                    if ((g & 1u) != me) continue;
                    const int s = g % kStages;
                    const uint32_t par = (g >> 1) & 1u;            // this issuer's use count of its slots, mod 2
                    const int nch = min(kUC, kc - u * kUC);
                    ok = __all_sync(0xffffffffu, bounded_wait(full_bar(s), (g / kStages) & 1u, ctl, p.status, 2, g));
                    if (!ok) break;
#pragma unroll
                    for (int j = 0; j < kUC; ++j) {
                        ok = __all_sync(0xffffffffu, wait_probed(probe_t[j], tempty_bar(slot0 + j), par ^ 1u, ctl, p.status, 3, g));
                        if (!ok) break;
                        tc_fence_after();
                        if (elect_one()) {
                            if (j < nch) {
                                const uint32_t sp = tiles + s * kStageBytes + j * kChunkBytes;
                                const uint64_t da = umma_desc_k_major_sw128(sp);
                                const uint64_t db = umma_desc_k_major_sw128(sp + kPRows * kChunk);
                                const uint32_t d_tmem = tmem_base + (slot0 + j) * kBN;
#pragma unroll
                                for (int k = 0; k < kChunk / 32; ++k) {
                                    // 32 bytes further along K inside the 128-byte swizzle atom: +2 in address units of 16 B
                                    tc_mma_f8_pair(d_tmem, da + 2u * k, db + 2u * k, idesc, k > 0 ? 1u : 0u);
                                }
                            }
                            // this chunk's product is complete in the TMEM of both CTAs
                            tc_commit_pair(tfull_bar(slot0 + j));
                            tc_commit_pair(mapa_shared(tfull_bar(slot0 + j), 1));
                        }
                        __syncwarp();
                    }
                    if (!ok) break;
                    // the stage is reusable in both CTAs once these MMAs have read it
                    if (elect_one()) {
                        tc_commit_pair(empty_bar(s));
                        tc_commit_pair(mapa_shared(empty_bar(s), 1));
                    }
                    __syncwarp();
                    const uint32_t parn = (((g + 2) >> 1) & 1u) ^ 1u;
#pragma unroll
                    for (int j = 0; j < kUC; ++j) probe_t[j] = mbar_test_wait(tempty_bar(slot0 + j), parn) ? 1u : 0u;
                }
            }
        }
    } else if (warp >= kFirstPromoWarp) {
        // ------------------------------------------------------------ promotion + epilogue (both CTAs)
        // Warps 4..7 own the left 64 columns of the CTA's 128 x 128 half, warps 8..11 the right 64; within a column
        // half a thread owns one accumulator row (TMEM lane).
        const int half = (warp - kFirstPromoWarp) >> 2;
        const int col0 = half * 64;
        const int quarter = warp & 3;                       // TMEM lane quarter this warp may access
        const int row = quarter * 32 + lane;                // accumulator row (TMEM lane)
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + col0;
        const uint32_t lead_tempty0 = mapa_shared(tempty_bar(0), 0);   // the leader's tempty[0], as seen from this CTA

        uint32_t va[64], vb[64];
        float2 acc[32];
        auto fold = [&](const uint32_t* v, float sc) {
            const float2 sc2 = make_float2(sc, sc);
#pragma unroll
            for (int j = 0; j < 32; ++j)
                acc[j] = __ffma2_rn(make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1])), sc2, acc[j]);
        };
        auto release = [&](int slot) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8u * slot);
        };
        // Result tile: the four warps of a column half stage their 128 x 64 bf16 box in shared memory (128-byte
        // swizzle: 16-byte slot c of row r sits at slot c ^ (r & 7), which also keeps the vector stores free of
        // bank conflicts) and one thread hands it to the TMA, which clips rows beyond M and columns beyond N.
        // The store of the previous tile is only known to have read the buffer once its issuer has waited for
        // it, hence the first barrier.  tp = token tile of this CTA.
        auto write_tile = [&](int tp, int tq) {
            if (static_cast<int64_t>(tp) * kPRows >= p.M) return;     // the odd half of the last pair: nothing to store
            const float* accf = reinterpret_cast<const float*>(acc);
            if (p.tma_store) {
                uint8_t* sbuf = store_buf + half * (kPRows * 128);
                const bool issuer = ((threadIdx.x & 127) == 0);
                if (issuer) bulk_wait_group_read0();
                asm volatile("bar.sync %0, 128;" ::"r"(2 + half) : "memory");
#pragma unroll
                for (int cidx = 0; cidx < 8; ++cidx) {
                    const int j = cidx * 8;
                    const uint4 o = make_uint4(pack_bf16x2(accf[j], accf[j + 1]), pack_bf16x2(accf[j + 2], accf[j + 3]),
                                               pack_bf16x2(accf[j + 4], accf[j + 5]), pack_bf16x2(accf[j + 6], accf[j + 7]));
                    *reinterpret_cast<uint4*>(sbuf + row * 128 + ((cidx ^ (row & 7)) << 4)) = o;
                }
                fence_proxy_async_shared();
                asm volatile("bar.sync %0, 128;" ::"r"(2 + half) : "memory");
                if (issuer) {
                    tma_store_2d(&tmap_c, smem_u32(sbuf), tq * kBN + half * 64, tp * kPRows);
                    bulk_commit_group();
                }
            } else {
                const int64_t m = static_cast<int64_t>(tp) * kPRows + row;
                const int64_t N = p.N;
                if (m < p.M) {
                    __nv_bfloat16* crow = p.c + m * N;
                    const int64_t n0 = static_cast<int64_t>(tq) * kBN + col0;
#pragma unroll
                    for (int j = 0; j < 64; ++j)
                        if (n0 + j < N) crow[n0 + j] = __float2bfloat16_rn(accf[j]);
                }
            }
        };

        bool ok = true;
        uint32_t g = 0;            // unit counter
        uint32_t probe = 0;        // result of test_wait on the tfull[] barrier that is waited for next
        bool pend = false;         // vb holds a chunk product that is not folded into acc yet
        float pend_sc = 0.0f;
        bool epi = false;          // acc (after the pending fold) is the finished previous tile, not written yet

        int tile = pair;
        if (tile < p.num_tiles) {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = make_float2(0.0f, 0.0f);
            while (true) {
                // scale rows of this tile for this thread: a_s of its token (clamped at the edge), b_s of the
                // weight tile.  The first unit's products are requested here and first used after the unit's
                // first read-back (and after the previous tile has been written), so their latency is covered.
                const Tile cur = decode_tile(tile, p);
                const int64_t tok = static_cast<int64_t>(2 * cur.pp + static_cast<int>(rank)) * kPRows + row;
                const float* as_ptr = p.a_s + min(tok, p.M - 1) * kc;
                const float* bs_ptr = p.b_s + static_cast<int64_t>(cur.q) * kc;
                float sa0 = __ldg(as_ptr) * __ldg(bs_ptr);
                float sa1 = kc > 1 ? __ldg(as_ptr + 1) * __ldg(bs_ptr + 1) : 0.0f;
                for (int u = 0; u < n_units; ++u, ++g) {
                    const int slot = static_cast<int>(g & 1u) * kUC;
                    const uint32_t par = (g >> 1) & 1u;
                    if (epi) {      // the previous tile is complete: fold its last chunk, write it, start the new one
                        if (pend) fold(vb, pend_sc);
                        pend = false;
                        const Tile prev = decode_tile(tile - n_pairs, p);
                        write_tile(2 * prev.pp + static_cast<int>(rank), prev.q);
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[j] = make_float2(0.0f, 0.0f);
                        epi = false;
                    }
                    // ---- first chunk of the unit -> va, while the previous chunk (vb) is folded
                    bool mine = wait_probed(probe, tfull_bar(slot), par, ctl, p.status, 4, g);
                    if (!__all_sync(0xffffffffu, mine)) { ok = false; break; }
                    tc_fence_after();
                    tc_ld_x64(t_lane + slot * kBN, va);
                    // row scales of the tile's next unit, one unit ahead (clamped: the last unit re-reads its own)
                    const int kn = min((u + 1) * kUC, kc - 1);
                    const int kn1 = min(kn + 1, kc - 1);
                    const float sb0 = __ldg(as_ptr + kn) * __ldg(bs_ptr + kn);
                    const float sb1 = __ldg(as_ptr + kn1) * __ldg(bs_ptr + kn1);
                    if (pend) fold(vb, pend_sc);
                    tc_wait_ld();
                    release(slot);
                    probe = mbar_test_wait(tfull_bar(slot + 1), par) ? 1u : 0u;
                    // ---- second chunk of the unit -> vb, while the first (va) is folded.  A K range with an odd
                    // number of chunks ends in a unit without a second product: the slot is read all the same
                    // (whatever it holds is never used) so that the loop body stays free of divergent register state.
                    mine = wait_probed(probe, tfull_bar(slot + 1), par, ctl, p.status, 4, g);
                    if (!__all_sync(0xffffffffu, mine)) { ok = false; break; }
                    tc_fence_after();
                    tc_ld_x64(t_lane + (slot + 1) * kBN, vb);
                    fold(va, sa0);
                    tc_wait_ld();
                    release(slot + 1);
                    {
                        const uint32_t gn = g + 1;
                        probe = mbar_test_wait(tfull_bar(static_cast<int>(gn & 1u) * kUC), (gn >> 1) & 1u) ? 1u : 0u;
                    }
                    pend = (u * kUC + 1 < kc);
                    pend_sc = sa1;
                    sa0 = sb0;
                    sa1 = sb1;
                }
                if (!ok) break;
                epi = true;
                if (tile + n_pairs >= p.num_tiles) break;
                tile += n_pairs;
            }
            if (ok) {     // `tile` is the last tile of this pair
                if (pend) fold(vb, pend_sc);
                if (epi) {
                    const Tile last = decode_tile(tile, p);
                    write_tile(2 * last.pp + static_cast<int>(rank), last.q);
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    if (warp >= kFirstPromoWarp && (threadIdx.x & 127) == 0) bulk_wait_group0();   // result tiles have left shared memory
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (ctl->abort_flag) {
        // give copies and MMAs that were already issued time to land before the CTA's
        // shared memory and TMEM are released
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    // neither CTA of the pair may go while the other can still signal its barriers or read its operands
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after();
        tc_dealloc_pair(tmem_base, kTmemCols);
    }
}

}  // namespace

bool tm_pair_supported(int64_t M, int64_t N, int64_t K, bool forced) {
    (void)N;
    // At least two token tiles (otherwise the second CTA of a pair would multiply zeros) and, when the choice is
    // the library's, at least 12 K chunks: with short K the per-tile work of the promotion warps (first scale
    // fetch, result tile) weighs more than the operand stream, and the single-CTA kernel with two-chunk hand-offs
    // is faster (measured on B200, M = 4096: K = 512: 135 vs 111 us at N = 32768; K = 1536: 202 vs 205 us at
    // N = 24576; K = 7168: 566 vs 617 us at N = 18432).
    if (M <= kPRows) return false;
    return forced || K >= 12 * kChunk;
}

int launch_fp8_gemm_tm(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N,
                       int64_t K, void* c, cudaStream_t stream) {
    const int64_t tiles_p = (M + kPRows - 1) / kPRows, tiles_q = (N + kBN - 1) / kBN;
    const int64_t tiles_pp = (tiles_p + 1) / 2;
    if (tiles_pp * tiles_q >= (1ll << 31)) {
        set_last_error("fp8_gemm: %lld x %lld output tiles are more than the work-item counter holds",
                       static_cast<long long>(tiles_p), static_cast<long long>(tiles_q));
        return DSV3_ERR_UNSUPPORTED;
    }
    CUtensorMap ta, tb, tc;
    memset(&tc, 0, sizeof(tc));
    int rc;
    if ((rc = make_tmap(&ta, a, M, K, kPRows)) != DSV3_OK) return rc;
    if ((rc = make_tmap(&tb, b, N, K, kBHalf)) != DSV3_OK) return rc;
    const bool tma_store = (N % 8) == 0;   // row pitch of the result must be a multiple of 16 bytes for a tensor map
    if (tma_store && (rc = make_tmap_out(&tc, c, M, N)) != DSV3_OK) return rc;
    TmParams prm;
    prm.a_s = a_s;
    prm.b_s = b_s;
    prm.c = static_cast<__nv_bfloat16*>(c);
    prm.status = status_device_ptr();
    if (!prm.status) return DSV3_ERR_CUDA;
    prm.M = M;
    prm.N = N;
    prm.kc = static_cast<int>((K + kChunk - 1) / kChunk);
    prm.tiles_pp = static_cast<int>(tiles_pp);
    prm.tiles_q = static_cast<int>(tiles_q);
    // Work order: as many token-tile pairs as keep their activations (raster x 256 x K bytes) within about a
    // quarter of L2 share consecutive weight tiles, so that the weights stream from HBM as few times as possible.
    const int64_t fit = (32ll << 20) / (static_cast<int64_t>(2 * kPRows) * K);
    prm.raster = static_cast<int>(fit < 4 ? 4 : (fit > 32 ? 32 : fit));
    prm.div_raster = make_fast_div(static_cast<uint32_t>(prm.raster));
    prm.div_per_group = make_fast_div(static_cast<uint32_t>(prm.raster) * static_cast<uint32_t>(prm.tiles_q));
    prm.tma_store = tma_store ? 1 : 0;
    prm.num_tiles = static_cast<int>(tiles_pp * tiles_q);

    auto kern = fp8_gemm_tm_kernel;
    static bool configured[64] = {};
    int dev = 0;
    DSV3_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_last_error("fp8_gemm: device ordinal %d is outside the supported range", dev);
        return DSV3_ERR_UNSUPPORTED;
    }
    if (!configured[dev]) {
        DSV3_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        configured[dev] = true;
    }
    const int max_pairs = num_sms() / 2;
    const int pairs = prm.num_tiles < max_pairs ? prm.num_tiles : max_pairs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kNumThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    DSV3_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, prm));
    return DSV3_OK;
}

}  // namespace dsv3
