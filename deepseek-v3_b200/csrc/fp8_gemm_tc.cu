// fp8_gemm for sm_100a: TMA-fed, warp-specialised, persistent tcgen05 kernel with
// software promotion of every 128-wide K chunk.
//
// Replaces inference/kernel.py:118-172 (fp8_gemm_kernel) and its launch at :194-195.
//
// Why promotion is done in software: the scales are fp32 (a_s per token per chunk,
// b_s per 128x128 weight block), not ue8m0, so the block-scaled MMA kinds cannot apply
// them.  Each chunk is therefore multiplied into its own TMEM accumulator
// (4 x tcgen05.mma kind::f8f6f4, K = 32 each), read back with tcgen05.ld by the
// promotion warps, and folded into fp32 registers as acc += dot * (a_s * b_s).
//
// The pipeline moves "units" of UC consecutive K chunks, numbered g = 0,1,2,... across all work
// items of a CTA (UC = 2 for token-major tiles, 1 for weight-major tiles):
//   warp 0 (1 lane)          TMA producer: waits empty[g % NS], loads the P and Q tiles of the unit's chunks
//   warps 1,2 (1 lane each)  MMA issuers, unit g belongs to issuer g % 2: wait tempty[g % NT] and full[g % NS],
//                            issue 4 MMAs per chunk, commit to empty[g % NS] and tfull[g % NT]
//   warps 4..11              promotion: wait tfull[g % NT], read the unit back from TMEM (token-major: both
//                            chunks behind a single tcgen05.wait::ld), release tempty, then do the FMAs; at
//                            the end of a work item write the result (token-major: through shared memory and
//                            a TMA store) or park a split-K partial tile
// Operand roles: P is the 128-row MMA "A" operand, Q the BN-row MMA "B" operand.
//   kSwap = false : P = 128 tokens of a,  Q = 128 rows of b  (M > 64: "token-major" tiles)
//   kSwap = true  : P = 128 rows of b,    Q = BN tokens of a (M <= 64: "weight-major", weights stream once)
// Split-K: a work item is (tile, split); partial tiles go to a workspace and the CTA that
// takes the last ticket of a tile adds them in split order (deterministic, no spinning).
//
// Hand-off costs set the structure: a dependent mbarrier.try_wait takes ~175 cycles even when the
// phase is already complete and tcgen05.fence::after_thread_sync is of the same order, while a chunk
// is only ~256 cycles of tensor-core work.  So a token-major unit is two chunks, the issue work is split
// over two threads, and every role probes the barrier of its next unit (a non-blocking test_wait whose
// result is consumed one iteration later) where that is safe.
//
// Every wait is bounded: after about a second the waiting thread records what it was
// waiting for in the status word, raises a CTA-wide abort flag and all roles fall
// through to the common teardown (which frees TMEM).
#include <cuda.h>

#include <cstring>
#include <mutex>
#include <type_traits>
#include <vector>

#include "common.cuh"
#include "gemm_plan.cuh"
#include "tc_wait.cuh"

namespace dsv3 {

namespace {

constexpr int kNumThreads = 384;          // warp 0: TMA producer, warps 1-2: MMA issuers, 3 idle, 4..11: promotion
constexpr int kIssuers = 2;
constexpr int kPromoThreads = 256;
constexpr int kFirstPromoWarp = 4;
// Register budget: 384 threads start with 168 each; the control warpgroup gives registers back and
// the two promotion warpgroups take them (64 accumulators + two 64-value read-back buffers).
constexpr int kRegsControl = 40;
constexpr int kRegsPromo = 232;
static_assert(128 * kRegsControl + 256 * kRegsPromo <= 384 * 168, "register pool");

constexpr int kTmemStages = 4;
constexpr int kMaxTickets = DSV3_WORKSPACE_HEADER_BYTES / 4;

struct TcParams {
    const float* a_s;
    const float* b_s;
    __nv_bfloat16* c;
    float* partials;        // [splits][tiles][bn / 4][128] float4 (padded partial tiles), only when splits > 1
    int* tickets;           // one per tile, zero on entry and on exit
    unsigned int* status;   // device status words
    int64_t M, N;
    int kc;                 // number of K chunks
    int tiles_p, tiles_q;
    int splits;
    FastDiv div_splits, div_per_group, div_raster, div_tiles_p;   // for the work-item decoder
    int raster;             // token-major tiles: P tiles (token tiles) that share consecutive Q tiles in the work order
    int tma_store;          // token-major tiles: results leave through shared memory and a TMA store (needs N % 8 == 0)
    int num_items;          // tiles_p * tiles_q * splits
    // Grouped mode (MoE experts; weight-major tiles only, no split-K): group e multiplies the activation
    // rows [g_seg[e], g_seg[e+1]) with its own weight.  n_groups == 0 means one ordinary GEMM.
    const CUtensorMap* g_tmaps;    // per-group weight tensor maps, in global memory
    const float* const* g_bs;      // per-group weight scale pointers, in global memory
    const int* g_seg;              // [n_groups + 1] row offsets, in global memory (written on the device)
    int n_groups;
    int g_slots;                   // upper bound on the number of token tiles over all groups
};

// K chunks of one weight-major work item whose scales fit the shared-memory table: 144 (K <= 18432) for
// 16- and 32-token tiles, 72 for 64-token tiles (the same 18 KB, which leaves room for four 48 KB stages;
// longer K is split, or uses the 32-token variant in grouped mode)
constexpr int scale_tab_chunks(int bn) { return bn >= 64 ? 72 : 144; }

template <int BN, bool kSwap>
struct Cfg {
    // The pipeline moves "units" of kUC consecutive K chunks: one smem stage, one TMEM stage and one
    // round of hand-offs per unit.  Token-major tiles pair two chunks so that every hand-off (each costs
    // several hundred cycles of latency) covers twice the tensor-core work.
    static constexpr int kUC = (kSwap && BN < 64) ? 1 : 2;
    static constexpr int kChunkBytes = kPRows * kChunk + BN * kChunk;      // P and Q tile of one chunk
    static constexpr int kStageBytes = kUC * kChunkBytes;
    // chunk products resident in TMEM: four 128-column accumulators, or eight of 64 columns
    static constexpr int kAccs = (kSwap && BN == 64) ? 8 : kTmemStages;
    static constexpr int kTmemUnits = kAccs / kUC;                          // unit products resident in TMEM
    // weight-major tiles: a_s * b_s of the item's chunks for the tile's BN tokens, [chunk][token]
    static constexpr int kScaleTabBytes = kSwap ? scale_tab_chunks(BN) * BN * 4 : 0;
    static constexpr int kGroupTabBytes = kSwap ? 2048 : 0;   // grouped mode: token-tile prefix per group
    // token-major tiles: the 128 x 128 bf16 result tile is staged here (two 128-byte-swizzled 128 x 64 boxes)
    static constexpr int kStoreBytes = !kSwap ? kPRows * 128 * 2 : 0;
    static constexpr int kStagesRaw =
        (232448 - 2048 - kStoreBytes - kScaleTabBytes - kGroupTabBytes) / kStageBytes;
    static constexpr int kStagesCap = kStagesRaw > 10 ? 10 : kStagesRaw;
    // weight-major tiles: an even stage count, so that a stage always belongs to the same MMA issuer and
    // the issuer may probe its next full[] barrier (see the issuer loop)
    static constexpr int kStages = kSwap ? (kStagesCap & ~1) : kStagesCap;
    static constexpr int kTmemCols = kAccs * BN;  // 64..512, a power of two
    // tiles + result staging + tables + barriers + control words + slack for the 1024-byte alignment of the tiles
    static constexpr int kSmemBytes =
        kStages * kStageBytes + kStoreBytes + kScaleTabBytes + kGroupTabBytes + 1024 + 1024;
    static_assert(kSmemBytes <= 232448, "shared memory per CTA");
    static_assert(kStages >= 3, "at least three smem stages");
    static_assert(kTmemCols >= 32 && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns");
    static_assert((BN * kChunk) % 1024 == 0, "Q tile must keep 1024-byte alignment");
    // more than half of an SM's shared memory, so two CTAs can never share an SM (and its TMEM)
    static_assert(kSmemBytes > 116 * 1024, "one CTA per SM");
};

struct Item {
    int p_idx, q_idx, split, tile;
    int c0, c1;     // chunk range
    int group;      // grouped mode: which weight
    int row0;       // weight-major tiles: first activation row of the tile
    int row_end;    // weight-major tiles: activation rows at and beyond this index are not part of the problem
};

constexpr int kMaxGroups = 256;

// g_prefix (shared memory, grouped mode): g_prefix[e] = number of token tiles of the groups before e.
template <int BN, bool kSwap>
__device__ __forceinline__ Item decode_item(int item, const TcParams& p, const int* g_prefix) {
    Item it;
    if (kSwap && p.n_groups > 0) {
        // item -> (weight tile p_idx, token-tile slot); slot -> (group, tile within the group) by binary search
        const int slot = static_cast<int>(fast_div(static_cast<uint32_t>(item), p.div_tiles_p));
        it.p_idx = item - slot * p.tiles_p;
        it.tile = item;
        it.split = 0;
        it.q_idx = 0;
        int lo = 0, hi = p.n_groups;          // invariant: g_prefix[lo] <= slot, answer in [lo, hi)
        if (slot >= g_prefix[p.n_groups]) {   // beyond the last real tile: an empty item
            it.group = 0;
            it.row0 = it.row_end = 0;
            it.c0 = it.c1 = 0;
            return it;
        }
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (g_prefix[mid] <= slot) lo = mid; else hi = mid;
        }
        it.group = lo;
        it.row0 = __ldg(p.g_seg + lo) + (slot - g_prefix[lo]) * BN;
        it.row_end = __ldg(p.g_seg + lo + 1);
        it.c0 = 0;
        it.c1 = p.kc;
        return it;
    }
    it.group = 0;
    it.tile = static_cast<int>(fast_div(static_cast<uint32_t>(item), p.div_splits));
    it.split = item - it.tile * p.splits;
    // work order: `raster` P tiles share consecutive Q tiles so that a wave re-uses both operands in L2
    const int kGroup = p.raster;
    const int per_group = kGroup * p.tiles_q;
    const int grp = static_cast<int>(fast_div(static_cast<uint32_t>(it.tile), p.div_per_group));
    const int first_p = grp * kGroup;
    const int gsz = min(kGroup, p.tiles_p - first_p);
    const int r = it.tile - grp * per_group;
    it.q_idx = (gsz == kGroup) ? static_cast<int>(fast_div(static_cast<uint32_t>(r), p.div_raster)) : r / gsz;   // the last group may be shorter
    it.p_idx = first_p + (r - it.q_idx * gsz);
    // kc * split < 2^31 (kc < 2^24, at most 64 splits)
    it.c0 = static_cast<int>(fast_div(static_cast<uint32_t>(p.kc * it.split), p.div_splits));
    it.c1 = static_cast<int>(fast_div(static_cast<uint32_t>(p.kc * (it.split + 1)), p.div_splits));
    it.row0 = it.q_idx * BN;
    it.row_end = static_cast<int>(p.M);
    return it;
}

template <int N>
__device__ __forceinline__ void tmem_load_cols(uint32_t taddr, uint32_t* v) {
    if constexpr (N == 8) {
        tc_ld_x8(taddr, v);
    } else if constexpr (N == 16) {
        tc_ld_x16(taddr, v);
    } else if constexpr (N == 32) {
        tc_ld_x32(taddr, v);
    } else {
        static_assert(N == 64, "columns per thread");
        tc_ld_x32(taddr, v);
        tc_ld_x32(taddr + 32, v + 32);
    }
}

// Barrier among the threads that write results (promotion group 0, or all promotion warps when
// there is a single group).
template <int kThreads>
__device__ __forceinline__ void promo_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory"); }

template <int BN, bool kSwap>
__global__ void __launch_bounds__(kNumThreads, 1)
fp8_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_p, const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ CUtensorMap tmap_c, const TcParams p) {
    using C = Cfg<BN, kSwap>;
    constexpr int NS = C::kStages;
    constexpr int UC = C::kUC;           // K chunks per pipeline unit
    constexpr int NT = C::kTmemUnits;    // TMEM stages, in units
    constexpr int CPT = BN / 2;       // accumulator columns per promotion thread (a thread owns half a row)
    constexpr int kWriters = kPromoThreads;
    static_assert(kSwap || BN == 128, "token-major tiles are 128 x 128 (one b_s value per tile and chunk)");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    uint8_t* gen_tiles = smem_raw + (tiles - raw);
    uint8_t* store_buf = gen_tiles + NS * C::kStageBytes;                       // 1024-byte aligned (swizzle atom)
    uint8_t* after_store = store_buf + C::kStoreBytes;
    float* sc_tab = reinterpret_cast<float*>(after_store);   // [chunk][token]
    int* g_prefix = reinterpret_cast<int*>(after_store + C::kScaleTabBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(after_store + C::kScaleTabBytes + C::kGroupTabBytes);
    Control* ctl = reinterpret_cast<Control*>(bars + 2 * NS + 2 * NT + 2);
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (NS + s); };
    auto tfull_bar = [&](int s) { return bar0 + 8u * (2 * NS + s); };
    auto tempty_bar = [&](int s) { return bar0 + 8u * (2 * NS + NT + s); };
    const uint32_t tab_ready_bar = bar0 + 8u * (2 * NS + 2 * NT);       // scale table of the item is filled
    const uint32_t tab_free_bar = bar0 + 8u * (2 * NS + 2 * NT + 1);    // scale table may be overwritten

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);   // uniform, and known to be
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < NT; ++s) {
            mbar_init(tfull_bar(s), 1);
            mbar_init(tempty_bar(s), kPromoThreads / 32);   // every promotion warp reads every stage
        }
        mbar_init(tab_ready_bar, kPromoThreads);
        mbar_init(tab_free_bar, kPromoThreads);
        ctl->abort_flag = 0;
        ctl->ticket[0] = 0;
        ctl->ticket[1] = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_p);
        tma_prefetch_desc(&tmap_q);
        if (!kSwap && p.tma_store) tma_prefetch_desc(&tmap_c);
    }
    if (warp == 1) tc_alloc(smem_u32(&ctl->tmem_base), C::kTmemCols);
    // Programmatic dependent launch: nothing above touches global memory, so it may overlap the tail of
    // the kernel before this one in the stream.  While waiting for that kernel, the producer thread pulls
    // the first weight boxes of this CTA's first work item into L2 (L2 is the point of coherence: should
    // the predecessor still be writing those weights, the later TMA loads see its data all the same).
    if (threadIdx.x == 0 && p.n_groups == 0 && static_cast<int>(blockIdx.x) < p.num_items) {
        const Item it = decode_item<BN, kSwap>(blockIdx.x, p, g_prefix);
        const void* wmap = kSwap ? static_cast<const void*>(&tmap_p) : static_cast<const void*>(&tmap_q);
        const int wrow = kSwap ? it.p_idx * kPRows : it.q_idx * BN;
        const int n_pre = min(it.c1 - it.c0, NS * UC);
        for (int j = 0; j < n_pre; ++j) tma_prefetch_l2_2d(wmap, (it.c0 + j) * kChunk, wrow);
    }
    griddep_launch_dependents();
    griddep_wait();
    if constexpr (kSwap) {
        if (p.n_groups > 0) {
            // token tiles per group, then an exclusive prefix sum (n_groups <= kMaxGroups)
            for (int e = threadIdx.x; e < p.n_groups; e += kNumThreads) {
                const int cnt = __ldg(p.g_seg + e + 1) - __ldg(p.g_seg + e);
                g_prefix[e + 1] = (cnt + BN - 1) / BN;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                int run = 0;
                g_prefix[0] = 0;
                for (int e = 1; e <= p.n_groups; ++e) {
                    run += g_prefix[e];
                    g_prefix[e] = run;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if constexpr (!kSwap) {
        if (warp < kFirstPromoWarp) {
            asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsControl));
        } else {
            asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsPromo));
        }
    }

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // The whole warp walks the loop (waits included) and one elected lane issues: control flow, addresses and
        // descriptors then stay warp-uniform, which is what makes TMA and tcgen05 instructions cheap to issue.
        {
            uint32_t g = 0;
            uint32_t probe = 0;   // result of try_wait on empty[] for chunk g, issued one chunk earlier
            bool ok = true;
            for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
                const Item it = decode_item<BN, kSwap>(item, p, g_prefix);
                const int p_row = it.p_idx * kPRows;
                const int q_row = kSwap ? it.row0 : it.q_idx * BN;
                const void* map_p = (kSwap && p.n_groups > 0) ? static_cast<const void*>(p.g_tmaps + it.group)
                                                               : static_cast<const void*>(&tmap_p);
                const int n_units = (it.c1 - it.c0 + UC - 1) / UC;
                for (int u = 0; u < n_units; ++u, ++g) {
                    const int s = g % NS;
                    ok = __all_sync(0xffffffffu, wait_probed(probe, empty_bar(s), ((g / NS) & 1u) ^ 1u, ctl, p.status, 1, g));
                    if (!ok) break;
                    probe = mbar_test_wait(empty_bar((g + 1) % NS), (((g + 1) / NS) & 1u) ^ 1u) ? 1u : 0u;
                    const int k0 = it.c0 + u * UC;
                    const int nch = min(UC, it.c1 - k0);
                    if (elect_one()) {
                        mbar_arrive_expect_tx(full_bar(s), nch * C::kChunkBytes);
                        for (int j = 0; j < nch; ++j) {
                            const uint32_t dst = tiles + s * C::kStageBytes + j * C::kChunkBytes;
                            tma_load_2d(dst, map_p, (k0 + j) * kChunk, p_row, full_bar(s));
                            tma_load_2d(dst + kPRows * kChunk, &tmap_q, (k0 + j) * kChunk, q_row, full_bar(s));
                        }
                    }
                    __syncwarp();
                }
            }
            // Nothing waits for the commits onto the empty[] barriers of the last units; wait for them here so
            // that none is in flight when the CTA leaves (it would land in whatever CTA gets this shared memory next).
            for (uint32_t d = (g > static_cast<uint32_t>(NS) ? g - NS : 0u); ok && d < g; ++d)
                ok = __all_sync(0xffffffffu, bounded_wait(empty_bar(d % NS), (d / NS) & 1u, ctl, p.status, 1, d));
        }
    } else if (warp <= kIssuers) {
        // ------------------------------------------------------------ MMA issuers (chunk g -> issuer g % kIssuers)
        // (converged warp, elected lane: see the producer)
        {
            constexpr uint32_t idesc = umma_idesc_e4m3_f32(kPRows, BN);
            const uint32_t me = static_cast<uint32_t>(warp - 1);
            uint32_t g = 0;
            uint32_t probe_t = 0, probe_f = 0;   // probes of tempty[] / full[] for this issuer's next unit
            bool ok = true;
            for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
                const Item it = decode_item<BN, kSwap>(item, p, g_prefix);
                const int n_units = (it.c1 - it.c0 + UC - 1) / UC;
                for (int u = 0; u < n_units; ++u, ++g) {
                    if (g % kIssuers != me) continue;
                    const int s = g % NS, ts = g % NT;
                    constexpr bool kProbeFull = (NS % kIssuers) == 0;
                    ok = __all_sync(0xffffffffu, wait_probed(probe_t, tempty_bar(ts), ((g / NT) & 1u) ^ 1u, ctl, p.status, 3, g) &&
                                                 wait_probed(kProbeFull ? probe_f : 0u, full_bar(s), (g / NS) & 1u, ctl, p.status, 2, g));
                    if (!ok) break;
                    {   // Probe the TMEM stage of this issuer's next unit now; the answer is read one iteration
                        // later.  A parity probe is only meaningful if the barrier's previous phase is known to be
                        // complete: true for tempty (NT is even, so a stage always belongs to the same issuer, which
                        // waited for that phase itself); for full[] only when NS is even as well (otherwise the previous
                        // phase of that stage belongs to the other issuer and the barrier is always waited for).
                        static_assert(NT % kIssuers == 0, "a TMEM stage must always be used by the same issuer");
                        const uint32_t gn = g + kIssuers;
                        probe_t = mbar_test_wait(tempty_bar(gn % NT), ((gn / NT) & 1u) ^ 1u) ? 1u : 0u;
                        if constexpr (kProbeFull) probe_f = mbar_test_wait(full_bar(gn % NS), (gn / NS) & 1u) ? 1u : 0u;
                    }
                    tc_fence_after();
                    const int nch = min(UC, it.c1 - it.c0 - u * UC);
                    if (elect_one()) {
                        for (int j = 0; j < nch; ++j) {
                            const uint32_t sp = tiles + s * C::kStageBytes + j * C::kChunkBytes;
                            const uint64_t dp = umma_desc_k_major_sw128(sp);
                            const uint64_t dq = umma_desc_k_major_sw128(sp + kPRows * kChunk);
                            const uint32_t d_tmem = tmem_base + (ts * UC + j) * BN;   // one TMEM region per chunk
#pragma unroll
                            for (int k = 0; k < kChunk / 32; ++k) {
                                // 32 bytes further along K inside the 128-byte swizzle atom: +2 in address units of 16 B
                                tc_mma_f8(d_tmem, dp + 2u * k, dq + 2u * k, idesc, k > 0 ? 1u : 0u);
                            }
                        }
                        tc_commit(empty_bar(s));   // smem stage reusable once these MMAs have read it
                        tc_commit(tfull_bar(ts));  // the unit's chunk products are complete in TMEM
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp >= kFirstPromoWarp) {
        // ------------------------------------------------------------ promotion + epilogue
        // All eight warps work on every unit: warps 4..7 own the left half of the tile's columns, warps 8..11
        // the right half; within a half, a thread owns one accumulator row (TMEM lane) and CPT columns.
        const int col0 = ((warp - kFirstPromoWarp) >> 2) * CPT;
        const int quarter = warp & 3;                       // TMEM lane quarter this warp may access
        const int row = quarter * 32 + lane;                // accumulator row (TMEM lane)
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + col0;
        const int64_t M = p.M, N = p.N;
        const int kc = p.kc;
        uint32_t g = 0;          // unit counter at the start of the current item
        uint32_t item_no = 0;    // non-empty items done by this CTA (phase of the scale-table barriers, ticket slot)
        bool ok = true;

        // A chunk is read back in SPC steps of HC columns so that one step's TMEM load is in flight
        // while the previous step's FMAs issue.
        constexpr int HC = (CPT >= 32) ? 32 : CPT;
        constexpr int SPC = CPT / HC;
        uint32_t probe = 0;   // result of test_wait on tfull[] for the next unit
        // token-major tiles: two read-back buffers of one chunk (64 columns) each
        constexpr bool kBatched = !kSwap;
        uint32_t va64[kBatched ? 64 : 1], vb64[kBatched ? 64 : 1];
        // Issues (does not wait for) the load of step `st` of chunk `j` of unit `gu`; the first step of a
        // unit first waits for the unit's products to be complete in TMEM.
        auto issue_load = [&](uint32_t gu, int j, int st, uint32_t* v) -> bool {
            const int ts = gu % NT;
            if (j == 0 && st == 0) {
                const bool mine = wait_probed(probe, tfull_bar(ts), (gu / NT) & 1u, ctl, p.status, 4, gu);
                if (!__all_sync(0xffffffffu, mine)) return false;
                probe = mbar_test_wait(tfull_bar((gu + 1) % NT), ((gu + 1) / NT) & 1u) ? 1u : 0u;
                tc_fence_after();
            }
            tmem_load_cols<HC>(t_lane + (ts * UC + j) * BN + st * HC, v);
            return true;
        };
        // Completes the outstanding load; `last` = it was the last load of the unit, whose TMEM stage
        // then goes back to the MMA issuers.
        auto finish_load = [&](uint32_t gu, bool last) {
            tc_wait_ld();
            if (last) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(gu % NT));
            }
        };

        for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
            const Item it = decode_item<BN, kSwap>(item, p, g_prefix);
            // grouped mode: slots beyond the last token tile carry no work; they cost a decode and nothing else
            if (it.c1 <= it.c0) continue;
            const uint32_t item_cur = item_no++;
            float2 acc[CPT / 2];
#pragma unroll
            for (int j = 0; j < CPT / 2; ++j) acc[j] = make_float2(0.0f, 0.0f);

            // token / weight-row coordinates of this thread
            const int64_t p_row = static_cast<int64_t>(it.p_idx) * kPRows + row;
            const int64_t q_base = (kSwap ? static_cast<int64_t>(it.row0) : static_cast<int64_t>(it.q_idx) * BN) + col0;
            const int64_t m_end = kSwap ? static_cast<int64_t>(it.row_end) : M;   // weight-major: token rows of this item end here
            const float* as_ptr;  // normal: this row's scales ; swap: scale matrix, indexed per token below
            const float* bs_ptr;
            if constexpr (!kSwap) {
                as_ptr = p.a_s + min(p_row, M - 1) * kc;
                bs_ptr = p.b_s + static_cast<int64_t>(it.q_idx) * kc;          // BN == 128
            } else {
                as_ptr = p.a_s;
                const float* bs_base = (p.n_groups > 0) ? p.g_bs[it.group] : p.b_s;
                bs_ptr = bs_base + static_cast<int64_t>(it.p_idx) * kc;        // 128 weight rows = one scale row
            }
            const int n_ch = it.c1 - it.c0;
            // Weight-major tiles: every thread needs a_s * b_s of all its tokens for every chunk; the
            // promotion warps put them into shared memory once per item ([chunk][token]) so that the
            // chunk loop reads them with a few broadcast vector loads.  (The host plan splits K so that an
            // item never has more chunks than the table holds.)
            if constexpr (kSwap) {
                {
                    bool mine = bounded_wait(tab_free_bar, (item_cur & 1u) ^ 1u, ctl, p.status, 7, item_cur);
                    ok = __all_sync(0xffffffffu, mine);
                    if (!ok) break;
                    const int tid = threadIdx.x - kFirstPromoWarp * 32;
                    for (int idx = tid; idx < n_ch * BN; idx += kPromoThreads) {
                        const int chl = idx / BN, col = idx - chl * BN;
                        const int64_t m = max(min(static_cast<int64_t>(it.row0) + col, m_end - 1), static_cast<int64_t>(0));
                        sc_tab[idx] = __ldg(as_ptr + m * kc + it.c0 + chl) * __ldg(bs_ptr + it.c0 + chl);
                    }
                    mbar_arrive(tab_ready_bar);
                    mine = bounded_wait(tab_ready_bar, item_cur & 1u, ctl, p.status, 8, item_cur);
                    ok = __all_sync(0xffffffffu, mine);
                    if (!ok) break;
                }
            }
            const int n_units = (n_ch + UC - 1) / UC;
            const int n_mine = n_units;
            auto unit_g = [&](int mu) -> uint32_t { return g + mu; };                        // pipeline counter
            auto unit_k = [&](int mu) -> int { return it.c0 + UC * mu; };                    // first K chunk of the unit
            auto unit_n = [&](int mu) -> int { return min(UC, it.c1 - unit_k(mu)); };        // chunks in the unit
            // scale of K chunk c for this thread's row (token-major tiles); clamped so that the
            // look-ahead never leaves the item
            auto row_scale = [&](int c) -> float {
                const int cc = min(c, it.c1 - 1);
                return __ldg(as_ptr + cc) * __ldg(bs_ptr + cc);
            };
            // acc[off ..] += v * (a_s * b_s) for K chunk ch; v holds HC columns starting at column 2*off
            auto fold = [&](int ch, const uint32_t* v, float sc, auto off_c) {
                constexpr int off = decltype(off_c)::value;
                if constexpr (!kSwap) {
                    const float2 sc2 = make_float2(sc, sc);
#pragma unroll
                    for (int j = 0; j < HC / 2; ++j)
                        acc[off + j] = __ffma2_rn(make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1])),
                                                  sc2, acc[off + j]);
                } else {
                    const float2* t2 = reinterpret_cast<const float2*>(sc_tab + (ch - it.c0) * BN + col0) + off;
#pragma unroll
                    for (int j = 0; j < HC / 2; ++j)
                        acc[off + j] = __ffma2_rn(make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1])),
                                                  t2[j], acc[off + j]);
                }
            };

            // Software pipeline over the load steps, two register buffers: while the FMAs of one step issue,
            // the TMEM load of the next step is in flight.
            uint32_t va[kBatched ? 1 : HC], vb[kBatched ? 1 : HC];
            if constexpr (kBatched) {
                if (n_mine > 0) {   // first unit of the item: wait and start its first load here
                    const uint32_t gu = unit_g(0);
                    const bool mine = wait_probed(probe, tfull_bar(gu % NT), (gu / NT) & 1u, ctl, p.status, 4, gu);
                    ok = __all_sync(0xffffffffu, mine);
                    if (ok) {
                        tc_fence_after();
                        tc_ld_x64(t_lane + ((gu % NT) * UC) * BN, va64);
                    }
                }
            } else {
                if (n_mine > 0) ok = issue_load(unit_g(0), 0, 0, va);
            }
            if constexpr (!kSwap) {
                static_assert(UC == 2, "token-major tiles pair two chunks per unit");
                // ---- token-major tiles: a thread reads its 64 columns of both
                // chunks of the unit in one batch (tcgen05.wait::ld has no per-load granularity, so one wait
                // per unit exposes the TMEM latency once), returns the TMEM stage at once and only then does
                // the FMAs; the other promotion warp of the scheduler overlaps with them.  Row scales (global
                // memory) are fetched one unit ahead.
                static_assert(CPT == 64, "token-major tiles: 64 columns per thread");
                float sa0 = row_scale(unit_k(0)), sa1 = row_scale(unit_k(0) + 1);     // this unit's two chunks
                for (int mu = 0; ok && mu < n_mine; ++mu) {
                    const uint32_t gu = unit_g(mu);
                    const int ts = gu % NT;
                    const int nch = unit_n(mu);
                    if (mu > 0) {
                        const bool mine = wait_probed(probe, tfull_bar(ts), (gu / NT) & 1u, ctl, p.status, 4, gu);
                        ok = __all_sync(0xffffffffu, mine);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    const uint32_t taddr = t_lane + (ts * UC) * BN;
                    if (mu > 0) tc_ld_x64(taddr, va64);
                    if (nch > 1) tc_ld_x64(taddr + BN, vb64);
                    float sb0 = 0.0f, sb1 = 0.0f;
                    if (mu + 1 < n_mine) {
                        sb0 = row_scale(unit_k(mu + 1));
                        sb1 = row_scale(unit_k(mu + 1) + 1);
                    }
                    tc_wait_ld();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar(ts));
                    // probe the next unit now: its answer is needed only after the FMAs below, by which time
                    // the probe has long returned (and the unit's MMAs, issued a unit ago, are usually complete)
                    probe = mbar_test_wait(tfull_bar((gu + 1) % NT), ((gu + 1) / NT) & 1u) ? 1u : 0u;
                    {
                        const float2 sc2 = make_float2(sa0, sa0);
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            acc[j] = __ffma2_rn(make_float2(__uint_as_float(va64[2 * j]), __uint_as_float(va64[2 * j + 1])),
                                                sc2, acc[j]);
                    }
                    if (nch > 1) {
                        const float2 sc2 = make_float2(sa1, sa1);
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            acc[j] = __ffma2_rn(make_float2(__uint_as_float(vb64[2 * j]), __uint_as_float(vb64[2 * j + 1])),
                                                sc2, acc[j]);
                    }
                    sa0 = sb0;
                    sa1 = sb1;
                }
            } else {
                // ---- weight-major tiles: a unit is one chunk (16- and 32-token tiles) or two (64-token tiles);
                // a chunk is read back in SPC steps, one trip covers max(2, SPC) steps
                constexpr int U = SPC > 2 ? SPC : 2;
                const int n_steps = n_ch * SPC;
                auto step = [&](int t, auto u_c, uint32_t* cur, uint32_t* nxt) {
                    constexpr int u = decltype(u_c)::value;
                    constexpr int st = u % SPC;
                    const int T = t + u;
                    if (!ok || T >= n_steps) return;
                    const int c = T / SPC;                              // chunk of the item
                    const bool last_of_unit = (st == SPC - 1) && ((c % UC) == UC - 1 || c == n_ch - 1);
                    finish_load(unit_g(c / UC), last_of_unit);
                    if (T + 1 < n_steps) {
                        const int cn = (T + 1) / SPC;
                        ok = issue_load(unit_g(cn / UC), cn % UC, (u + 1) % SPC, nxt);
                    }
                    fold(it.c0 + c, cur, 0.0f, std::integral_constant<int, st * (HC / 2)>{});
                };
                for (int t = 0; ok && t < n_steps; t += U) {
                    step(t, std::integral_constant<int, 0>{}, va, vb);
                    step(t, std::integral_constant<int, 1>{}, vb, va);
                    if constexpr (U == 4) {
                        step(t, std::integral_constant<int, 2>{}, va, vb);
                        step(t, std::integral_constant<int, 3>{}, vb, va);
                    }
                }
            }
            g += n_units;
            if (!ok) break;
            if constexpr (kSwap) {
                mbar_arrive(tab_free_bar);   // this thread is done reading the scale table
            }

            float* accf = reinterpret_cast<float*>(acc);

            // ---------------------------------------------------- write-out
            // normal: thread = token row, CPT consecutive output columns
            // swap  : thread = output column (weight row), CPT tokens
            bool write_out = true;
            if (p.splits > 1) {
                // Split-K: park the partial sums, take a ticket; the last arrival of the tile sums the
                // partial tiles in split order (deterministic) and writes the result.  Partial tiles use a
                // private layout chosen for coalescing, [split][tile][group of 4 columns][128 rows] float4:
                // a warp (32 consecutive rows, one column group) moves 512 contiguous bytes, and rows and
                // columns beyond M or N are stored like the rest, so nothing here is predicated and the
                // compiler is free to keep a whole batch of loads in flight.
                constexpr int kTileVec = BN * kPRows / 4;
                const int64_t split_stride = static_cast<int64_t>(p.tiles_p) * p.tiles_q * kTileVec;
                float4* tile_part = reinterpret_cast<float4*>(p.partials) + static_cast<int64_t>(it.tile) * kTileVec +
                                    (col0 / 4) * kPRows + row;
                {
                    float4* dst = tile_part + it.split * split_stride;
#pragma unroll
                    for (int j = 0; j < CPT / 4; ++j)
                        __stcg(dst + j * kPRows, make_float4(accf[4 * j], accf[4 * j + 1], accf[4 * j + 2], accf[4 * j + 3]));
                }
                // Release: the barrier orders every writer's stores before the ticket thread's fence, which
                // is cumulative.  The ticket slot alternates between items, so the next item's ticket cannot
                // overwrite this one before every thread has read it (a barrier of the next item lies between).
                const int slot = static_cast<int>(item_cur & 1u);
                promo_barrier<kWriters>();
                if (threadIdx.x == kFirstPromoWarp * 32) {
                    // one acquire-release atomic: releases the partial tiles (cumulative over the barrier above) and
                    // acquires the other splits' tiles for the reads below
                    int t;
                    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(t) : "l"(p.tickets + it.tile) : "memory");
                    if (t == p.splits - 1) p.tickets[it.tile] = 0;  // last arrival: leave the ticket clean
                    ctl->ticket[slot] = t;
                }
                promo_barrier<kWriters>();
                write_out = (ctl->ticket[slot] == p.splits - 1);
                if (write_out) {
#pragma unroll
                    for (int j = 0; j < CPT; ++j) accf[j] = 0.0f;
                    constexpr int kBatch = (CPT >= 64) ? 1 : 64 / CPT;   // splits whose loads are in flight together (64 registers)
                    for (int sp0 = 0; sp0 < p.splits; sp0 += kBatch) {
                        float4 t4[kBatch][CPT / 4];
#pragma unroll
                        for (int bi = 0; bi < kBatch; ++bi) {
                            const float4* src = tile_part + min(sp0 + bi, p.splits - 1) * split_stride;
#pragma unroll
                            for (int j = 0; j < CPT / 4; ++j) t4[bi][j] = __ldcg(src + j * kPRows);
                        }
#pragma unroll
                        for (int bi = 0; bi < kBatch; ++bi) {
                            if (sp0 + bi < p.splits) {
#pragma unroll
                                for (int j = 0; j < CPT / 4; ++j) {
                                    accf[4 * j] += t4[bi][j].x;
                                    accf[4 * j + 1] += t4[bi][j].y;
                                    accf[4 * j + 2] += t4[bi][j].z;
                                    accf[4 * j + 3] += t4[bi][j].w;
                                }
                            }
                        }
                    }
                }
            }
            if (write_out) {
                if constexpr (!kSwap) {
                    if (C::kStoreBytes > 0 && p.tma_store) {
                        // The four warps of a column half stage their 128 x 64 bf16 box in shared memory (128-byte
                        // swizzle: 16-byte slot c of row r sits at slot c ^ (r & 7), which also keeps the
                        // vector stores free of bank conflicts) and one thread hands it to the TMA, which clips
                        // rows beyond M and columns beyond N.  The store of the previous tile is only known to
                        // have read the buffer once its issuer has waited for it, hence the first barrier.
                        static_assert(CPT == 64, "one 128-byte box row per thread");
                        const int half = (warp - kFirstPromoWarp) >> 2;
                        uint8_t* sbuf = store_buf + half * (kPRows * 128);
                        const bool issuer = ((threadIdx.x & 127) == 0);
                        if (issuer) bulk_wait_group_read0();
                        asm volatile("bar.sync %0, 128;" ::"r"(2 + half) : "memory");
#pragma unroll
                        for (int cidx = 0; cidx < CPT / 8; ++cidx) {
                            const int j = cidx * 8;
                            const uint4 o = make_uint4(pack_bf16x2(accf[j], accf[j + 1]), pack_bf16x2(accf[j + 2], accf[j + 3]),
                                                       pack_bf16x2(accf[j + 4], accf[j + 5]), pack_bf16x2(accf[j + 6], accf[j + 7]));
                            *reinterpret_cast<uint4*>(sbuf + row * 128 + ((cidx ^ (row & 7)) << 4)) = o;
                        }
                        fence_proxy_async_shared();
                        asm volatile("bar.sync %0, 128;" ::"r"(2 + half) : "memory");
                        if (issuer) {
                            tma_store_2d(&tmap_c, smem_u32(sbuf), it.q_idx * BN + half * 64, it.p_idx * kPRows);
                            bulk_commit_group();
                        }
                    } else if (p_row < M) {
                        __nv_bfloat16* crow = p.c + p_row * N;
                        const bool vec_ok = (N % 8) == 0;
#pragma unroll
                        for (int j = 0; j < CPT; j += 8) {
                            const int64_t n = q_base + j;
                            if (vec_ok && n + 8 <= N) {
                                uint4 o = make_uint4(pack_bf16x2(accf[j], accf[j + 1]), pack_bf16x2(accf[j + 2], accf[j + 3]),
                                                     pack_bf16x2(accf[j + 4], accf[j + 5]), pack_bf16x2(accf[j + 6], accf[j + 7]));
                                *reinterpret_cast<uint4*>(crow + n) = o;
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; ++e)
                                    if (n + e < N) crow[n + e] = __float2bfloat16_rn(accf[j + e]);
                            }
                        }
                    }
                } else {
                    if (p_row < N) {
#pragma unroll
                        for (int j = 0; j < CPT; ++j) {
                            const int64_t m = q_base + j;
                            if (m < m_end) p.c[m * N + p_row] = __float2bfloat16_rn(accf[j]);
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    if (!kSwap && warp >= kFirstPromoWarp && (threadIdx.x & 127) == 0) bulk_wait_group0();   // result tiles have left shared memory
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
    if (warp == 1) {
        tc_fence_after();
        tc_dealloc(tmem_base, C::kTmemCols);
    }
}

// -------------------------------------------------------------------- host side

}  // namespace

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// [rows, K] bytes, row-major; box = 128 bytes x box_rows, 128-byte swizzle, zero fill outside.
int make_tmap(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_last_error("cuTensorMapEncodeTiled is not available from the driver");
        return DSV3_ERR_CUDA;
    }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kChunk), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld K=%lld box_rows=%d)", static_cast<int>(r),
                       static_cast<long long>(rows), static_cast<long long>(K), box_rows);
        return DSV3_ERR_CUDA;
    }
    return DSV3_OK;
}

// Result matrix [M, N] bf16, row-major; box = 64 columns (128 bytes) x 128 rows, 128-byte swizzle.
int make_tmap_out(CUtensorMap* map, void* base, int64_t M, int64_t N) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_last_error("cuTensorMapEncodeTiled is not available from the driver");
        return DSV3_ERR_CUDA;
    }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(N) * 2};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(kPRows)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled (result matrix) failed with CUresult %d (M=%lld N=%lld)", static_cast<int>(r),
                       static_cast<long long>(M), static_cast<long long>(N));
        return DSV3_ERR_CUDA;
    }
    return DSV3_OK;
}

namespace {

template <int BN, bool kSwap>
int launch_variant(const CUtensorMap& tp, const CUtensorMap& tq, const CUtensorMap& tc, const TcParams& prm,
                   cudaStream_t stream) {
    using C = Cfg<BN, kSwap>;
    auto kern = fp8_gemm_tc_kernel<BN, kSwap>;
    static bool configured[64] = {};
    int dev = 0;
    DSV3_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        DSV3_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        configured[dev] = true;
    }
    int grid = prm.num_items < num_sms() ? prm.num_items : num_sms();
    DSV3_CUDA_TRY(launch_dependent(kern, dim3(grid), dim3(kNumThreads), C::kSmemBytes, stream, tp, tq, tc, prm));
    return DSV3_OK;
}

}  // namespace

bool tc_supported(const void* a, const void* b, const void* c, int64_t M, int64_t N, int64_t K) {
    return M > 0 && N > 0 && K >= 16 && (K % 16) == 0 && (reinterpret_cast<uintptr_t>(a) % 16) == 0 &&
           (reinterpret_cast<uintptr_t>(b) % 16) == 0 && (reinterpret_cast<uintptr_t>(c) % 16) == 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31);
}

// Pinned values (dsv3_set_gemm_policy) are honoured or refused (pl.error), never rewritten; the automatic
// plan adapts freely.
TcPlan tc_plan(int64_t M, int64_t N, int64_t K, int force_kernel, int force_split) {
    TcPlan pl;
    pl.error = DSV3_OK;
    pl.pair = false;
    pl.wide = false;
    pl.splits = 1;
    pl.kc = static_cast<int>((K + kChunk - 1) / kChunk);
    pl.swap = (force_kernel == 3) || (force_kernel == 0 && M <= 64);
    if (pl.swap) {
        pl.bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
        pl.tiles_p = static_cast<int>((N + kPRows - 1) / kPRows);
        pl.tiles_q = static_cast<int>((M + pl.bn - 1) / pl.bn);
    } else {
        pl.bn = 128;
        pl.tiles_p = static_cast<int>((M + kPRows - 1) / kPRows);
        pl.tiles_q = static_cast<int>((N + 127) / 128);
    }
    const int64_t tiles = static_cast<int64_t>(pl.tiles_p) * pl.tiles_q;
    if (tiles * 64 >= (1ll << 31)) {     // the work-item counters are 32-bit (at most 64 splits)
        set_last_error("fp8_gemm: %lld output tiles are more than the work-item counter holds", static_cast<long long>(tiles));
        pl.error = DSV3_ERR_UNSUPPORTED;
        return pl;
    }
    int splits = 1;
    const int tab = pl.swap ? scale_tab_chunks(pl.bn) : (1 << 30);   // chunks per item the scale table holds
    if (force_split > 0) {
        splits = force_split;
        const char* why = nullptr;
        if (splits > pl.kc) why = "more splits than 128-wide K chunks";
        else if (splits > 1 && tiles > kMaxTickets) why = "more output tiles than the workspace header has tickets";
        else if ((pl.kc + splits - 1) / splits > tab) why = "K range per split exceeds the weight-major kernel's scale table";
        else if ((force_kernel == 4 || force_kernel == 6) && splits > 1) why = "the CTA-pair kernels do not split K";
        if (why) {
            set_last_error("fp8_gemm: pinned split factor %d cannot be used for M=%lld N=%lld K=%lld: %s", force_split,
                           static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(K), why);
            pl.error = DSV3_ERR_UNSUPPORTED;
            return pl;
        }
    } else if (force_kernel == 4 || force_kernel == 6) {
        splits = 1;
    } else if (tiles <= kMaxTickets) {
        // Splitting K fills idle SMs, but every split item pays for parking its partial tile, a fence and a
        // ticket, and the last arrival of a tile sums the partial tiles.  Estimate, fitted to B200
        // measurements (microseconds; the launch's fixed cost is the same for every factor and left out):
        //   rounds(S) * (chunks_per_item(S) * c + (S > 1 ? e0 + e1 * S : 0)),   rounds = ceil(tiles * S / SMs)
        // with c the time per K chunk of one CTA, never below the time the whole problem needs at HBM
        // bandwidth.  The factor with the lowest estimate wins (ties: fewer splits).
        const int sms = num_sms();
        const double c = pl.swap ? (pl.bn == 64 ? 0.30 : 0.22) : 0.26;
        const double e0 = pl.swap ? 2.2 : 2.3, e1 = pl.swap ? 0.2 * pl.bn / 64.0 : 0.5;
        const double hbm_floor = (static_cast<double>(N) * K + static_cast<double>(M) * K) / 6.0e6;
        double best = 1e30;
        for (int sfac = 1; sfac <= 8 && sfac <= pl.kc; ++sfac) {
            const int per_item = (pl.kc + sfac - 1) / sfac;
            if (per_item > tab) continue;
            const int64_t rounds = (tiles * sfac + sms - 1) / sms;
            double t = static_cast<double>(rounds) * per_item * c;
            if (t < hbm_floor) t = hbm_floor;
            if (sfac > 1) t += static_cast<double>(rounds) * (e0 + e1 * sfac);
            if (t < best - 1e-9) {
                best = t;
                splits = sfac;
            }
        }
    }
    if (force_split == 0 && (pl.kc + splits - 1) / splits > tab) {
        // the weight-major kernel keeps an item's scales in a shared-memory table: split K until an item fits
        splits = (pl.kc + tab - 1) / tab;
        if (splits > 32 || tiles > kMaxTickets) {
            if (force_kernel == 3) {
                set_last_error("fp8_gemm: K=%lld is too long for the weight-major kernel's scale table", static_cast<long long>(K));
                pl.error = DSV3_ERR_UNSUPPORTED;
                return pl;
            }
            return tc_plan(M, N, K, 2, 0);   // automatic choice, absurdly long K: token-major tiles instead
        }
    }
    pl.splits = splits;
    if (force_kernel == 4 && !tm_pair_supported(M, N, K, true)) {
        set_last_error("fp8_gemm: the CTA-pair kernel needs more than 128 tokens (M=%lld)", static_cast<long long>(M));
        pl.error = DSV3_ERR_UNSUPPORTED;
        return pl;
    }
    if (force_kernel == 6 && !tw_pair_supported(M, N, K, true)) {
        set_last_error("fp8_gemm: the 256-wide CTA-pair kernel needs more than 128 tokens and more than 128 weight rows (M=%lld, N=%lld)",
                       static_cast<long long>(M), static_cast<long long>(N));
        pl.error = DSV3_ERR_UNSUPPORTED;
        return pl;
    }
    if (!pl.swap && splits == 1) {
        pl.pair = force_kernel == 4 || (force_kernel == 0 && tm_pair_supported(M, N, K, false));
        pl.wide = force_kernel == 6;
        if (force_kernel == 0 && tw_pair_supported(M, N, K, false)) {
            // 256-wide pair tiles against the best 128-wide alternative, in units of one SM working through one
            // 128 x 128 tile: rounds over the machine times the tile's size, times the measured cost per flop of
            // the wide kernel relative to the alternative (B200: 0.90-0.94 for K >= 1536 against the 128-wide
            // pair kernel, 0.79-0.80 for shorter K against the single-CTA kernel).  Wide tiles lose where they
            // fill the machine's last round badly (few token tiles, N a small multiple of 256).
            const int sms = num_sms(), pairs = sms / 2;
            const int64_t pp = (static_cast<int64_t>(pl.tiles_p) + 1) / 2;
            const int64_t t_wide = pp * ((N + 255) / 256);
            const double cost_wide = static_cast<double>((t_wide + pairs - 1) / pairs) * 2.0 * (pl.kc >= 12 ? 0.92 : 0.80);
            const double cost_narrow = pl.pair ? static_cast<double>((pp * pl.tiles_q + pairs - 1) / pairs)
                                               : static_cast<double>((tiles + sms - 1) / sms);
            pl.wide = cost_wide <= cost_narrow;
        }
        pl.pair = pl.pair || pl.wide;
    }
    return pl;
}

size_t tc_workspace_bytes(const TcPlan& pl, int64_t M, int64_t N) {
    if (pl.splits <= 1) return 0;
    // one padded tile (128 x bn fp32) per (split, tile)
    (void)M;
    (void)N;
    return static_cast<size_t>(DSV3_WORKSPACE_HEADER_BYTES) +
           static_cast<size_t>(pl.splits) * pl.tiles_p * pl.tiles_q * kPRows * pl.bn * sizeof(float);
}

int launch_fp8_gemm_tc(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N,
                       int64_t K, void* c, void* workspace, size_t workspace_bytes, const TcPlan& pl,
                       cudaStream_t stream) {
    if (pl.splits > 1) {
        const size_t need = tc_workspace_bytes(pl, M, N);
        if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) % 256) != 0) {
            set_last_error("fp8_gemm: split-K needs a 256-byte aligned workspace of %zu bytes (got %zu)", need,
                           workspace ? workspace_bytes : static_cast<size_t>(0));
            return DSV3_ERR_WORKSPACE;
        }
    }
    if (pl.error != DSV3_OK) return pl.error;
    if (pl.wide) return launch_fp8_gemm_tw(a, a_s, b, b_s, M, N, K, c, stream);
    if (pl.pair) return launch_fp8_gemm_tm(a, a_s, b, b_s, M, N, K, c, stream);
    CUtensorMap tp, tq, tc;
    memset(&tc, 0, sizeof(tc));
    int rc;
    bool tma_store = false;
    if (pl.swap) {
        if ((rc = make_tmap(&tp, b, N, K, kPRows)) != DSV3_OK) return rc;
        if ((rc = make_tmap(&tq, a, M, K, pl.bn)) != DSV3_OK) return rc;
    } else {
        if ((rc = make_tmap(&tp, a, M, K, kPRows)) != DSV3_OK) return rc;
        if ((rc = make_tmap(&tq, b, N, K, pl.bn)) != DSV3_OK) return rc;
        tma_store = (N % 8) == 0;   // row pitch of the result must be a multiple of 16 bytes for a tensor map
        if (tma_store && (rc = make_tmap_out(&tc, c, M, N)) != DSV3_OK) return rc;
    }
    TcParams prm;
    prm.a_s = a_s;
    prm.b_s = b_s;
    prm.c = static_cast<__nv_bfloat16*>(c);
    prm.tickets = static_cast<int*>(workspace);
    prm.partials = workspace ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + DSV3_WORKSPACE_HEADER_BYTES)
                             : nullptr;
    prm.status = status_device_ptr();
    if (!prm.status) return DSV3_ERR_CUDA;
    prm.M = M;
    prm.N = N;
    prm.kc = pl.kc;
    prm.tiles_p = pl.tiles_p;
    prm.tiles_q = pl.tiles_q;
    prm.splits = pl.splits;
    prm.tma_store = tma_store ? 1 : 0;
    // Work order: `raster` token tiles share consecutive weight tiles.  For token-major tiles the group is
    // made as tall as keeps its activations (raster x 128 x K bytes) within about a quarter of L2, so that
    // the weights are streamed from HBM as few times as possible.
    prm.raster = 8;
    if (!pl.swap) {
        const int64_t fit = (32ll << 20) / (static_cast<int64_t>(kPRows) * K);
        prm.raster = static_cast<int>(fit < 8 ? 8 : (fit > 64 ? 64 : fit));
    }
    prm.div_splits = make_fast_div(static_cast<uint32_t>(prm.splits));
    prm.div_raster = make_fast_div(static_cast<uint32_t>(prm.raster));
    prm.div_per_group = make_fast_div(static_cast<uint32_t>(prm.raster) * static_cast<uint32_t>(prm.tiles_q));
    prm.div_tiles_p = make_fast_div(static_cast<uint32_t>(prm.tiles_p));
    prm.num_items = pl.tiles_p * pl.tiles_q * pl.splits;   // < 2^31: checked by tc_plan
    prm.g_tmaps = nullptr;
    prm.g_bs = nullptr;
    prm.g_seg = nullptr;
    prm.n_groups = 0;
    prm.g_slots = 0;
    if (pl.swap) {
        switch (pl.bn) {
            case 16: return launch_variant<16, true>(tp, tq, tc, prm, stream);
            case 32: return launch_variant<32, true>(tp, tq, tc, prm, stream);
            case 64: return launch_variant<64, true>(tp, tq, tc, prm, stream);
        }
    } else if (pl.bn == 128) {
        // long K: two promotion groups on alternate chunks; short K: the end-of-tile combine would
        // cost more than it saves
        return launch_variant<128, false>(tp, tq, tc, prm, stream);
    }
    set_last_error("fp8_gemm: no tcgen05 variant for tile width %d", pl.bn);
    return DSV3_ERR_UNSUPPORTED;
}


// ---------------------------------------------------------------------------------------------
// Grouped GEMM (MoE experts): one launch, group e multiplies rows [seg[e], seg[e+1]) of `a` with its
// own weight.  The table holds, in device memory, n tensor maps followed by n scale pointers.
// ---------------------------------------------------------------------------------------------
size_t group_table_bytes(int n) { return static_cast<size_t>(n) * (sizeof(CUtensorMap) + sizeof(const float*)); }

int build_group_table(void* table_dev, const void* const* weights, const float* const* scales, int n, int64_t N,
                      int64_t K, cudaStream_t stream) {
    if (n <= 0 || n > kMaxGroups) {
        set_last_error("group table: between 1 and %d groups are supported (got %d)", kMaxGroups, n);
        return DSV3_ERR_UNSUPPORTED;
    }
    if ((K % 16) != 0 || (reinterpret_cast<uintptr_t>(table_dev) % 64) != 0) {
        set_last_error("group table: needs K %% 16 == 0 and a 64-byte aligned table");
        return DSV3_ERR_UNSUPPORTED;
    }
    std::vector<uint8_t> host(group_table_bytes(n));
    CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(host.data());
    const float** sp = reinterpret_cast<const float**>(host.data() + static_cast<size_t>(n) * sizeof(CUtensorMap));
    for (int e = 0; e < n; ++e) {
        if (!weights[e] || !scales[e] || (reinterpret_cast<uintptr_t>(weights[e]) % 16) != 0) {
            set_last_error("group table: weight %d is null or not 16-byte aligned", e);
            return DSV3_ERR_INVALID_ARGUMENT;
        }
        CUtensorMap m;
        const int rc = make_tmap(&m, weights[e], N, K, kPRows);
        if (rc != DSV3_OK) return rc;
        memcpy(maps + e, &m, sizeof(m));
        sp[e] = scales[e];
    }
    DSV3_CUDA_TRY(cudaMemcpyAsync(table_dev, host.data(), host.size(), cudaMemcpyHostToDevice, stream));
    DSV3_CUDA_TRY(cudaStreamSynchronize(stream));   // `host` goes out of scope
    return DSV3_OK;
}

int launch_fp8_gemm_grouped(const void* table_dev, int n, const void* a, const float* a_s, const int* seg_dev,
                            int64_t rows_total, int64_t rows_hint, int64_t N, int64_t K, void* c, cudaStream_t stream) {
    if (rows_total <= 0 || N <= 0) return DSV3_OK;
    if (!tc_supported(a, a, c, rows_total, N, K) || n <= 0 || n > kMaxGroups) {
        set_last_error("grouped fp8_gemm: needs K %% 16 == 0, 16-byte aligned a and c, and 1..%d groups", kMaxGroups);
        return DSV3_ERR_UNSUPPORTED;
    }
    const int kc = static_cast<int>((K + kChunk - 1) / kChunk);
    if (kc > scale_tab_chunks(32)) {
        set_last_error("grouped fp8_gemm: K = %lld exceeds %d (scale table of the weight-major kernel)",
                       static_cast<long long>(K), scale_tab_chunks(32) * kChunk);
        return DSV3_ERR_UNSUPPORTED;
    }
    // the counts themselves live on the device: the token tile is sized for the expected load per group
    const int64_t expect = (rows_hint > 0 && rows_hint < rows_total) ? rows_hint : rows_total;
    const int64_t avg = (expect + n - 1) / n;
    int bn = avg <= 16 ? 16 : (avg <= 32 ? 32 : 64);
    if (kc > scale_tab_chunks(bn)) bn = 32;                // the 64-token variant's table is shorter
    CUtensorMap tq, dummy;
    int rc;
    if ((rc = make_tmap(&tq, a, rows_total, K, bn)) != DSV3_OK) return rc;
    memset(&dummy, 0, sizeof(dummy));
    TcParams prm;
    prm.a_s = a_s;
    prm.b_s = nullptr;
    prm.c = static_cast<__nv_bfloat16*>(c);
    prm.tickets = nullptr;
    prm.partials = nullptr;
    prm.status = status_device_ptr();
    if (!prm.status) return DSV3_ERR_CUDA;
    prm.M = rows_total;
    prm.N = N;
    prm.kc = kc;
    prm.tiles_p = static_cast<int>((N + kPRows - 1) / kPRows);
    prm.tiles_q = 1;
    prm.splits = 1;
    prm.raster = 8;
    prm.tma_store = 0;
    prm.div_splits = make_fast_div(1);
    prm.div_raster = make_fast_div(8);
    prm.div_per_group = make_fast_div(8);
    prm.div_tiles_p = make_fast_div(static_cast<uint32_t>(prm.tiles_p));
    prm.g_tmaps = static_cast<const CUtensorMap*>(table_dev);
    prm.g_bs = reinterpret_cast<const float* const*>(static_cast<const uint8_t*>(table_dev) +
                                                     static_cast<size_t>(n) * sizeof(CUtensorMap));
    prm.g_seg = seg_dev;
    prm.n_groups = n;
    prm.g_slots = static_cast<int>((rows_total + bn - 1) / bn) + n;
    const int64_t items = static_cast<int64_t>(prm.tiles_p) * prm.g_slots;
    if (items >= (1ll << 31)) {
        set_last_error("grouped fp8_gemm: too many work items");
        return DSV3_ERR_UNSUPPORTED;
    }
    prm.num_items = static_cast<int>(items);
    switch (bn) {
        case 16: return launch_variant<16, true>(dummy, tq, dummy, prm, stream);
        case 32: return launch_variant<32, true>(dummy, tq, dummy, prm, stream);
        default: return launch_variant<64, true>(dummy, tq, dummy, prm, stream);
    }
}

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded wait the tcgen05 kernels are built on: one thread waits, with the given limit, for
// an mbarrier phase that nothing will ever complete.  The wait runs out, records (kind 9, counter, CTA) in the
// status words and the kernel returns normally: nothing traps, faults or spins without a bound.
// ---------------------------------------------------------------------------------------------
namespace {

__global__ void bounded_wait_selftest_kernel(unsigned int* status, uint64_t limit_ns) {
    __shared__ uint64_t bar;
    __shared__ Control ctl;
    if (threadIdx.x == 0) {
        ctl.abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        mbar_fence_init();
        (void)bounded_wait_ns(smem_u32(&bar), 0, &ctl, status, 9, 0, limit_ns);
    }
}

}  // namespace

int launch_bounded_wait_selftest(uint64_t limit_ns, cudaStream_t stream) {
    unsigned int* status = status_device_ptr();
    if (!status) return DSV3_ERR_CUDA;
    bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, limit_ns);
    DSV3_CUDA_TRY(cudaGetLastError());
    return DSV3_OK;
}

}  // namespace dsv3
