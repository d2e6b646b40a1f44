// fp8_gemm for sm_100a, token-major tiles on CTA pairs with 256-wide accumulators: two CTAs (a cluster of two
// SMs) work on one 256 x 256 tile, each holding 128 token rows x 256 weight columns, with software promotion of
// every 128-wide K chunk.
//
// Replaces inference/kernel.py:118-172 (fp8_gemm_kernel) and its launch at :194-195 for prefill-sized M.
//
// Why 256 columns.  A tcgen05.mma reads its operands from shared memory every time it is issued: M128 N128 K32
// (per SM) takes 8 KB for 64 tensor-core cycles, 128 B/clk, which is all shared memory delivers, and the TMA
// writes of the next operands compete for the same bandwidth; measured, such tiles stop at half of the tensor
// pipe's rate.  With N = 256 an instruction runs 128 cycles on 12 KB (4 KB of tokens, 8 KB of weights of which
// half sit in the peer's shared memory), 96 B/clk, and a chunk needs 32 KB of loads per SM for 512 tensor-core
// cycles instead of 24 KB for 256.  The price: the fp32 accumulator of one SM is 128 x 256 (128 registers in each
// of 256 promotion threads), TMEM holds only two chunk products, and the read-back buffers shrink to 2 x 32
// registers per thread.
//
// Roles, per CTA (r = rank in the pair; the even CTA is the leader):
//   warp 0 (1 lane)   TMA producer: stage = one K chunk = 16 KB tokens + 16 KB weights (this CTA's 128 of the
//                     tile's 256 weight rows), five stages.  Both producers' loads complete on the LEADER's full[]
//                     barrier (ordinary, non-multicast loads; only the completion signal crosses to the peer),
//                     each waits on its own empty[].
//   warps 1,2 (1 lane each)  leader only: MMA issuers; chunk g belongs to issuer g % 2, which owns TMEM slot g % 2.
//                     Per chunk: wait full[stage], wait tempty[slot] (16 arrivals: the promotion warps of both CTAs),
//                     4 x tcgen05.mma.cta_group::2 kind::f8f6f4 (M256 N256 K32), commit -> tfull[slot] and
//                     empty[stage] of both CTAs.  Stages alternate between the issuers, so full[] is waited for
//                     without a probe.
//   warps 4..11       promotion of this CTA's 128 x 256 half: warps 4..7 own columns 0..127 (one b_s block), warps
//                     8..11 columns 128..255; a thread owns one accumulator row.  A chunk product is read back in
//                     four pieces of 32 columns into two alternating buffers: while the tcgen05.ld of one piece is
//                     in flight the FMAs of the piece before issue; the last piece of a chunk is folded under the
//                     first load of the next chunk.  The slot goes back to the issuer when its last load has landed.
//                     Result tile: bf16 through shared memory and TMA stores.
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
// setmaxnreg.inc waits for registers of the CTA's pool, which is what the launch allocated (168 per thread, the
// most 384 threads can have): the two budgets must fit into it or the promotion warps would wait forever.
static_assert(128 * kRegsControl + 256 * kRegsPromo <= 384 * 168, "register pool");

constexpr int kBN = 256;                              // tile width: two b_s blocks, one per promotion warp group
constexpr int kBHalf = kBN / 2;                       // weight rows each CTA of the pair loads
constexpr int kChunkBytes = (kPRows + kBHalf) * kChunk;   // per CTA: token tile + half weight tile of one chunk
constexpr int kStorePasses = 1;                       // result tile staged whole (1) or one 64-column box per warp group at a time (2)
constexpr int kStages = kStorePasses == 1 ? 5 : 6;    // of one chunk each
constexpr int kSlots = 2;                             // TMEM slots of one chunk product (256 columns) each
constexpr int kTmemCols = kSlots * kBN;
constexpr int kPiece = 32;                            // columns per read-back
constexpr int kPieces = 128 / kPiece;                 // read-backs per chunk product and thread
static_assert(kPieces % 2 == 0, "a chunk's first piece goes to buffer 0 while buffer 1 holds the last piece of the chunk before");
constexpr int kStoreBytes = kPRows * kBN * 2 / kStorePasses;   // bf16 result tile: 128-byte-swizzled 128 x 64 boxes
constexpr int kSmemBytes = kStages * kChunkBytes + kStoreBytes + 1024 + 1024;
static_assert(kSmemBytes <= 232448, "shared memory per CTA");
static_assert(kSmemBytes > 116 * 1024, "one CTA per SM (it allocates all of TMEM)");
static_assert(kTmemCols == 512, "all of TMEM");
// The issuers alternate, so a stage's full[] barrier is waited for by one issuer at one use and by the other at the
// next.  A parity wait is only exact for a barrier that is at most one phase behind.  That holds here: an issuer
// reaches chunk g after it was given its TMEM slot for chunk g - 2, i.e. after the promotion warps have read chunk
// g - 4 and, in order, every chunk before it -- among them chunk g - kStages, the stage's previous use, whose
// product could only exist after the other issuer had waited for that use's loads.
static_assert(kStages >= 4 && kSlots == 2, "phase argument for the full[] waits of alternating issuers");
static_assert((kPRows * kChunk) % 1024 == 0 && kChunkBytes % 1024 == 0, "operand tiles keep the swizzle atom's alignment");

struct TwParams {
    const float* a_s;
    const float* b_s;
    __nv_bfloat16* c;
    unsigned int* status;
    int64_t M, N;
    int kc;                 // K chunks
    int nblk;               // rows of b_s (128-wide weight blocks)
    int tiles_pp, tiles_q;  // pairs of token tiles, 256-wide weight tiles
    int raster;             // token-tile pairs that share consecutive weight tiles in the work order
    FastDiv div_per_group, div_raster;
    int tma_store;          // results leave through shared memory and a TMA store (needs N % 8 == 0)
    int num_tiles;          // tiles_pp * tiles_q
};

struct Tile {
    int pp, q;
};

// Work order: `raster` token-tile pairs share consecutive weight tiles so that a wave re-uses both operands in L2.
__device__ __forceinline__ Tile decode_tile(int tile, const TwParams& p) {
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
fp8_gemm_tw_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_c, const TwParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;     // the same offset in both CTAs of the pair
    uint8_t* gen_tiles = smem_raw + (tiles - raw);
    uint8_t* store_buf = gen_tiles + kStages * kChunkBytes;                       // 1024-byte aligned (swizzle atom)
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
        const int n_pre = min(kc, kStages);
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
        if (warp == 0) {
            // ------------------------------------------------------------ TMA producer (both CTAs)
            // (converged warp, elected lane: see the issuers)
            {
                uint32_t g = 0;
                uint32_t probe = 0;   // result of test_wait on empty[] for chunk g, issued one chunk earlier
                bool ok = true;
                for (int tile = pair; ok && tile < p.num_tiles; tile += n_pairs) {
                    const Tile t = decode_tile(tile, p);
                    const int a_row = (2 * t.pp + static_cast<int>(rank)) * kPRows;
                    const int b_row = t.q * kBN + static_cast<int>(rank) * kBHalf;
                    for (int k = 0; k < kc; ++k, ++g) {
                        const int s = g % kStages;
                        ok = __all_sync(0xffffffffu, wait_probed(probe, empty_bar(s), ((g / kStages) & 1u) ^ 1u, ctl, p.status, 1, g));
                        if (!ok) break;
                        probe = mbar_test_wait(empty_bar((g + 1) % kStages), (((g + 1) / kStages) & 1u) ^ 1u) ? 1u : 0u;
                        const uint32_t lead_full = mapa_shared(full_bar(s), 0);
                        // the leader's barrier expects the bytes of both CTAs; the peer's loads may complete on it
                        // before this arrive has been made (the phase cannot complete without it)
                        const uint32_t dst = tiles + s * kChunkBytes;
                        if (elect_one()) {
                            if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * kChunkBytes);
                            tma_load_2d_pair(dst, &tmap_a, k * kChunk, a_row, lead_full);
                            tma_load_2d_pair(dst + kPRows * kChunk, &tmap_b, k * kChunk, b_row, lead_full);
                        }
                        __syncwarp();
                    }
                }
                // Nothing waits for the commits onto the empty[] barriers of the last chunks; wait for them here so
                // that none is in flight when the CTA leaves (it would land in whatever CTA gets this shared memory next).
                for (uint32_t d = (g > kStages ? g - kStages : 0u); ok && d < g; ++d)
                    ok = __all_sync(0xffffffffu, bounded_wait(empty_bar(d % kStages), (d / kStages) & 1u, ctl, p.status, 1, d));
            }
        } else if (warp <= 2) {
            // ------------------------------------------------------------ MMA issuers (leader CTA; chunk g -> issuer g % 2)
            // One thread issues about one tcgen05 instruction per hundred cycles, and a chunk costs eight (four MMAs,
            // four commits) for 512 tensor-core cycles: two threads share the chunks, each owning one TMEM slot.
            // The whole warp walks the loop (waits included) and one elected lane issues: control flow, addresses
            // and descriptors then stay warp-uniform, which is what makes a tcgen05 instruction cheap to issue.
            if (rank == 0) {
                constexpr uint32_t idesc = umma_idesc_e4m3_f32(2 * kPRows, kBN);
                const uint32_t me = static_cast<uint32_t>(warp - 1);
                const int slot = static_cast<int>(me);
                const uint32_t peer_tfull = mapa_shared(tfull_bar(slot), 1);
                const uint32_t peer_empty0 = mapa_shared(empty_bar(0), 1);
                const uint32_t d_tmem = tmem_base + slot * kBN;
                bool ok = true;
                uint32_t g = 0;
                for (int tile = pair; ok && tile < p.num_tiles; tile += n_pairs) {
                    for (int k = 0; k < kc; ++k, ++g) {
                        if ((g & 1u) != me) continue;
                        const int s = g % kStages;
                        ok = __all_sync(0xffffffffu, bounded_wait(full_bar(s), (g / kStages) & 1u, ctl, p.status, 2, g));
                        if (!ok) break;
                        ok = __all_sync(0xffffffffu, bounded_wait(tempty_bar(slot), ((g >> 1) & 1u) ^ 1u, ctl, p.status, 3, g));
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t sp = tiles + s * kChunkBytes;
                        const uint64_t da = umma_desc_k_major_sw128(sp);
                        const uint64_t db = umma_desc_k_major_sw128(sp + kPRows * kChunk);
                        if (elect_one()) {
#pragma unroll
                            for (int kk = 0; kk < kChunk / 32; ++kk) {
                                // 32 bytes further along K inside the 128-byte swizzle atom: +2 in address units of 16 B
                                tc_mma_f8_pair(d_tmem, da + 2u * kk, db + 2u * kk, idesc, kk > 0 ? 1u : 0u);
                            }
                            // this chunk's product is complete in the TMEM of both CTAs; the stage is reusable in both
                            tc_commit_pair(tfull_bar(slot));
                            tc_commit_pair(peer_tfull);
                            tc_commit_pair(empty_bar(s));
                            tc_commit_pair(peer_empty0 + 8u * s);
                        }
                        __syncwarp();
                    }
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsPromo));
        // ------------------------------------------------------------ promotion + epilogue (both CTAs)
        // Warps 4..7 own the left 128 columns of the CTA's 128 x 256 half, warps 8..11 the right 128; within a
        // column half a thread owns one accumulator row (TMEM lane).
        const int half = (warp - kFirstPromoWarp) >> 2;
        const int col0 = half * 128;
        const int quarter = warp & 3;                       // TMEM lane quarter this warp may access
        const int row = quarter * 32 + lane;                // accumulator row (TMEM lane)
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + col0;
        const uint32_t lead_tempty0 = mapa_shared(tempty_bar(0), 0);   // the leader's tempty[0], as seen from this CTA

        uint32_t v[2][kPiece];
        float2 acc[64];
        // fold piece `pc` of a chunk product (a constant once the loops around the calls are unrolled)
        auto fold = [&](const uint32_t* vv, float sc, int pc) {
            const float2 sc2 = make_float2(sc, sc);
#pragma unroll
            for (int j = 0; j < kPiece / 2; ++j)
                acc[pc * (kPiece / 2) + j] = __ffma2_rn(make_float2(__uint_as_float(vv[2 * j]), __uint_as_float(vv[2 * j + 1])), sc2,
                                                        acc[pc * (kPiece / 2) + j]);
        };
        auto load_piece = [&](uint32_t taddr, uint32_t* vv) {
            if constexpr (kPiece == 32) tc_ld_x32(taddr, vv);
            else tc_ld_x16(taddr, vv);
        };
        auto release = [&](int slot) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8u * slot);
        };
        // Result tile: the four warps of a column half stage their two 128 x 64 bf16 boxes in shared memory (128-byte
        // swizzle: 16-byte slot c of row r sits at slot c ^ (r & 7), which also keeps the vector stores free of
        // bank conflicts) and one thread hands them to the TMA, which clips rows beyond M and columns beyond N.
        // The stores of the previous tile are only known to have read the buffer once their issuer has waited for
        // them, hence the first barrier.  tp = token tile of this CTA.
        auto write_tile = [&](int tp, int tq) {
            if (static_cast<int64_t>(tp) * kPRows >= p.M) return;     // the odd half of the last pair: nothing to store
            const int64_t n0 = static_cast<int64_t>(tq) * kBN + col0;
            if (n0 >= p.N) return;                                    // the tile's right half lies beyond N
            if (p.tma_store) {
                constexpr int kBoxes = 2 / kStorePasses;               // boxes per warp group and pass
                uint8_t* sbuf = store_buf + half * (kBoxes * kPRows * 128);
                const bool issuer = (((threadIdx.x - kFirstPromoWarp * 32) & 127) == 0);
#pragma unroll
                for (int pass = 0; pass < kStorePasses; ++pass) {
                    if (issuer) bulk_wait_group_read0();
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + half) : "memory");
#pragma unroll
                    for (int c8 = 0; c8 < 8 * kBoxes; ++c8) {      // 16-byte slot of the thread's columns: box cc / 8, slot cc % 8
                        const int cc = pass * 8 * kBoxes + c8;
                        const uint4 o = make_uint4(pack_bf16x2(acc[4 * cc].x, acc[4 * cc].y), pack_bf16x2(acc[4 * cc + 1].x, acc[4 * cc + 1].y),
                                                   pack_bf16x2(acc[4 * cc + 2].x, acc[4 * cc + 2].y), pack_bf16x2(acc[4 * cc + 3].x, acc[4 * cc + 3].y));
                        *reinterpret_cast<uint4*>(sbuf + (c8 >> 3) * (kPRows * 128) + row * 128 + (((c8 & 7) ^ (row & 7)) << 4)) = o;
                    }
                    fence_proxy_async_shared();
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + half) : "memory");
                    if (issuer) {
#pragma unroll
                        for (int bx = 0; bx < kBoxes; ++bx) {
                            const int64_t n = n0 + (pass * kBoxes + bx) * 64;
                            if (n < p.N) tma_store_2d(&tmap_c, smem_u32(sbuf + bx * (kPRows * 128)), static_cast<int>(n), tp * kPRows);
                        }
                        bulk_commit_group();
                    }
                }
            } else {
                const int64_t m = static_cast<int64_t>(tp) * kPRows + row;
                const int64_t N = p.N;
                if (m < p.M) {
                    __nv_bfloat16* crow = p.c + m * N;
#pragma unroll
                    for (int j = 0; j < 64; ++j) {
                        if (n0 + 2 * j < N) crow[n0 + 2 * j] = __float2bfloat16_rn(acc[j].x);
                        if (n0 + 2 * j + 1 < N) crow[n0 + 2 * j + 1] = __float2bfloat16_rn(acc[j].y);
                    }
                }
            }
        };

        // Scale rows of a tile for this thread, as element offsets: a_s of its token (clamped at the edge), b_s of
        // the weight block of its column half (clamped where that half lies beyond N).
        auto as_row = [&](const Tile& t) {
            const int64_t tok = static_cast<int64_t>(2 * t.pp + static_cast<int>(rank)) * kPRows + row;
            return p.a_s + min(tok, p.M - 1) * kc;
        };
        auto bs_row = [&](const Tile& t) { return p.b_s + static_cast<int64_t>(min(2 * t.q + half, p.nblk - 1)) * kc; };

        bool ok = true;
        uint32_t g = 0;            // chunk counter
        int tile = pair;
        if (tile < p.num_tiles) {
            Tile cur = decode_tile(tile, p);
            float first = __ldg(as_row(cur)) * __ldg(bs_row(cur));     // product of the scales of the tile's first chunk
            while (true) {
                const float* as_ptr = as_row(cur);
                const float* bs_ptr = bs_row(cur);
                float sc = first;
#pragma unroll
                for (int j = 0; j < 64; ++j) acc[j] = make_float2(0.0f, 0.0f);
                for (int k = 0; k < kc; ++k, ++g) {
                    const int slot = static_cast<int>(g & 1u);
                    const bool mine = bounded_wait_lean(tfull_bar(slot), (g >> 1) & 1u, ctl, p.status, 4, g);
                    ok = __all_sync(0xffffffffu, mine);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t t_slot = t_lane + slot * kBN;
                    // The left 64 columns are read back and folded, then the right 64 are read back and the slot
                    // returns to the issuer: two read-back latencies per chunk; the last fold follows the release.
                    tc_ld_x64(t_slot, &v[0][0]);
                    // product of the scales of the tile's next chunk, one chunk ahead (clamped: the last re-reads its own)
                    const int kn = min(k + 1, kc - 1);
                    const float sc_next = __ldg(as_ptr + kn) * __ldg(bs_ptr + kn);
                    tc_wait_ld();
                    fold(v[0], sc, 0);
                    fold(v[1], sc, 1);
                    tc_ld_x64(t_slot + 2 * kPiece, &v[0][0]);
                    tc_wait_ld();
                    release(slot);
                    fold(v[0], sc, 2);
                    fold(v[1], sc, 3);
                    sc = sc_next;
                }
                if (!ok) break;
                // the next tile's first scales are requested before this tile is written, so that their latency
                // (and the tile decode) hides under the epilogue while the issuer already fills both TMEM slots
                const int next = tile + n_pairs;
                const bool more = next < p.num_tiles;
                Tile nt = cur;
                if (more) {
                    nt = decode_tile(next, p);
                    first = __ldg(as_row(nt)) * __ldg(bs_row(nt));
                }
                write_tile(2 * cur.pp + static_cast<int>(rank), cur.q);
                if (!more) break;
                tile = next;
                cur = nt;
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    if (warp >= kFirstPromoWarp && ((threadIdx.x - kFirstPromoWarp * 32) & 127) == 0) bulk_wait_group0();   // result tiles have left shared memory
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

bool tw_pair_supported(int64_t M, int64_t N, int64_t K, bool forced) {
    (void)K;
    (void)forced;
    // At least two token tiles (otherwise the second CTA of a pair would multiply zeros) and more than one weight
    // block (otherwise half of every accumulator would).  Whether it is the faster kernel for a problem is the
    // plan's decision (tc_plan).
    return M > kPRows && N > 128;
}

int launch_fp8_gemm_tw(const void* a, const float* a_s, const void* b, const float* b_s, int64_t M, int64_t N,
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
    TwParams prm;
    prm.a_s = a_s;
    prm.b_s = b_s;
    prm.c = static_cast<__nv_bfloat16*>(c);
    prm.status = status_device_ptr();
    if (!prm.status) return DSV3_ERR_CUDA;
    prm.M = M;
    prm.N = N;
    prm.kc = static_cast<int>((K + kChunk - 1) / kChunk);
    prm.nblk = static_cast<int>((N + 127) / 128);
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

    auto kern = fp8_gemm_tw_kernel;
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
