/*
 * dsv3_b200 -- C ABI of the B200 (sm_100a) FP8 GEMM path for DeepSeek-V3 inference.
 *
 * Every entry point replaces one function of the reference's operator module
 * `inference/kernel.py` (imported by `inference/model.py:10` and
 * `inference/fp8_cast_bf16.py:10`) or a caller directly above it.  The reference
 * binds these names in Python; a drop-in `kernel.py` that calls this library
 * through ctypes is shipped next to it.
 *
 * Conventions
 *   - plain device pointers and 64-bit sizes; no framework types;
 *   - all tensors are row-major and contiguous, on the current CUDA device;
 *   - work is enqueued on `stream` (a cudaStream_t) and the call returns without
 *     synchronising; no entry point allocates device memory unless it says so;
 *   - the return value is 0 on success or a negative DSV3_ERR_* code; a
 *     human-readable detail of the last failure of the calling thread is
 *     available from dsv3_last_error().
 *   - e4m3 means float8_e4m3fn bytes; bf16 means bfloat16 bit patterns.
 */
#ifndef DSV3_B200_H_
#define DSV3_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSV3_OK 0
#define DSV3_ERR_INVALID_ARGUMENT (-1)  /* null pointer, negative size, bad block size      */
#define DSV3_ERR_UNSUPPORTED (-2)       /* shape or option the CUDA path does not implement */
#define DSV3_ERR_CUDA (-3)              /* a CUDA runtime / driver call failed              */
#define DSV3_ERR_WORKSPACE (-4)         /* workspace missing or too small                   */
#define DSV3_ERR_DEVICE_TIMEOUT (-5)    /* a bounded device-side wait gave up               */

#define DSV3_SCALE_FMT_FP32 0  /* scale_fmt=None  : s = amax/448                 (kernel.py:28)    */
#define DSV3_SCALE_FMT_UE8M0 1 /* scale_fmt="ue8m0": s = 2^ceil(log2(amax/448))  (kernel.py:29-31) */

typedef void* dsv3_stream_t; /* cudaStream_t */

/* Library version: major*10000 + minor*100 + patch. */
int dsv3_version(void);
const char* dsv3_strerror(int status);
const char* dsv3_last_error(void);

/*
 * act_quant -- replaces kernel.py:38-57 (kernel :9-35).
 *   x : bf16 [rows, K], K % block_size == 0 (the reference asserts this, :52)
 *   y : e4m3 [rows, K]           s : fp32 [rows, K / block_size]
 * Per block of block_size consecutive elements: s = max(amax,1e-4)/448, y = e4m3(x/s),
 * bit-identical to the reference kernel compiled for a GPU (approximate full-range
 * division, round-to-nearest-even saturating cast).  block_size must be a multiple
 * of 8 and at most 1024; 128 takes the tuned path.
 */
int dsv3_act_quant(const void* x, int64_t rows, int64_t K, int block_size, int scale_fmt,
                   void* y, float* s, dsv3_stream_t stream);

/*
 * SwiGLU + act_quant in one launch -- replaces `F.silu(w1(x)) * w3(x)` (model.py:532, 633) together with the
 * act_quant that linear() applies to the product in front of w2 (model.py:158-159).
 *   a, b : bf16 [rows, K] (the outputs of w1 and w3), K % 128 == 0
 *   y    : e4m3 [rows, K]    s : fp32 [rows, K / 128]
 * h = bf16(bf16(silu(a)) * b) with the rounding points of the framework's bf16 kernels, then (y, s) = act_quant(h);
 * h is not written.  Bit-identical to the three-launch form.
 */
int dsv3_swiglu_quant(const void* a, const void* b, int64_t rows, int64_t K, int scale_fmt, void* y, float* s,
                      dsv3_stream_t stream);

/*
 * weight_dequant -- replaces kernel.py:89-110 (kernel :60-86).
 *   w : e4m3 [N, K]   s : fp32 [ceil(N/block), ceil(K/block)]   y : bf16 [N, K]
 *   y = bf16(float(w) * s[n / block, k / block])
 */
int dsv3_weight_dequant(const void* w, const float* s, int64_t N, int64_t K, int block_size,
                        void* y, dsv3_stream_t stream);

/*
 * fp8_gemm -- replaces kernel.py:175-196 (kernel :118-172, tile configs :113-116).
 *   a : e4m3 [M, K]   a_s : fp32 [M, ceil(K/128)]
 *   b : e4m3 [N, K]   b_s : fp32 [ceil(N/128), ceil(K/128)]
 *   c : bf16 [M, N]   c = sum over 128-wide K chunks of (a_chunk . b_chunk^T) * a_s * b_s,
 *                     accumulated in fp32.
 * `workspace` is scratch for the split-K variants: at least
 * dsv3_fp8_gemm_workspace_bytes(M, N, K) bytes, 256-byte aligned, and its first
 * DSV3_WORKSPACE_HEADER_BYTES must be zero before the first call (every call leaves
 * them zero again).  One workspace must not be shared by calls that can overlap on
 * the GPU.  It may be NULL when the size query returns 0.
 */
#define DSV3_WORKSPACE_HEADER_BYTES 16384
size_t dsv3_fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);
int dsv3_fp8_gemm(const void* a, const float* a_s, const void* b, const float* b_s,
                  int64_t M, int64_t N, int64_t K, void* c,
                  void* workspace, size_t workspace_bytes, dsv3_stream_t stream);

/*
 * Decode-sized Linear in one launch -- replaces the FP8 branch of linear(), model.py:158-160
 * (`y = fp8_gemm(*act_quant(x, block_size, scale_fmt), weight, weight.scale)`), for at most 16 rows.
 *   x : bf16 [M, K], 1 <= M <= 16, K % 128 == 0      w : e4m3 [N, K]      w_s : fp32 [ceil(N/128), K/128]
 *   c : bf16 [M, N]
 * The activations are quantised in the kernel's prologue with the arithmetic of dsv3_act_quant (the FP8 codes
 * and scales the GEMM consumes are bit-identical to what dsv3_act_quant would have written), each 128-wide chunk
 * product is scaled as the reference does (acc += (dot * a_s) * b_s, kernel.py:162), K is split across warps and
 * CTA clusters and summed in a fixed order: the result is deterministic and lies within the fp8_gemm tolerance
 * of dsv3_act_quant followed by dsv3_fp8_gemm (the order of the fp32 partial sums differs).  No workspace.
 * Other shapes return DSV3_ERR_UNSUPPORTED: call the two operators instead.
 */
int dsv3_fp8_linear(const void* x, int64_t M, int64_t K, const void* w, const float* w_s, int64_t N,
                    int scale_fmt, void* c, dsv3_stream_t stream);

/*
 * fp8_gemm for hosts that have no device memory to lend -- no counterpart in the reference, whose
 * Python wrapper simply lets torch allocate.  Same arithmetic and the same kernels as dsv3_fp8_gemm,
 * but the split-K scratch is a fixed array of DSV3_STATIC_SCRATCH_BYTES inside the library image, so the
 * call performs no device allocation of any kind.  Meant for a process that committed all device
 * memory to its own arena at start-up (an allocation in the request path would fail, or would stall all
 * streams while the driver synchronises), and for C programs with no framework allocator to borrow from.
 *   - Every GPU that loads the library carries the array until the process exits.
 *   - When the automatic split-K plan needs more scratch than that, the call uses the largest split factor
 *     that fits (down to none); a split factor pinned with dsv3_set_gemm_policy that does not fit is refused
 *     with DSV3_ERR_WORKSPACE.  Shapes the tcgen05 kernels cannot take (K % 16 != 0, unaligned pointers)
 *     and gemm policy 1 (the CUDA-core kernel, which needs no scratch at all) are refused with
 *     DSV3_ERR_UNSUPPORTED.
 *   - The first call on a device looks up the array's device address (that device must be current); make
 *     that first call before starting any stream capture.
 *   - All calls on a device share the array: calls that can overlap on the GPU race on it.  The part that
 *     must start at zero is cleared on `stream` ahead of each launch.
 */
#define DSV3_STATIC_SCRATCH_BYTES (16384 + (8u << 20))
size_t dsv3_fp8_gemm_static_scratch_bytes(void);
int dsv3_fp8_gemm_static(const void* a, const float* a_s, const void* b, const float* b_s,
                         int64_t M, int64_t N, int64_t K, void* c, dsv3_stream_t stream);

/*
 * Kernel selection for fp8_gemm, for tests and benchmarks:
 *   0 = automatic (default), 1 = CUDA-core tiled kernel (any shape),
 *   2 = tcgen05 kernel, tokens on the MMA M axis, one CTA per 128 x 128 tile,
 *   3 = tcgen05 kernel, weights on the MMA M axis (small M),
 *   4 = tcgen05 kernel, tokens on the MMA M axis, CTA pairs on 256 x 128 tiles (needs M > 128, no split-K),
 *   5 = decode kernel (warp-level FP8 MMA on weights streamed through registers; needs M <= 16),
 *   6 = tcgen05 kernel, tokens on the MMA M axis, CTA pairs on 256 x 256 tiles (needs M > 128, N > 128, no split-K).
 * split_k = 0 lets the library choose.  A pinned kernel or split factor is honoured or the GEMM call fails
 * with DSV3_ERR_UNSUPPORTED (shape the kernel cannot take, split factor that does not fit); it is never
 * silently replaced.  The setting is one process-wide pair of integers read by every later dsv3_fp8_gemm /
 * dsv3_fp8_gemm_static call of any thread; change it only while no other thread is inside the library.
 */
int dsv3_set_gemm_policy(int kernel, int split_k);

/*
 * SMs the persistent tcgen05 GEMM kernels (and the plans that size split-K for them) may occupy; 0 = all
 * (default).  No counterpart in the reference.  For hosts that run a collective next to the GEMMs: a persistent
 * kernel that fills every SM keeps the collective's CTAs waiting until it ends, and the GEMM launched after that
 * finds SMs taken and runs a straggling round; leaving the collective its SMs (about as many as it has
 * channels) avoids both.  Process-wide like the policy above: read when a GEMM is launched (or captured), so it can
 * be changed between the launches of one captured graph; change it only while no other thread is inside the library.
 */
int dsv3_set_num_sms(int n);

/*
 * Grouped fp8_gemm over per-expert weights -- replaces the expert loop of MoE.forward
 * (model.py:683-689: one act_quant + fp8_gemm triple per expert and two host synchronisations per
 * expert) by one launch per projection.
 *   table    : device buffer of dsv3_group_table_bytes(n) bytes, 64-byte aligned, filled once by
 *              dsv3_group_table_build from host arrays of the n expert weight pointers (e4m3 [N, K] each)
 *              and scale pointers (fp32 [ceil(N/128), ceil(K/128)] each); the call synchronises `stream`.
 *   a, a_s   : e4m3 [rows_total, K] and fp32 [rows_total, ceil(K/128)]: the tokens routed to the experts,
 *              sorted by expert
 *   seg      : int32 [n + 1] in DEVICE memory: expert e owns rows [seg[e], seg[e+1]); rows at and
 *              beyond seg[n] are ignored.  Nothing is read back to the host.
 *   rows_hint: how many rows the n groups are expected to own together (seg[n] itself stays on the device), or 0
 *              if unknown (then rows_total).  Only a tuning input: it picks the token-tile width.  With tensor
 *              parallelism a rank owns n of the E experts and about rows_total * n / E of the rows.
 *   c        : bf16 [rows_total, N]; row r = a[r] @ weight[e(r)]^T with the block scales applied.
 * Limits: n <= 256, K <= 18432, K % 16 == 0.
 */
size_t dsv3_group_table_bytes(int n_groups);
int dsv3_group_table_build(void* table, const void* const* weights, const float* const* scales, int n_groups,
                           int64_t N, int64_t K, dsv3_stream_t stream);
int dsv3_fp8_gemm_grouped(const void* table, int n_groups, const void* a, const float* a_s, const int32_t* seg,
                          int64_t rows_total, int64_t rows_hint, int64_t N, int64_t K, void* c, dsv3_stream_t stream);

/*
 * Routing bookkeeping of the expert loop in one launch -- replaces `counts = torch.bincount(indices.flatten())`
 * and the per-expert `idx, top = torch.where(indices == i)` of model.py:680-686 (two host synchronisations per
 * expert in the reference).  Groups the (token, expert) pairs by local expert and orders every token's pairs by
 * expert id.  All arrays are device memory.
 *   indices : int64 [T, topk] expert ids           weights : float [T, topk] routing weights
 *   start, n_local : this rank owns experts [start, start + n_local), n_local <= 256, topk <= 32
 *   seg  : int32 [n_local + 1] out; seg[e] = first row of expert e, seg[n_local] = number of local pairs
 *   tok  : int32 [T*topk] out; token of the pair at each row (rows >= seg[n_local]: pairs of other ranks' experts)
 *   pair_row : int32 [T*topk] scratch
 *   pos_sorted : int32 [T, topk] out; w_sorted : bf16 [T, topk] out -- the `pos` and `w` of dsv3_moe_combine
 * The order of the rows inside one expert is not specified; no result depends on it.
 */
int dsv3_moe_route(const int64_t* indices, const float* weights, int64_t T, int topk, int start, int n_local,
                   int32_t* seg, int32_t* tok, int32_t* pair_row, int32_t* pos_sorted, void* w_sorted,
                   dsv3_stream_t stream);

/*
 * Scatter-add of the expert outputs -- the `y[idx] += expert(x[idx]) * weights[idx, top, None]` of
 * model.py:689 for all experts at once, with the same bf16 rounding (product, then every partial sum) and
 * the same ascending-expert order per token.
 *   o   : bf16 [rows, dim] expert outputs        pos : int32 [T, topk], row of `o` for the token's j-th
 *   w   : bf16 [T, topk] routing weights               smallest expert id, or -1 when that expert is not local
 *   y   : bf16 [T, dim] (overwritten)            dim % 8 == 0
 */
int dsv3_moe_combine(const void* o, const int32_t* pos, const void* w, int64_t T, int topk, int64_t dim, void* y,
                     dsv3_stream_t stream);

/*
 * One-shot all-reduce of a decode-sized bf16 tensor over peer-mapped buffers -- replaces `dist.all_reduce(y)` after
 * a row-parallel Linear and after the MoE expert loop (model.py:263-264, 691-692) for small y, where a ring or tree
 * collective is bound by latency.  One process per GPU; every rank
 *   1. dsv3_p2p_create(rank, world, max_bytes, &comm, handle): allocates (cudaMalloc, once) this rank's exported
 *      buffer and returns an inter-process handle of dsv3_p2p_handle_bytes() bytes;
 *   2. exchanges the handles with all ranks by any host channel (torch.distributed.all_gather_object, a file, ...);
 *   3. dsv3_p2p_connect(comm, handles): maps the peers' buffers (handles: world entries in rank order);
 *   4. per all-reduce: dsv3_allreduce_oneshot(comm, in, out, count, limit_ns, stream) on every rank, in the same
 *      order with the same count.  in: this rank's partial sums, out: the sum over ranks (may be the same pointer),
 *      both bf16 [count], 16-byte aligned, count * 2 <= max_bytes.  Sums are formed in fp32 in rank order, so all
 *      ranks obtain the same bits.  The call enqueues one kernel and returns; it may be captured in a CUDA graph.
 * Peer memory is read with ordinary loads; nothing is multicast.  Every device-side wait is bounded by limit_ns
 * (0 = one second): a rank that does not hear from a peer records the fact in the device status words
 * (dsv3_check_device_status returns DSV3_ERR_DEVICE_TIMEOUT) and leaves `out` unwritten.  All ranks must destroy
 * their communicators (dsv3_p2p_destroy) only after every rank's last all-reduce has completed.
 * dsv3_p2p_connect_local / dsv3_p2p_base / dsv3_allreduce_oneshot_pair_on_one_gpu serve tests that play two ranks
 * inside one process on one GPU: the two ranks' CTAs wait for each other, so they run as ONE cooperative launch.
 */
size_t dsv3_p2p_handle_bytes(void);
int dsv3_p2p_create(int rank, int world, size_t max_bytes, void** comm_out, void* handle_out);
int dsv3_p2p_connect(void* comm, const void* handles);
int dsv3_p2p_connect_local(void* comm, void* const* bases);
void* dsv3_p2p_base(void* comm);
int dsv3_allreduce_oneshot(void* comm, const void* in, void* out, int64_t count, uint64_t limit_ns, dsv3_stream_t stream);
int dsv3_allreduce_oneshot_pair_on_one_gpu(void* comm0, void* comm1, const void* in0, const void* in1, void* out0, void* out1,
                                           int64_t count, uint64_t limit_ns, dsv3_stream_t stream);
int dsv3_p2p_destroy(void* comm);

/*
 * Harness weight quantiser (the reference ships only the inverse, weight_dequant;
 * the checkpoint format is described in README_WEIGHTS.md:60-92).
 *   w : bf16 [N, K] -> q : e4m3 [N, K], s : fp32 [ceil(N/128), ceil(K/128)]
 *   per 128x128 block: s = max(amax,1e-4)/448 (IEEE division), q = e4m3(w / s).
 */
int dsv3_weight_quant(const void* w, int64_t N, int64_t K, void* q, float* s, dsv3_stream_t stream);

/*
 * Device status word.  Kernels with bounded waits record a give-up here instead of
 * spinning forever.  Synchronises `stream`, returns DSV3_OK or DSV3_ERR_DEVICE_TIMEOUT
 * and clears the word; `detail` (may be NULL) receives 4 words describing the wait.
 */
int dsv3_check_device_status(dsv3_stream_t stream, uint32_t detail[4]);

/*
 * Self-test of the bounded device-side wait: enqueues a one-thread kernel that waits for an mbarrier phase nothing
 * completes; after limit_ns (1 ns .. 1 s) the wait gives up and records kind 9 in the status words, so the next
 * dsv3_check_device_status returns DSV3_ERR_DEVICE_TIMEOUT.  The kernel returns normally; nothing faults or traps.
 * Callers of the GEMM entry points should poll dsv3_check_device_status at step boundaries: after a give-up the
 * affected result is incomplete.
 */
int dsv3_selftest_bounded_wait(uint64_t limit_ns, dsv3_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* DSV3_B200_H_ */
