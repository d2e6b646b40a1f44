// One-shot all-reduce of a decode-sized bf16 tensor over peer-mapped buffers (NVLink / NVSwitch).
//
// Replaces `dist.all_reduce(y)` after a row-parallel Linear and after the MoE expert loop (inference/model.py:264,
// 692) when y is small (14 KB - 1 MB at decode batch 1 - 64): such a message is latency-bound, and a ring or tree
// collective pays several hops of launch and synchronisation latency for it.  Here every rank keeps an exported
// buffer (two slots) and one small kernel per rank does everything; CTA b of every rank owns stripe b of the tensor:
//   1. it copies this rank's partial sums of the stripe into the rank's exported slot (the partial was just written
//      by the GEMM and sits in L2),
//   2. tells CTA b of every peer "stripe b of my partial number seq is in place" (one release store per peer),
//   3. waits, with a bound, until CTA b of every peer has said the same,
//   4. reads the stripe of all partial sums with ordinary loads from peer memory (16 bytes per lane per peer), adds
//      them in fp32 in rank order (so every rank computes bit-identical sums) and writes bf16 into the output.
// No TMA, no multicast objects, no library kernel is handed a peer pointer: plain ld.global on peer addresses.
//
// The sequence number lives in device memory (the last CTA of a launch advances it), so a launch captured in a
// CUDA graph behaves the same on every replay.  Slots alternate with the parity of seq: a rank may start partial
// seq+1 while a slower peer still reads partial seq.  Partial seq+2 reuses the slot of seq, and by then every peer
// has finished reading it: a rank finishes launch seq+1 only after hearing a signal seq+1 from every peer, and a
// peer sends that from its launch seq+1, which starts after its launch seq (and all its reads) has completed.
//
// Bounded waits: a CTA that does not hear from a peer within the limit records (kind 10, seq, rank/peer) in the
// device status words and writes nothing; dsv3_check_device_status reports DSV3_ERR_DEVICE_TIMEOUT.
#include <cstring>

#include "common.cuh"

namespace dsv3 {

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 64;             // CTAs per launch: all resident at once on any B200, one flag line each
constexpr int kFlagWords = 8;            // uint32 per (rank, CTA) flag: 32 bytes
constexpr int kArThreads = 256;
constexpr uint32_t kMagic = 0x44535633u;
// layout of a rank's allocation: [private: seq, done counter][flags: kMaxRanks x kMaxCtas x 32 B][slot 0][slot 1]
constexpr size_t kPrivateBytes = 256;
constexpr size_t kFlagsBytes = static_cast<size_t>(kMaxRanks) * kMaxCtas * kFlagWords * 4;
constexpr size_t kHeaderBytes = kPrivateBytes + kFlagsBytes;

struct RankCtx {
    uint8_t* base[kMaxRanks];      // every rank's allocation, this rank's included
    const __nv_bfloat16* in;       // this rank's partial sums
    __nv_bfloat16* out;
    unsigned int* status;
    int rank, world;
};

struct ArParams {
    RankCtx ctx[2];          // [0] for a real launch; two entries when one launch plays two ranks (single-GPU test)
    int64_t slot_bytes;
    int64_t count;           // bf16 elements
    uint64_t limit_ns;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_acquire_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ uint4 ld_peer(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t* flag_of(uint8_t* base, int rank, int cta) {
    return reinterpret_cast<uint32_t*>(base + kPrivateBytes) + (static_cast<size_t>(rank) * kMaxCtas + cta) * kFlagWords;
}

__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(const ArParams p) {
    const RankCtx& c = p.ctx[blockIdx.y];
    __shared__ uint32_t s_seq;
    __shared__ int s_ok;
    griddep_launch_dependents();
    griddep_wait();                         // the producer of this rank's partial has finished: its stores are visible
    uint32_t* priv = reinterpret_cast<uint32_t*>(c.base[c.rank]);     // [0] sequence number, [1] CTAs done
    if (threadIdx.x == 0) {
        s_seq = *reinterpret_cast<volatile uint32_t*>(priv) + 1u;
        s_ok = 1;
    }
    __syncthreads();
    const uint32_t seq = s_seq;
    const int64_t slot_off = static_cast<int64_t>(kHeaderBytes) + static_cast<int64_t>(seq & 1u) * p.slot_bytes;
    // stripe of this CTA, in 16-byte vectors (the last CTA also takes the tail elements)
    const int64_t nvec = p.count / 8;
    const int64_t per = (nvec + gridDim.x - 1) / gridDim.x;
    const int64_t v0 = min(nvec, per * blockIdx.x), v1 = min(nvec, v0 + per);
    const int tail = (blockIdx.x == gridDim.x - 1) ? static_cast<int>(p.count - nvec * 8) : 0;
    // 1. this rank's stripe into its exported slot
    {
        uint4* dst = reinterpret_cast<uint4*>(c.base[c.rank] + slot_off);
        const uint4* src = reinterpret_cast<const uint4*>(c.in);
        for (int64_t i = v0 + threadIdx.x; i < v1; i += kArThreads) dst[i] = src[i];
        if (threadIdx.x < tail)
            reinterpret_cast<__nv_bfloat16*>(c.base[c.rank] + slot_off)[nvec * 8 + threadIdx.x] = c.in[nvec * 8 + threadIdx.x];
    }
    // The CTA barrier orders every thread's copy before the signalling threads' release stores, which are
    // cumulative: a peer that acquires the flag sees the whole stripe.
    __syncthreads();
    // 2. signal CTA b of every peer; 3. wait for CTA b of every peer
    if (threadIdx.x < c.world) {
        st_release_sys(flag_of(c.base[threadIdx.x], c.rank, blockIdx.x), seq);
        const uint32_t* f = flag_of(c.base[c.rank], threadIdx.x, blockIdx.x);
        uint64_t t0 = 0;
        for (uint32_t spins = 0;; ++spins) {
            if (static_cast<int32_t>(ld_relaxed_sys(f) - seq) >= 0) {
                fence_acquire_sys();
                break;
            }
            if ((spins & 63u) == 63u) {
                const uint64_t now = global_timer_ns();
                if (t0 == 0) {
                    t0 = now;
                } else if (now - t0 > p.limit_ns) {
                    if (atomicCAS(&c.status[0], 0u, 1u) == 0u) {
                        c.status[1] = 10u;                // all-reduce: a peer's signal did not arrive
                        c.status[2] = seq;
                        c.status[3] = (static_cast<uint32_t>(c.rank) << 16) | threadIdx.x;
                    }
                    s_ok = 0;
                    break;
                }
            }
        }
    }
    __syncthreads();
    if (s_ok) {
        // 4. reduce the stripe: 8 bf16 per lane per peer, fp32 sums in rank order.  The loads of two vectors from
        // every rank are issued before any of them is used: a peer load is an NVLink round trip, and one dependent
        // round trip per loop trip would dominate a decode-sized message.
        constexpr int kU = 2;
        for (int64_t i0 = v0 + threadIdx.x; i0 < v1; i0 += kU * kArThreads) {
            uint4 v[kU][kMaxRanks];
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int64_t i = i0 + u * kArThreads;
#pragma unroll
                for (int r = 0; r < kMaxRanks; ++r)
                    if (r < c.world && i < v1) v[u][r] = ld_peer(reinterpret_cast<const uint4*>(c.base[r] + slot_off) + i);
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int64_t i = i0 + u * kArThreads;
                if (i >= v1) break;
                float acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll
                for (int r = 0; r < kMaxRanks; ++r) {
                    if (r < c.world) {
                        const uint32_t w[4] = {v[u][r].x, v[u][r].y, v[u][r].z, v[u][r].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            acc[2 * j] += bf16_bits_to_float(w[j] & 0xFFFFu);
                            acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
                        }
                    }
                }
                reinterpret_cast<uint4*>(c.out)[i] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                                pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
            }
        }
        if (threadIdx.x < tail) {
            const int64_t e = nvec * 8 + threadIdx.x;
            float a = 0.0f;
            for (int r = 0; r < c.world; ++r)
                a += bf16_bits_to_float(*reinterpret_cast<const volatile uint16_t*>(c.base[r] + slot_off + e * 2));
            c.out[e] = __float2bfloat16_rn(a);
        }
    }
    // the last CTA of this rank's launch advances the sequence number (also after a time-out: the ranks stay in step)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(priv + 1, 1u) == gridDim.x - 1) {
            priv[1] = 0u;
            *reinterpret_cast<volatile uint32_t*>(priv) = seq;
            __threadfence();
        }
    }
}

struct Comm {
    uint32_t magic;
    int rank, world, device;
    size_t slot_bytes;           // capacity of one data slot
    uint8_t* base;               // this rank's allocation
    uint8_t* peer_base[kMaxRanks];
    bool opened[kMaxRanks];
    bool connected;
};

Comm* as_comm(void* h) {
    Comm* c = static_cast<Comm*>(h);
    if (!c || c->magic != kMagic) {
        set_last_error("p2p: not a communicator handle");
        return nullptr;
    }
    return c;
}

void fill_ctx(RankCtx* ctx, const Comm* c, const void* in, void* out, unsigned int* status) {
    for (int r = 0; r < kMaxRanks; ++r) ctx->base[r] = r < c->world ? c->peer_base[r] : nullptr;
    ctx->in = static_cast<const __nv_bfloat16*>(in);
    ctx->out = static_cast<__nv_bfloat16*>(out);
    ctx->status = status;
    ctx->rank = c->rank;
    ctx->world = c->world;
}

int check_call(const Comm* c, int64_t count, const void* in, const void* out) {
    if (!c->connected) {
        set_last_error("allreduce: the communicator is not connected to its peers");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (count < 0 || !in || !out || (reinterpret_cast<uintptr_t>(out) % 16) != 0 || (reinterpret_cast<uintptr_t>(in) % 16) != 0) {
        set_last_error("allreduce: negative count, or input / output null or not 16-byte aligned");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (static_cast<size_t>(count) * 2 > c->slot_bytes) {
        set_last_error("allreduce: %lld elements exceed the communicator's buffer of %zu bytes", static_cast<long long>(count),
                       c->slot_bytes);
        return DSV3_ERR_WORKSPACE;
    }
    return DSV3_OK;
}

int grid_for(int64_t count) {
    const int64_t nvec = count / 8;
    int64_t g = (nvec + kArThreads * 2 - 1) / (kArThreads * 2);      // two 16-byte vectors per thread while the CTAs last
    if (g < 1) g = 1;
    if (g > kMaxCtas) g = kMaxCtas;
    return static_cast<int>(g);
}

}  // namespace

}  // namespace dsv3

using namespace dsv3;

extern "C" {

size_t dsv3_p2p_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

int dsv3_p2p_create(int rank, int world, size_t max_bytes, void** comm_out, void* handle_out) {
    if (!comm_out || !handle_out || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || max_bytes == 0) {
        set_last_error("p2p_create: needs 1..%d ranks, 0 <= rank < world, a buffer size and two output pointers", kMaxRanks);
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    Comm* c = new Comm();
    memset(c, 0, sizeof(*c));
    c->magic = kMagic;
    c->rank = rank;
    c->world = world;
    DSV3_CUDA_TRY(cudaGetDevice(&c->device));
    c->slot_bytes = (max_bytes + 255) & ~static_cast<size_t>(255);
    const size_t total = kHeaderBytes + 2 * c->slot_bytes;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->base), total);
    if (e != cudaSuccess) {
        delete c;
        return cuda_fail(e, "cudaMalloc (p2p buffer)");
    }
    e = cudaMemset(c->base, 0, total);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle_out), c->base);
    if (e != cudaSuccess) {
        cudaFree(c->base);
        delete c;
        return cuda_fail(e, "cudaIpcGetMemHandle");
    }
    c->peer_base[rank] = c->base;
    *comm_out = c;
    return DSV3_OK;
}

int dsv3_p2p_connect(void* comm, const void* handles) {
    Comm* c = as_comm(comm);
    if (!c || !handles) return DSV3_ERR_INVALID_ARGUMENT;
    const cudaIpcMemHandle_t* h = static_cast<const cudaIpcMemHandle_t*>(handles);
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank || c->opened[r]) continue;
        void* ptr = nullptr;
        DSV3_CUDA_TRY(cudaIpcOpenMemHandle(&ptr, h[r], cudaIpcMemLazyEnablePeerAccess));
        c->peer_base[r] = static_cast<uint8_t*>(ptr);
        c->opened[r] = true;
    }
    c->connected = true;
    return DSV3_OK;
}

int dsv3_p2p_connect_local(void* comm, void* const* bases) {
    Comm* c = as_comm(comm);
    if (!c || !bases) return DSV3_ERR_INVALID_ARGUMENT;
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank) c->peer_base[r] = static_cast<uint8_t*>(bases[r]);
    c->connected = true;
    return DSV3_OK;
}

void* dsv3_p2p_base(void* comm) {
    Comm* c = as_comm(comm);
    return c ? c->base : nullptr;
}

int dsv3_allreduce_oneshot(void* comm, const void* in, void* out, int64_t count, uint64_t limit_ns, dsv3_stream_t stream) {
    Comm* c = as_comm(comm);
    if (!c) return DSV3_ERR_INVALID_ARGUMENT;
    const int rc = check_call(c, count, in, out);
    if (rc != DSV3_OK) return rc;
    if (count == 0) return DSV3_OK;
    ArParams prm;
    memset(&prm, 0, sizeof(prm));
    unsigned int* status = status_device_ptr();
    if (!status) return DSV3_ERR_CUDA;
    fill_ctx(&prm.ctx[0], c, in, out, status);
    prm.slot_bytes = static_cast<int64_t>(c->slot_bytes);
    prm.count = count;
    prm.limit_ns = limit_ns ? limit_ns : 1000ull * 1000ull * 1000ull;
    DSV3_CUDA_TRY(launch_dependent(allreduce_oneshot_kernel, dim3(grid_for(count), 1), dim3(kArThreads), 0,
                                   static_cast<cudaStream_t>(stream), prm));
    return DSV3_OK;
}

int dsv3_allreduce_oneshot_pair_on_one_gpu(void* comm0, void* comm1, const void* in0, const void* in1, void* out0, void* out1,
                                           int64_t count, uint64_t limit_ns, dsv3_stream_t stream) {
    Comm* c0 = as_comm(comm0);
    Comm* c1 = as_comm(comm1);
    if (!c0 || !c1) return DSV3_ERR_INVALID_ARGUMENT;
    int rc = check_call(c0, count, in0, out0);
    if (rc == DSV3_OK) rc = check_call(c1, count, in1, out1);
    if (rc != DSV3_OK) return rc;
    if (c0->world != 2 || c1->world != 2 || c0->rank != 0 || c1->rank != 1 || c0->slot_bytes != c1->slot_bytes) {
        set_last_error("allreduce (one-GPU pair): needs ranks 0 and 1 of a world of 2 with equal buffer sizes");
        return DSV3_ERR_INVALID_ARGUMENT;
    }
    if (count == 0) return DSV3_OK;
    ArParams prm;
    memset(&prm, 0, sizeof(prm));
    unsigned int* status = status_device_ptr();
    if (!status) return DSV3_ERR_CUDA;
    fill_ctx(&prm.ctx[0], c0, in0, out0, status);
    fill_ctx(&prm.ctx[1], c1, in1, out1, status);
    prm.slot_bytes = static_cast<int64_t>(c0->slot_bytes);
    prm.count = count;
    prm.limit_ns = limit_ns ? limit_ns : 1000ull * 1000ull * 1000ull;
    void* args[] = {&prm};
    DSV3_CUDA_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(allreduce_oneshot_kernel), dim3(grid_for(count), 2),
                                              dim3(kArThreads), args, 0, static_cast<cudaStream_t>(stream)));
    return DSV3_OK;
}

int dsv3_p2p_destroy(void* comm) {
    Comm* c = as_comm(comm);
    if (!c) return DSV3_ERR_INVALID_ARGUMENT;
    for (int r = 0; r < c->world; ++r)
        if (c->opened[r]) cudaIpcCloseMemHandle(c->peer_base[r]);
    cudaFree(c->base);
    c->magic = 0;
    delete c;
    return DSV3_OK;
}

}  // extern "C"
