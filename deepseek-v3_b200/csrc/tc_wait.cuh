// Pieces shared by the tcgen05 fp8_gemm kernels: tile constants, the CTA control block and the
// bounded mbarrier wait.
#pragma once

#include "common.cuh"

namespace dsv3 {

constexpr int kPRows = 128;               // MMA M
constexpr int kChunk = 128;               // K elements (= bytes) per chunk
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;

struct Control {
    volatile uint32_t abort_flag;
    uint32_t tmem_base;
    volatile int ticket[2];
};

// Waits for the phase with the given parity.  The common case costs one or a few try_wait
// instructions; the wall-clock budget is only consulted after a few thousand failed polls (reading
// the global timer is slow enough to throttle the pipeline if it sat on the fast path).  When the
// budget (limit_ns) runs out the thread records what it was waiting for in the status words, raises
// the CTA-wide abort flag and returns false; it never traps and never spins without a bound.
__device__ __forceinline__ bool bounded_wait_ns(uint32_t bar, uint32_t parity, Control* ctl, unsigned int* status,
                                                uint32_t what, uint32_t g, uint64_t limit_ns) {
    uint64_t t0 = 0;
    for (uint32_t spins = 0;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if (spins >= 4096u && (spins & 255u) == 0u) {
            if (ctl->abort_flag) return false;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                ctl->abort_flag = 1;
                if (atomicCAS(&status[0], 0u, 1u) == 0u) {
                    status[1] = what;        // 1 empty, 2 full, 3 tmem-empty, 4 tmem-full, 7-8 scale table, 9 self-test
                    status[2] = g;           // chunk / unit counter of the waiting role
                    status[3] = blockIdx.x;
                }
                return false;
            }
        }
    }
}

__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, Control* ctl, unsigned int* status,
                                             uint32_t what, uint32_t g) {
    return bounded_wait_ns(bar, parity, ctl, status, what, g, kWaitLimitNs);
}

// The same wait for loops that are short of registers (the promotion loop of the 256-wide kernel): bounded by a
// poll count instead of the clock, so that the only state is one counter.  A failed try_wait suspends the thread for
// a hardware-defined time before it reports back, which makes the bound a matter of seconds.
constexpr uint32_t kWaitLimitPolls = 1u << 22;
__device__ __forceinline__ bool bounded_wait_lean(uint32_t bar, uint32_t parity, Control* ctl, unsigned int* status,
                                                  uint32_t what, uint32_t g) {
#pragma unroll 1
    for (uint32_t spins = 0; spins < kWaitLimitPolls; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 1023u) == 1023u && ctl->abort_flag) return false;
    }
    ctl->abort_flag = 1;
    if (atomicCAS(&status[0], 0u, 1u) == 0u) {
        status[1] = what;
        status[2] = g;
        status[3] = blockIdx.x;
    }
    return false;
}

// bounded_wait preceded by the result of an earlier probe of the same barrier and parity.
//
// A parity probe (mbarrier.test_wait.parity P) answers "has the phase with parity P completed?", which is
// true both when the wanted phase n has completed and when the barrier is still two phases behind (in phase
// n-1, whose predecessor n-2 has the same parity).  A probe may therefore only be trusted by a thread that
// itself waited for phase n-1 of that barrier (or otherwise knows it complete): then the barrier is in phase
// n-1 or n and the answer is exact.  Every probe in these kernels is issued by the thread that waited for the
// previous phase of the same barrier; where ownership of a barrier alternates between threads the barrier is
// waited for without a probe.
__device__ __forceinline__ bool wait_probed(uint32_t probed, uint32_t bar, uint32_t parity, Control* ctl,
                                            unsigned int* status, uint32_t what, uint32_t g) {
    return probed != 0u || bounded_wait(bar, parity, ctl, status, what, g);
}

}  // namespace dsv3
