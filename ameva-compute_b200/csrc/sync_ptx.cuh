// Shared-memory barrier (mbarrier) wrappers, bounded waits and ring counters shared by the TMA / bulk-copy pipelines.
#pragma once
#include "common.cuh"

namespace amv {
namespace ptx {

constexpr long long kWaitCycles = 2000000000ll;     // about one second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

struct Ctl {             // shared control words
    uint32_t tmem_base;
    volatile uint32_t abort;
    uint32_t trace_slot;   // timeline build only
};

// Bounded wait: false when the CTA is aborting (this or another thread ran out of budget). Waiters other than the MMA
// issuer back off between polls (BACKOFF): a spinning warp takes issue slots from the warps that share its scheduler.
// The blocked part of mbar_wait, out of line: the K loops of the callers keep only the first poll and a branch.
template <bool BACKOFF>
__device__ __noinline__ bool mbar_wait_blocked(uint32_t bar, uint32_t parity, Ctl* ctl, uint32_t* status, uint32_t tag,
                                               long long* waited) {
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (BACKOFF) __nanosleep(64);
        if ((++spins & 63u) == 0u) {
            if (ctl->abort) return false;
            if (clock64() - t0 > kWaitCycles) {
                ctl->abort = 1u;
                if (atomicCAS(status, DEV_STATUS_OK, DEV_STATUS_WAIT_TIMEOUT) == DEV_STATUS_OK) status[1] = tag;
                return false;
            }
        }
    }
    if (waited) *waited += clock64() - t0;   // diagnostic: cycles this thread spent blocked here
    return true;
}

template <bool BACKOFF = true>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Ctl* ctl, uint32_t* status, uint32_t tag,
                                          long long* waited = nullptr) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_blocked<BACKOFF>(bar, parity, ctl, status, tag, waited);
}

// Position in a ring of n slots: slot index and the parity of the current pass (no divisions in the K loop).
struct Ring {
    uint32_t idx, phase, n;
    __device__ __forceinline__ Ring(uint32_t slots) : idx(0u), phase(0u), n(slots) {}
    __device__ __forceinline__ void advance() {
        if (++idx == n) {
            idx = 0u;
            phase ^= 1u;
        }
    }
};

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

}  // namespace ptx
}  // namespace amv
