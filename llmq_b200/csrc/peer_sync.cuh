// Flag words shared between GPUs: release-store / acquire-load at system scope and a bounded wait.
// Flags hold generation numbers that only grow; a wait that runs out returns false so the caller can record an
// error status and finish in an orderly way (a lost peer must never hang this GPU).
#pragma once
#include "ptx_sm100.cuh"

namespace peer {

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// true when *p >= target (wrap-around safe) was seen within the limit
__device__ __forceinline__ bool wait_flag(const unsigned int* p, unsigned int target, uint64_t limit_ns) {
    if (static_cast<int>(ld_acquire_sys(p) - target) >= 0) return true;
    const uint64_t t0 = sm100::globaltimer_ns();
    unsigned int spins = 0;
    while (static_cast<int>(ld_acquire_sys(p) - target) < 0) {
        if ((++spins & 63u) == 0u && sm100::globaltimer_ns() - t0 > limit_ns) return false;
        __nanosleep(64);
    }
    return true;
}
// Orders the acquire above before later async-proxy (TMA) reads of the data the flag guards.
__device__ __forceinline__ void fence_before_tma_reads() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

}  // namespace peer
