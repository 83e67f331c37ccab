// mbarrier waits with a limit.  Every wait of the tensor-core kernels (TMA arrivals, MMA
// commits, hand-overs between warps) goes through mbar_wait: it is bounded by time, not by
// polls (a poll may itself block for a while).  When the limit passes, or as soon as another
// thread of the CTA has given up, it sets the CTA's abort flag and returns false; the caller
// records that in a status word, drains what it has in flight, frees its tensor memory and
// returns, so that the context stays usable and the host learns of it.
#pragma once
#include <stdint.h>

constexpr long long KIPP_WAIT_LIMIT_CYCLES = 2000000000ll;   // about a second of SM clocks: a wait that long has failed

__device__ __forceinline__ uint32_t kipp_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool kipp_mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(kipp_smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool kipp_mbar_wait_limited(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                       long long limit_cycles) {
    if (kipp_mbar_try_wait(bar, parity)) return true;      // mostly the phase is complete already: no clock read
    const long long t0 = clock64();
    for (unsigned i = 0;; ++i) {
        if (kipp_mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit_cycles) break;
        }
    }
    *abort_flag = 1;
    return false;
}
