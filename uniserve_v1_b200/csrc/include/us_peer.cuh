// System-scope flag helpers shared by the kernels that talk to other GPUs.
// Every wait is bounded: on expiry the caller records US_DEV_TIMEOUT_PEER in the
// status word and carries on; once the word is set later waits give up at once.
// The budget of a wait (SM clocks) is the 64-bit word at byte 8 of the status block
// (us_set_peer_wait_clocks; kWaitClocks when it was never set).
#pragma once
#include "us_common.cuh"

namespace peer {

constexpr int kMaxRanks = 8;
constexpr long long kWaitClocks = 3000000000LL;  // about 1.5 s

struct Table {
  uint8_t* base[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld16_sys(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st16_sys(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Spins until *flag >= epoch (wrap-safe).  Returns false when the budget ran out.
__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int epoch,
                                          unsigned int* status) {
  const long long t0 = clock64();
  long long budget = kWaitClocks;
  if (status) {
    const long long set = *reinterpret_cast<volatile long long*>(status + 2);
    if (set > 0) budget = set;
    if (*(volatile unsigned int*)status) budget = 0;
  }
  while ((int)(ld_acquire_sys(flag) - epoch) < 0) {
    if (clock64() - t0 > budget) {
      us_dev_fail(status, US_DEV_TIMEOUT_PEER);
      return false;
    }
  }
  return true;
}

}  // namespace peer
