// Device helpers of the peer-memory exchange: system-scope flag stores / loads and the bounded flag wait.
#pragma once
#include "hb_common.cuh"

namespace hb {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// flag ≥ step (wrap-safe), polled at most err[kErrWaitPolls] times (the context's wait limit; 2^24 by default, seconds) with back-off;
// false = gave up.  Once the error word is set by
// anybody, waits return at once.
__device__ __forceinline__ bool ep_wait_flag(const uint32_t* flag, uint32_t step, uint32_t* err, uint32_t site) {
  const uint32_t limit = err[kErrWaitPolls];
  for (uint32_t it = 0; it < limit; ++it) {
    if ((int32_t)(ld_acquire_sys(flag) - step) >= 0) return true;
    if (it > 32) __nanosleep(it < 4096 ? 64 : 256);
    if ((it & 1023) == 1023 && *reinterpret_cast<volatile uint32_t*>(err)) return false;
  }
  atomicOr(err, site);
  return false;
}

}  // namespace hb
