// Flags in peer-addressable memory: system-scope release stores, acquire loads and a
// bounded wait.  A flag only ever grows (it carries the sequence number of the call that
// set it), so "arrived" is "flag >= target" in wrap-around arithmetic.
#pragma once

#include <cstdint>

namespace hb {

__device__ __forceinline__ uint32_t peer_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Orders every global store this thread has made or observed (a CTA barrier before the call
// extends that to the whole CTA) before the flag becomes visible to the peer.
__device__ __forceinline__ void peer_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// false when `limit` polls passed without the flag reaching `target`.
__device__ __forceinline__ bool peer_wait_ge(const uint32_t* p, uint32_t target, uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if ((int32_t)(peer_ld_acquire(p) - target) >= 0) return true;
    if (it > 64) __nanosleep(40);
  }
  return false;
}

}  // namespace hb
