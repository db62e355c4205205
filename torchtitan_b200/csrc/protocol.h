// Flag primitives of the peer-memory protocols, for the device and for the host.
//
// The collectives of this framework order ranks with version flags in peer-mapped memory: a producer stores a version
// with release semantics after its data writes, a consumer loads with acquire semantics until the flag reaches the
// version it expects and only then touches the data. On the device these are `st.release.sys` / `ld.acquire.sys`; built
// for the host (no __CUDACC__) the same names map to C++ atomics, so the protocols' state machines can be exercised by
// CPU threads under ThreadSanitizer (tests/native/fsdp_flags_race.cc): plain data accesses that the flags do not order
// show up there as data races.
//
// Waits are bounded everywhere: `wait_flag_ge` gives up after `limit` polls (host) or nanoseconds (device) and returns
// false; callers record where they gave up and return.
#pragma once

#include <stdint.h>

#ifdef __CUDACC__

namespace tt {
namespace proto {

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Poll until *flag >= expected; false (with the last value seen in *seen) when `limit_ns` ran out.
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int expected, uint64_t t0, uint64_t limit_ns, int* seen) {
  int v;
  while ((v = ld_acquire_sys(flag)) < expected) {
    if (now_ns() - t0 > limit_ns) {
      *seen = v;
      return false;
    }
    __nanosleep(500);
  }
  *seen = v;
  return true;
}

}  // namespace proto
}  // namespace tt

#else  // host build: the same operations on C++ atomics

#include <atomic>
#include <thread>

namespace tt {
namespace proto {

inline int ld_acquire_sys(const int* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline void st_release_sys(int* p, int v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
inline bool wait_flag_ge(const int* flag, int expected, uint64_t /*t0*/, uint64_t limit_polls, int* seen) {
  int v;
  uint64_t polls = 0;
  while ((v = ld_acquire_sys(flag)) < expected) {
    if (++polls > limit_polls) {
      *seen = v;
      return false;
    }
    std::this_thread::yield();
  }
  *seen = v;
  return true;
}

}  // namespace proto
}  // namespace tt

#endif
