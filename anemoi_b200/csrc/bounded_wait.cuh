// Bounded mbarrier waits shared by the attention kernel and its self-test.
//
// No wait in this library spins without a limit.  A waiter polls the barrier; after
// `limit_ns` (measured with %globaltimer) it records `where` in the status word in global
// memory, raises the CTA's abort flag and returns.  Once the flag is up every other wait of
// the CTA returns at its next look at the flag, so all roles run their loops to the end with
// unchanged control flow, the CTA frees its tensor memory and exits; the host reads the status
// word (non-zero: the output of that launch is invalid).
#pragma once

#include <stdint.h>

#include "sm100_primitives.cuh"

namespace sm100 {

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// What a waiter needs, kept in shared memory (one copy per CTA, no registers held for it).
struct WaitContext {
  volatile int abort;  // raised by the first waiter that gives up
  int32_t* status;     // device status word (first give-up wins)
  uint64_t limit_ns;
};

// kSleepNs > 0: sleep between polls (roles that mostly wait and must not take issue slots
// from the arithmetic warps of their scheduler).
template <int kSleepNs>
__device__ __noinline__ void wait_slow(WaitContext* w, uint64_t* bar, uint32_t parity, int where) {
  uint64_t t0 = 0;
  for (;;) {
#pragma unroll 1
    for (int k = 0; k < (kSleepNs > 0 ? 32 : 128); ++k) {
      if (mbar_try_wait(bar, parity)) return;
      if (kSleepNs > 0) asm volatile("nanosleep.u32 %0;" ::"n"(kSleepNs));
    }
    if (w->abort) return;
    const uint64_t now = globaltimer_ns();
    if (t0 == 0) t0 = now;
    if (now - t0 > w->limit_ns) break;
  }
  w->abort = 1;
  atomicCAS(w->status, 0, where);
}

template <int kSleepNs = 0>
__device__ __forceinline__ void wait(WaitContext* w, uint64_t* bar, uint32_t parity, int where) {
  if (mbar_try_wait(bar, parity)) return;
  wait_slow<kSleepNs>(w, bar, parity, where);
}

// Wait that ignores the abort flag (used while unwinding: copies and MMAs already in flight
// must land before shared or tensor memory is given back), with a limit of its own.
__device__ __noinline__ bool drain_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int k = 0; k < 32; ++k) {
      if (mbar_try_wait(bar, parity)) return true;
      asm volatile("nanosleep.u32 64;");
    }
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}

}  // namespace sm100
