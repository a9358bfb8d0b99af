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

// Two flavours.  kSpin: tight polls (the softmax rows, whose hand-offs are on the critical path
// and arrive within tens of cycles).  kPark: mbarrier.try_wait with a suspend-time hint parks the
// thread in hardware until the phase completes or the hint runs out, so a role that mostly waits
// (loader, MMA issue) takes no issue slots from the arithmetic warps of its scheduler.  Between
// batches of polls, or parked tries, the waiter looks at the abort flag and the clock.
enum WaitMode : int { kSpin = 0, kPark = 1 };
constexpr uint32_t kParkNs = 2000;

template <int kMode>
__device__ __noinline__ void wait_slow(WaitContext* w, uint64_t* bar, uint32_t parity, int where) {
  uint64_t t0 = 0;
  for (;;) {
    if (kMode == kPark) {
      if (mbar_try_wait_hint(bar, parity, kParkNs)) return;
    } else {
#pragma unroll 1
      for (int k = 0; k < 256; ++k)
        if (mbar_try_wait(bar, parity)) return;
    }
    if (w->abort) return;
    const uint64_t now = globaltimer_ns();
    if (t0 == 0) t0 = now;
    if (now - t0 > w->limit_ns) break;
  }
  w->abort = 1;
  atomicCAS(w->status, 0, where);
}

// One inline poll; the bounded loop is a shared out-of-line function (code size).
template <int kMode = kSpin>
__device__ __forceinline__ void wait(WaitContext* w, uint64_t* bar, uint32_t parity, int where) {
  if (mbar_try_wait(bar, parity)) return;
  wait_slow<kMode>(w, bar, parity, where);
}

// Wait that ignores the abort flag (used while unwinding: copies and MMAs already in flight
// must land before shared or tensor memory is given back), with a limit of its own.
__device__ __noinline__ bool drain_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    if (mbar_try_wait_hint(bar, parity, kParkNs)) return true;
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}

}  // namespace sm100
