// Hand-over between the three parties of a warp-specialised CTA (exec_kernel.cu,
// p2p_sendrecv.cu): a waiter thread that runs ahead and waits for the flags of
// the coming steps, data warps that stream step after step without a CTA-wide
// barrier, and a poster thread that follows behind, fences the data warps'
// stores and publishes the step's flags.  Counters in shared memory carry the
// hand-over: steps ready (written by the waiter) and, per data warp, steps
// done.  (One shared count of finished (warp, step) pairs would not do: the
// data warps are not in lock-step, and a warp that is two steps ahead would
// stand in for one that has not finished the step being published.)  All
// spins are bounded.
#pragma once

#include <cstdint>

#include "flags.cuh"

namespace ibcomm {
namespace dev {

constexpr int kMaxDataWarps = 16;

struct RoleSync {
  unsigned ready;                // steps whose flags have arrived (written by the waiter)
  unsigned done[kMaxDataWarps];  // per data warp: steps whose stores it has issued
  int stop;                      // a wait gave up or a self-check failed: everybody leaves
};

__device__ __forceinline__ void RoleSyncInit(RoleSync* s) {
  s->ready = 0;
  for (int i = 0; i < kMaxDataWarps; ++i) s->done[i] = 0;
  s->stop = 0;
}

__device__ __forceinline__ unsigned SmemU32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ unsigned LdAcquireShared(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(SmemU32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void StReleaseShared(unsigned* p, unsigned v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(SmemU32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void AddReleaseShared(unsigned* p, unsigned v) {
  asm volatile("red.release.cta.shared.add.u32 [%0], %1;" ::"r"(SmemU32(p)), "r"(v) : "memory");
}

// Spins until *counter >= target.  False when the call was stopped, or after
// twice the wait limit (a safety net: the waiter's own limit fires first).
__device__ __forceinline__ bool SpinShared(const unsigned* counter, unsigned target, RoleSync* sync, uint64_t timeout_ns) {
  if (LdAcquireShared(counter) >= target) return true;
  const uint64_t t0 = GlobalTimerNs();
  for (uint32_t spin = 1;; ++spin) {
    if (LdAcquireShared(counter) >= target) return true;
    if (*reinterpret_cast<volatile int*>(&sync->stop) != 0) return false;
    if ((spin & 1023u) == 0u && GlobalTimerNs() - t0 > 2 * timeout_ns) {
      *reinterpret_cast<volatile int*>(&sync->stop) = 1;
      return false;
    }
  }
}

// Spins until every one of the `warps` data warps has finished `target` steps.
__device__ __forceinline__ bool SpinAllWarpsDone(RoleSync* sync, int warps, unsigned target, uint64_t timeout_ns) {
  for (int w = 0; w < warps; ++w)
    if (!SpinShared(&sync->done[w], target, sync, timeout_ns)) return false;
  return true;
}

}  // namespace dev
}  // namespace ibcomm
