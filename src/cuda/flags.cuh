// Device-side synchronisation primitives: system-scope acquire/release
// accesses to the peer-visible control words, the bounded wait every spin in
// this library goes through, and failure reporting.  A wait that runs out
// never traps or hangs: it records what it was waiting for, tells the other
// CTAs and the peers to stop, and makes the kernel return normally.
#pragma once

#include <cstdint>

#include "ibcomm/device_types.h"

namespace ibcomm {
namespace dev {

__device__ __forceinline__ uint64_t LdAcquireSys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t LdRelaxedSys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void StReleaseSys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void StRelaxedSys(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void FenceSys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ uint64_t GlobalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ ControlPage* Ctl(const PeerTable& peers, int rank) {
  return reinterpret_cast<ControlPage*>(peers.arena[rank]);
}

// What a waiter needs to know to give up cleanly.
struct WaitCtx {
  const PeerTable* peers;
  DeviceStatus* status;  // device memory
  uint32_t* doorbell;    // host-mapped word, set non-zero on failure
  uint64_t seq;
  uint64_t timeout_ns;
  int rank;
  int world_size;
  int channel;
};

__device__ inline void ReportFailure(const WaitCtx& w, uint32_t code, uint32_t kind, int peer, int op_index,
                                     uint64_t expected, uint64_t seen) {
  if (w.status != nullptr && atomicCAS(&w.status->code, 0u, code) == 0u) {
    w.status->kind = kind;
    w.status->rank = w.rank;
    w.status->peer = peer;
    w.status->channel = w.channel;
    w.status->op_index = op_index;
    w.status->expected = expected;
    w.status->seen = seen;
    w.status->seq = w.seq;
    __threadfence_system();
  }
  if (w.doorbell != nullptr) *reinterpret_cast<volatile uint32_t*>(w.doorbell) = code;
}

// Sequence number of the running collective: one more than the number this
// rank has completed.  Call with all threads of the CTA; `scratch` is a
// __shared__ word.
__device__ inline uint64_t BeginCollective(const PeerTable& peers, int rank, uint64_t* scratch) {
  if (threadIdx.x == 0) *scratch = LdRelaxedSys(&Ctl(peers, rank)->call_seq) + 1;
  __syncthreads();
  return *scratch;
}

// Every CTA of the rank calls this exactly once, on every path out of the
// kernel; the last one publishes the new count.  `ctas` = CTAs of this rank.
__device__ inline void EndCollective(const PeerTable& peers, int rank, uint64_t seq, unsigned ctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    ControlPage* me = Ctl(peers, rank);
    __threadfence();
    const unsigned prev = atomicAdd(&me->done_ctas, 1u);
    if (prev + 1 == ctas) {
      me->done_ctas = 0;
      __threadfence();
      StRelaxedSys(&me->call_seq, seq);
    }
  }
}

// Makes every CTA of every rank of this call stop waiting.
__device__ inline void BroadcastAbort(const WaitCtx& w) {
  for (int r = 0; r < w.world_size; ++r) StRelaxedSys(&Ctl(*w.peers, r)->abort_seq, w.seq);
  __threadfence_system();
}

// Spins until *flag >= target.  Returns false after the limit, or when this
// call was aborted elsewhere; the failure has then been reported.
__device__ inline bool WaitGE(const uint64_t* flag, uint64_t target, const WaitCtx& w, uint32_t kind, int peer,
                              int op_index) {
  uint64_t v = LdAcquireSys(flag);
  if (v >= target) return true;
  const uint64_t t0 = GlobalTimerNs();
  const uint64_t* abort_word = &Ctl(*w.peers, w.rank)->abort_seq;
  for (uint32_t spin = 1;; ++spin) {
    v = LdAcquireSys(flag);
    if (v >= target) return true;
    if ((spin & 31u) == 0u) {
      if (LdRelaxedSys(abort_word) == w.seq) {
        ReportFailure(w, kStatusPeerAbort, kind, peer, op_index, target, v);
        return false;
      }
      if (GlobalTimerNs() - t0 > w.timeout_ns) {
        ReportFailure(w, kStatusWaitTimeout, kind, peer, op_index, target, v);
        BroadcastAbort(w);
        return false;
      }
      if (spin > 4096u) __nanosleep(100);
    }
  }
}

}  // namespace dev
}  // namespace ibcomm
