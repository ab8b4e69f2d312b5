// Bulk asynchronous copies (TMA, the non-tensor form `cp.async.bulk`) between
// this GPU's global memory and shared memory, with the mbarrier that tracks a
// load's bytes.  Used for LOCAL staging only: the source of a load and the
// destination of a store are always memory of the GPU that runs the kernel,
// and no form with cluster multicast exists in this library.  Addresses and
// sizes must be multiples of 16 bytes.  Every wait is bounded.
#pragma once

#include <cstdint>

namespace ibcomm {
namespace dev {

constexpr uint32_t kMbarSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t SmemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void MbarInit(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarInitFence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void MbarExpectTx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
// Bounded wait on a phase; false when the limit ran out.
__device__ __forceinline__ bool MbarWait(uint64_t* bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kMbarSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(SmemAddr(bar)), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// global -> shared; completion is counted in bytes on `bar`.
__device__ __forceinline__ void BulkLoad(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(SmemAddr(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(SmemAddr(bar))
               : "memory");
}
// shared -> global, as part of the thread's current bulk group.
__device__ __forceinline__ void BulkStore(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(SmemAddr(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void BulkCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of the thread's bulk groups still READ shared memory.
template <int N>
__device__ __forceinline__ void BulkWaitRead() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Waits until every bulk group of the thread is complete (its writes done).
__device__ __forceinline__ void BulkWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Orders accesses through the generic proxy (ordinary loads and stores, also
// those of other GPUs that a flag made visible) against accesses through the
// asynchronous proxy (the bulk copies), in both directions.
__device__ __forceinline__ void FenceProxyAsyncAll() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void FenceProxyAsyncShared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace dev
}  // namespace ibcomm
