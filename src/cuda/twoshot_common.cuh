// Helpers of the two-shot allreduce kernel (nvls_kernel.cu): multimem accessors, vector copies, range splitting and
// the per-CTA cross-rank barrier.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "flags.cuh"
#include "kernels.h"
#include "vec_ops.cuh"

namespace ibcomm {
namespace dev {

constexpr int kNvlsThreads = 512;

template <typename T> struct Multimem {
  // Types without a multimem form (integers, fp64) only run the direct variant.
  __device__ __forceinline__ static uint4 LdReduce(const void*) { return make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ static void St(void*, uint4) {}
};

template <> struct Multimem<float> {
  __device__ __forceinline__ static uint4 LdReduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
  __device__ __forceinline__ static void St(void* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct Multimem<__half> {
  __device__ __forceinline__ static uint4 LdReduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
  __device__ __forceinline__ static void St(void* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct Multimem<__nv_bfloat16> {
  __device__ __forceinline__ static uint4 LdReduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
  __device__ __forceinline__ static void St(void* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};

// dst[b..e) = src[b..e) in 16-byte vectors, eight loads in flight per thread.
template <bool kStrongSrc>
__device__ __forceinline__ void CopyVectors(uint4* dst, const uint4* src, uint64_t b, uint64_t e) {
  constexpr int kU = 8;
  for (uint64_t i = b + threadIdx.x; i < e; i += static_cast<uint64_t>(blockDim.x) * kU) {
    uint4 v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t idx = i + static_cast<uint64_t>(u) * blockDim.x;
      if (idx < e) v[u] = kStrongSrc ? Ld16Strong(src + idx) : Ld16(src + idx);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t idx = i + static_cast<uint64_t>(u) * blockDim.x;
      if (idx < e) St16(dst + idx, v[u]);
    }
  }
}

// Units [b, e) of 16 bytes at `off` in every rank's buffer, summed in rank
// order (so the bits do not depend on who reduces), scaled, and handed to
// `store(index, value)`.  Peer loads are latency-bound: kU vectors per rank
// are in flight per thread, for at most kR ranks (kU * kR <= 8 keeps the
// loads in registers).
template <typename T, int kU, int kR, typename Store>
__device__ __forceinline__ void PeerReduceUnits(unsigned char* const* peer, int ws, uint64_t off, uint64_t b, uint64_t e,
                                                bool do_scale, double scale, Store store, unsigned tid, unsigned nthr) {
  using A = typename Acc<T>::type;
  constexpr int kVecElems = 16 / static_cast<int>(sizeof(T));
  for (uint64_t i = b + tid; i < e; i += static_cast<uint64_t>(nthr) * kU) {
    uint4 v[kU][kR];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t idx = i + static_cast<uint64_t>(u) * nthr;
#pragma unroll
      for (int q = 0; q < kR; ++q)
        if (q < ws && idx < e) v[u][q] = Ld16Strong(peer[q] + off + idx * 16);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t idx = i + static_cast<uint64_t>(u) * nthr;
      if (idx < e) {
        A acc[kVecElems];
        VecIO<T>::Load(v[u][0], acc);
#pragma unroll
        for (int q = 1; q < kR; ++q)
          if (q < ws) VecIO<T>::Add(v[u][q], acc);
        if (do_scale) {
#pragma unroll
          for (int k = 0; k < kVecElems; ++k) acc[k] = ScaleAcc<A>(acc[k], scale);
        }
        store(idx, VecIO<T>::Store(acc));
      }
    }
  }
}

// The kernels are compiled per world-size class kR (2, 4 or 8 ranks at most)
// with 8 / kR vectors in flight per rank: 2 ranks x 4 vectors, 4 x 2, 8 x 1.
// The whole CTA takes part ...
template <typename T, int kR, typename Store>
__device__ __forceinline__ void PeerReduce(unsigned char* const* peer, int ws, uint64_t off, uint64_t b, uint64_t e,
                                           bool do_scale, double scale, Store store) {
  PeerReduceUnits<T, kMaxRanks / kR, kR>(peer, ws, off, b, e, do_scale, scale, store, threadIdx.x, blockDim.x);
}
// ... or a group of `nthr` threads of it, numbered `tid` = 0 .. nthr - 1.
template <typename T, int kR, typename Store>
__device__ __forceinline__ void PeerReduceGroup(unsigned char* const* peer, int ws, uint64_t off, uint64_t b, uint64_t e,
                                                bool do_scale, double scale, Store store, unsigned tid, unsigned nthr) {
  PeerReduceUnits<T, kMaxRanks / kR, kR>(peer, ws, off, b, e, do_scale, scale, store, tid, nthr);
}
inline int RankClass(int world_size) { return world_size <= 2 ? 2 : (world_size <= 4 ? 4 : kMaxRanks); }

// Barrier between CTA `cta` of every rank.  Returns false when it gave up.
__device__ inline bool CrossRankBarrier(const PeerTable& peers, const WaitCtx& w, int cta, uint32_t phase, int* s_stop) {
  __syncthreads();
  const uint64_t val = (w.seq << 32) | phase;
  if (threadIdx.x < w.world_size && static_cast<int>(threadIdx.x) != w.rank) {
    // The release store orders everything this CTA wrote before the barrier
    // (observed by this thread through __syncthreads) ahead of the flag.
    StReleaseSys(&Ctl(peers, threadIdx.x)->bar[cta][w.rank], val);
    if (!WaitGE(&Ctl(peers, w.rank)->bar[cta][threadIdx.x], val, w, kWaitBarrier, threadIdx.x, static_cast<int>(phase)))
      *s_stop = 1;
  }
  __syncthreads();
  return *s_stop == 0;
}

template <typename T> struct HasMultimem { static constexpr bool value = false; };
template <> struct HasMultimem<float> { static constexpr bool value = true; };
template <> struct HasMultimem<__half> { static constexpr bool value = true; };
template <> struct HasMultimem<__nv_bfloat16> { static constexpr bool value = true; };

}  // namespace dev
}  // namespace ibcomm
