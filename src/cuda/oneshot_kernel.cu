// One-shot allreduce for small messages: every rank stores its whole message
// into a slot of every peer's arena, raises one flag per peer, waits for the
// peers' flags and sums the world_size copies locally in rank order (so every
// rank computes bit-identical results).  One NVLink hop instead of the
// 2*(ws-1) hops of the ring: this is the latency end of the size sweep, for
// which the reference has no dedicated path.
//
// The slots are double-buffered by the parity of the call number, so
// consecutive calls need no exit barrier: a peer can only reach call k+2 after
// it consumed this rank's data of call k+1, which this rank sent after it had
// finished reading call k.
#include <cooperative_groups.h>

#include "flags.cuh"
#include "ibcomm/communicator.h"
#include "kernels.h"
#include "vec_ops.cuh"

namespace ibcomm {
namespace dev {

constexpr int kOneShotThreads = 512;

// Body of the one-shot kernel for one CTA; returns early when a wait gave up.
template <typename T>
__device__ void OneShotBody(const OneShotParams& p, uint64_t seq, int& s_stop) {
  using A = typename Acc<T>::type;
  constexpr int kVecElems = 16 / static_cast<int>(sizeof(T));
  const int cta = blockIdx.x, ncta = gridDim.x;
  const int ws = p.world_size, me = p.rank;
  // Slots are double-buffered by the parity of the call number; two one-shot
  // calls with the same parity always have another collective (with its entry
  // barrier) or a one-shot call of the other parity between them.
  const unsigned parity = static_cast<unsigned>(seq & 1u);
  const T* sendbuf = static_cast<const T*>(p.sendbuf);
  T* recvbuf = static_cast<T*>(p.recvbuf);

  WaitCtx w;
  w.peers = &p.peers;
  w.status = p.status;
  w.doorbell = p.doorbell;
  w.seq = seq;
  w.timeout_ns = p.timeout_ns;
  w.rank = me;
  w.world_size = ws;
  w.channel = cta;

  // This CTA's element range, on 16-byte vector boundaries.
  uint64_t lo, hi;
  {
    const uint64_t nvec = (p.len_elements + kVecElems - 1) / kVecElems;
    const uint64_t per = (nvec + static_cast<uint64_t>(ncta) - 1) / static_cast<uint64_t>(ncta);
    lo = per * static_cast<uint64_t>(cta) * kVecElems;
    hi = lo + per * kVecElems;
    if (lo > p.len_elements) lo = p.len_elements;
    if (hi > p.len_elements) hi = p.len_elements;
  }
  auto slot = [&](int owner_rank, int src_rank) -> T* {
    return reinterpret_cast<T*>(p.peers.arena[owner_rank] + p.slot_offset +
                                (static_cast<uint64_t>(parity) * static_cast<uint64_t>(ws) + static_cast<uint64_t>(src_rank)) * p.slot_bytes);
  };
  const bool aligned = ((reinterpret_cast<uintptr_t>(sendbuf) | reinterpret_cast<uintptr_t>(recvbuf)) & 15u) == 0;
  const uint64_t nfull = aligned ? (hi - lo) / kVecElems : 0;  // whole vectors handled by the vector path

  // (1) push my slice to every peer.
  for (int k = 1; k < ws; ++k) {
    const int q = (me + k) % ws;  // start with a different peer on every rank
    T* dst = slot(q, me);
    constexpr int kU = 4;  // vectors in flight per thread
    for (uint64_t i = threadIdx.x; i < nfull; i += static_cast<uint64_t>(blockDim.x) * kU) {
      uint4 v[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const uint64_t idx = i + static_cast<uint64_t>(u) * blockDim.x;
        if (idx < nfull) v[u] = Ld16(reinterpret_cast<const uint4*>(sendbuf + lo) + idx);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const uint64_t idx = i + static_cast<uint64_t>(u) * blockDim.x;
        if (idx < nfull) St16(reinterpret_cast<uint4*>(dst + lo) + idx, v[u]);
      }
    }
    for (uint64_t i = lo + nfull * kVecElems + threadIdx.x; i < hi; i += blockDim.x) dst[i] = sendbuf[i];
  }
  __syncthreads();
  // (2) tell them, (3) wait for theirs.
  if (threadIdx.x < ws && static_cast<int>(threadIdx.x) != me) {
    const int q = threadIdx.x;
    StReleaseSys(&Ctl(p.peers, q)->oneshot_flag[parity][cta][me], seq);  // release: the pushes above come first
    if (!WaitGE(&Ctl(p.peers, me)->oneshot_flag[parity][cta][q], seq, w, kWaitOneShot, q, -1)) s_stop = 1;
  }
  __syncthreads();
  if (s_stop) return;
  // (4) sum in rank order.
  const bool do_scale = p.scale != 1.0;
  for (uint64_t i = threadIdx.x; i < nfull; i += blockDim.x) {
    A acc[kVecElems];
#pragma unroll
    for (int e = 0; e < kVecElems; ++e) acc[e] = A(0);
    for (int q = 0; q < ws; ++q) {
      const uint4 v = (q == me) ? Ld16(reinterpret_cast<const uint4*>(sendbuf + lo) + i)
                                : Ld16Strong(reinterpret_cast<const uint4*>(slot(me, q) + lo) + i);
      VecIO<T>::Add(v, acc);
    }
    if (do_scale) {
#pragma unroll
      for (int e = 0; e < kVecElems; ++e) acc[e] = ScaleAcc<A>(acc[e], p.scale);
    }
    St16(reinterpret_cast<uint4*>(recvbuf + lo) + i, VecIO<T>::Store(acc));
  }
  for (uint64_t i = lo + nfull * kVecElems + threadIdx.x; i < hi; i += blockDim.x) {
    A acc = A(0);
    for (int q = 0; q < ws; ++q) acc += (q == me) ? ToAcc<A, T>(sendbuf[i]) : ToAcc<A, T>(LdScalarStrong<T>(slot(me, q) + i));
    if (do_scale) acc = ScaleAcc<A>(acc, p.scale);
    recvbuf[i] = FromAcc<T, A>(acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(kOneShotThreads, 1)
OneShotKernel(const __grid_constant__ OneShotParams p0, const OneShotParams* __restrict__ emu) {
  __shared__ OneShotParams p;
  __shared__ int s_stop;
  __shared__ uint64_t s_seq;
  {
    const uint32_t* src = (emu != nullptr) ? reinterpret_cast<const uint32_t*>(emu + blockIdx.y) : reinterpret_cast<const uint32_t*>(&p0);
    for (unsigned i = threadIdx.x; i < sizeof(OneShotParams) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(&p)[i] = src[i];
    if (threadIdx.x == 0) s_stop = 0;
  }
  __syncthreads();
  const uint64_t seq = BeginCollective(p.peers, p.rank, &s_seq);
  OneShotBody<T>(p, seq, s_stop);
  EndCollective(p.peers, p.rank, seq, gridDim.x);
}

}  // namespace dev

template <typename T>
static cudaError_t LaunchOneShotTyped(const OneShotParams& p, const OneShotParams* emu, int emu_ranks, int blocks, cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(emu != nullptr ? emu_ranks : 1));
  if (emu != nullptr) {
    void* args[] = {const_cast<OneShotParams*>(&p), &emu};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(dev::OneShotKernel<T>), grid, dim3(dev::kOneShotThreads), args, 0, stream);
  }
  dev::OneShotKernel<T><<<grid, dev::kOneShotThreads, 0, stream>>>(p, nullptr);
  return cudaGetLastError();
}

cudaError_t LaunchOneShotKernel(const OneShotParams& p, const OneShotParams* emu, int emu_ranks, int blocks, cudaStream_t stream) {
  switch (static_cast<DType>(p.dtype)) {
    case DType::kFloat32: return LaunchOneShotTyped<float>(p, emu, emu_ranks, blocks, stream);
    case DType::kFloat64: return LaunchOneShotTyped<double>(p, emu, emu_ranks, blocks, stream);
    case DType::kInt32: return LaunchOneShotTyped<int>(p, emu, emu_ranks, blocks, stream);
    case DType::kInt64: return LaunchOneShotTyped<long long>(p, emu, emu_ranks, blocks, stream);
    case DType::kFloat16: return LaunchOneShotTyped<__half>(p, emu, emu_ranks, blocks, stream);
    case DType::kBFloat16: return LaunchOneShotTyped<__nv_bfloat16>(p, emu, emu_ranks, blocks, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace ibcomm
