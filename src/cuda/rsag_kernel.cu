// Reduce-scatter and all-gather: the two halves of the two-shot allreduce as
// collectives of their own (block r of the message belongs to rank r).  The
// reference has neither (its ring runs them back to back inside
// AllreduceRing, allreduce_cpu_impl.h:23-244); they are what tensor-, sequence-
// and fully-sharded data parallel code consumes.
//
//   reduce-scatter  in: ws blocks of m elements per rank   out: m elements
//                   rank r sums block r of every rank (switch `multimem.ld_reduce`,
//                   or peer loads added in rank order), scales, stores locally.
//   all-gather      in: m elements per rank                out: ws blocks of m
//                   rank r writes its block into block r of every rank's output
//                   (`multimem.st`, or one peer store per rank).
//
// The remote side (the input of a reduce-scatter, the output of an
// all-gather) is either a buffer every rank has mapped (symmetric memory or a
// registered buffer), used in place, or the arena's pool: then the message
// moves window by window, a window holding ws sub-blocks side by side, with
// the local copies in the same kernel.  CTA b always handles part b of every
// sub-block, on every rank and in every window, so the barriers are per CTA.
//
// Work is split in units of 16 bytes when a block is a whole number of them
// (the same decision on every rank), else in units of one element.  A user
// buffer that is only element-aligned is accessed element by element inside
// the same split.
#include <cooperative_groups.h>

#include "flags.cuh"
#include "ibcomm/communicator.h"
#include "kernels.h"
#include "twoshot_common.cuh"
#include "vec_ops.cuh"

namespace ibcomm {
namespace dev {

template <int kBytes> struct UIntOf;
template <> struct UIntOf<2> { using type = unsigned short; };
template <> struct UIntOf<4> { using type = unsigned int; };
template <> struct UIntOf<8> { using type = unsigned long long; };

// 16 bytes from / to a user buffer that may be only element-aligned.
template <typename T>
__device__ __forceinline__ uint4 LdUser16(const unsigned char* p, bool aligned) {
  if (aligned) return Ld16(p);
  using U = typename UIntOf<sizeof(T)>::type;
  constexpr int kN = 16 / static_cast<int>(sizeof(T));
  union { uint4 v; U e[kN]; } u;
  const U* s = reinterpret_cast<const U*>(p);
#pragma unroll
  for (int k = 0; k < kN; ++k) u.e[k] = s[k];
  return u.v;
}
template <typename T>
__device__ __forceinline__ void StUser16(unsigned char* p, uint4 v, bool aligned) {
  if (aligned) {
    St16(p, v);
    return;
  }
  using U = typename UIntOf<sizeof(T)>::type;
  constexpr int kN = 16 / static_cast<int>(sizeof(T));
  union { uint4 v; U e[kN]; } u;
  u.v = v;
  U* d = reinterpret_cast<U*>(p);
#pragma unroll
  for (int k = 0; k < kN; ++k) d[k] = u.e[k];
}

template <typename T, bool kMultimem, bool kVec, int kR>
__device__ void RsAgBody(const RsAgParams& p, uint64_t seq, int& s_stop) {
  using A = typename Acc<T>::type;
  constexpr int kUnitElems = kVec ? 16 / static_cast<int>(sizeof(T)) : 1;
  constexpr uint64_t kUnitBytes = kVec ? 16 : sizeof(T);
  const int cta = blockIdx.x, ncta = gridDim.x;
  const int ws = p.world_size, me = p.rank;
  WaitCtx w;
  w.peers = &p.peers;
  w.status = p.status;
  w.doorbell = p.doorbell;
  w.seq = seq;
  w.timeout_ns = p.timeout_ns;
  w.rank = me;
  w.world_size = ws;
  w.channel = cta;
  const unsigned char* send = static_cast<const unsigned char*>(p.sendbuf);
  unsigned char* recv = static_cast<unsigned char*>(p.recvbuf);
  const bool send_aligned = (reinterpret_cast<uintptr_t>(send) & 15u) == 0;
  const bool recv_aligned = (reinterpret_cast<uintptr_t>(recv) & 15u) == 0;
  const uint64_t block_units = p.block_elems / kUnitElems;
  const uint64_t win_units = p.window_elems / kUnitElems;
  const bool do_scale = p.scale != 1.0;
  uint32_t phase = 0;

  // Entry: CTA `cta` of every rank has started this call, so whatever used the
  // pool or the peers' buffers before it is over.
  if (!CrossRankBarrier(p.peers, w, cta, ++phase, &s_stop)) return;

  for (uint64_t w0 = 0; w0 < block_units; w0 += win_units) {
    const uint64_t wn = (block_units - w0 < win_units) ? block_units - w0 : win_units;
    uint64_t b, e;
    WindowPart(win_units, wn, 0, 1, cta, ncta, &b, &e);
    // Where unit i of this window sits inside a sub-block of the remote side.
    const uint64_t remote_base = p.staged ? 0 : w0 * kUnitBytes;
    const bool last = w0 + wn >= block_units;

    if (p.mode == kRsAgReduceScatter) {
      if (p.staged) {
        // Copy my part of every sub-block into my pool window.
        for (int s = 0; s < ws; ++s) {
          const unsigned char* src = send + (static_cast<uint64_t>(s) * block_units + w0) * kUnitBytes;
          unsigned char* dst = p.peer_buf[me] + static_cast<uint64_t>(s) * p.sub_stride_bytes;
          for (uint64_t i = b + threadIdx.x; i < e; i += blockDim.x) {
            if constexpr (kVec) {
              St16(dst + i * 16, LdUser16<T>(src + i * 16, send_aligned));
            } else {
              reinterpret_cast<T*>(dst)[i] = reinterpret_cast<const T*>(src)[i];
            }
          }
        }
        if (!CrossRankBarrier(p.peers, w, cta, ++phase, &s_stop)) return;
      }
      const uint64_t off = static_cast<uint64_t>(me) * p.sub_stride_bytes + remote_base;
      unsigned char* out = recv + w0 * kUnitBytes;
      if constexpr (kVec && kMultimem) {
        for (uint64_t i = b + threadIdx.x; i < e; i += blockDim.x) {
          uint4 r = Multimem<T>::LdReduce(p.mc_buf + off + i * 16);
          if (do_scale) {
            A acc[kUnitElems];
            VecIO<T>::Load(r, acc);
#pragma unroll
            for (int k = 0; k < kUnitElems; ++k) acc[k] = ScaleAcc<A>(acc[k], p.scale);
            r = VecIO<T>::Store(acc);
          }
          StUser16<T>(out + i * 16, r, recv_aligned);
        }
      } else if constexpr (kVec) {
        PeerReduce<T, kR>(p.peer_buf, ws, off, b, e, do_scale, p.scale,
                      [&](uint64_t idx, uint4 r) { StUser16<T>(out + idx * 16, r, recv_aligned); });
      } else {
        for (uint64_t i = b + threadIdx.x; i < e; i += blockDim.x) {
          A acc = A(0);
          for (int q = 0; q < ws; ++q) acc += ToAcc<A, T>(LdScalarStrong<T>(reinterpret_cast<const T*>(p.peer_buf[q] + off) + i));
          if (do_scale) acc = ScaleAcc<A>(acc, p.scale);
          reinterpret_cast<T*>(out)[i] = FromAcc<T, A>(acc);
        }
      }
      // The peers have read my window (my buffer): it may be overwritten.
      if (!CrossRankBarrier(p.peers, w, cta, ++phase, &s_stop)) return;
    } else {
      // All-gather: my part of the window goes into sub-block `me` everywhere.
      const unsigned char* src = send + w0 * kUnitBytes;
      const uint64_t off = static_cast<uint64_t>(me) * p.sub_stride_bytes + remote_base;
      for (uint64_t i = b + threadIdx.x; i < e; i += blockDim.x) {
        if constexpr (kVec) {
          const uint4 v = LdUser16<T>(src + i * 16, send_aligned);
          if constexpr (kMultimem) {
            Multimem<T>::St(p.mc_buf + off + i * 16, v);
          } else {
#pragma unroll
            for (int q = 0; q < kMaxRanks; ++q)
              if (q < ws) St16(p.peer_buf[q] + off + i * 16, v);
          }
        } else {
          const T v = reinterpret_cast<const T*>(src)[i];
          for (int q = 0; q < ws; ++q) reinterpret_cast<T*>(p.peer_buf[q] + off)[i] = v;
        }
      }
      // Everybody's part `cta` has arrived here.
      if (!CrossRankBarrier(p.peers, w, cta, ++phase, &s_stop)) return;
      if (p.staged) {
        for (int s = 0; s < ws; ++s) {
          const unsigned char* from = p.peer_buf[me] + static_cast<uint64_t>(s) * p.sub_stride_bytes;
          unsigned char* to = recv + (static_cast<uint64_t>(s) * block_units + w0) * kUnitBytes;
          for (uint64_t i = b + threadIdx.x; i < e; i += blockDim.x) {
            if constexpr (kVec) {
              StUser16<T>(to + i * 16, Ld16Strong(from + i * 16), recv_aligned);
            } else {
              reinterpret_cast<T*>(to)[i] = LdScalarStrong<T>(reinterpret_cast<const T*>(from) + i);
            }
          }
        }
        // My window is free again before anybody writes the next one into it.
        if (!last && !CrossRankBarrier(p.peers, w, cta, ++phase, &s_stop)) return;
      }
    }
  }
}

template <typename T, bool kMultimem, bool kVec, int kR>
__global__ void __launch_bounds__(kNvlsThreads, 1) RsAgKernel(const __grid_constant__ RsAgParams p0, const RsAgParams* __restrict__ emu) {
  __shared__ RsAgParams p;
  __shared__ int s_stop;
  __shared__ uint64_t s_seq;
  {
    const uint32_t* src = (emu != nullptr) ? reinterpret_cast<const uint32_t*>(emu + blockIdx.y) : reinterpret_cast<const uint32_t*>(&p0);
    for (unsigned i = threadIdx.x; i < sizeof(RsAgParams) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(&p)[i] = src[i];
    if (threadIdx.x == 0) s_stop = 0;
  }
  __syncthreads();
  const uint64_t seq = BeginCollective(p.peers, p.rank, &s_seq);
  RsAgBody<T, kMultimem, kVec, kR>(p, seq, s_stop);
  EndCollective(p.peers, p.rank, seq, gridDim.x);
}

}  // namespace dev

template <typename T, bool kMultimem, bool kVec, int kR>
static cudaError_t LaunchRsAgU(const RsAgParams& p, const RsAgParams* emu, int emu_ranks, int blocks, cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(emu != nullptr ? emu_ranks : 1));
  if (emu != nullptr) {
    // Emulated ranks wait on each other inside this launch: cooperative, so
    // the runtime refuses a grid that cannot be co-resident.
    void* args[] = {const_cast<RsAgParams*>(&p), &emu};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(dev::RsAgKernel<T, kMultimem, kVec, kR>), grid, dim3(dev::kNvlsThreads), args, 0, stream);
  }
  dev::RsAgKernel<T, kMultimem, kVec, kR><<<grid, dev::kNvlsThreads, 0, stream>>>(p, nullptr);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t LaunchRsAgTyped(const RsAgParams& p, const RsAgParams* emu, int emu_ranks, int blocks, cudaStream_t stream) {
  const bool vec = (p.block_elems * sizeof(T)) % 16 == 0;
  if (p.use_multimem) {
    if constexpr (dev::HasMultimem<T>::value) {
      if (!vec) return cudaErrorInvalidValue;
      return LaunchRsAgU<T, true, true, kMaxRanks>(p, emu, emu_ranks, blocks, stream);
    } else {
      return cudaErrorInvalidValue;
    }
  }
  if (!vec) return LaunchRsAgU<T, false, false, kMaxRanks>(p, emu, emu_ranks, blocks, stream);
  // Peer loads: compiled per world-size class (loads in flight per rank).
  switch (dev::RankClass(p.world_size)) {
    case 2: return LaunchRsAgU<T, false, true, 2>(p, emu, emu_ranks, blocks, stream);
    case 4: return LaunchRsAgU<T, false, true, 4>(p, emu, emu_ranks, blocks, stream);
    default: return LaunchRsAgU<T, false, true, kMaxRanks>(p, emu, emu_ranks, blocks, stream);
  }
}

cudaError_t LaunchRsAgKernel(const RsAgParams& p, const RsAgParams* emu, int emu_ranks, int blocks, cudaStream_t stream) {
  switch (static_cast<DType>(p.dtype)) {
    case DType::kFloat32: return LaunchRsAgTyped<float>(p, emu, emu_ranks, blocks, stream);
    case DType::kFloat16: return LaunchRsAgTyped<__half>(p, emu, emu_ranks, blocks, stream);
    case DType::kBFloat16: return LaunchRsAgTyped<__nv_bfloat16>(p, emu, emu_ranks, blocks, stream);
    case DType::kFloat64: return LaunchRsAgTyped<double>(p, emu, emu_ranks, blocks, stream);
    case DType::kInt32: return LaunchRsAgTyped<int>(p, emu, emu_ranks, blocks, stream);
    case DType::kInt64: return LaunchRsAgTyped<long long>(p, emu, emu_ranks, blocks, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace ibcomm
