// Two-shot allreduce for buffers the peers cannot map (ordinary device
// memory), with the staging copies overlapped with the collective itself.
//
// The message moves through the arena's pool in windows.  The pool holds two
// input and two output windows; every rank runs `pairs` reducer CTAs and
// `pairs` mover CTAs in ONE cooperative launch:
//
//   mover b    copies window w+1 of sendbuf into the input area and window
//              w-1 of the output area into recvbuf, while
//   reducer b  reduces window w (multimem.ld_reduce + multimem.st in the
//              NVSwitch, or peer loads + peer stores) and runs the one
//              cross-rank barrier per window.
//
// A mover and the reducer of the same index hand windows to each other through
// three local counters; across ranks, CTA b only ever synchronises with CTA b,
// because mover b copies exactly the parts that reducer b of every rank reads
// and writes.  The same kernel body without this overlap is nvls_kernel.cu
// (used for small messages and for buffers in symmetric memory).  The
// reference stages every chunk through pinned host memory with separate copy
// and reduce launches (ibcomm/allreduce_cuda_impl.h:129-135, 503-516).
#include <cooperative_groups.h>

#include "ibcomm/communicator.h"
#include "twoshot_common.cuh"

namespace ibcomm {
namespace dev {

// Element-wise fallback of CopyVectors for user buffers that are only
// element-aligned; [b, e) are vector indices.
template <typename T>
__device__ __forceinline__ void CopyElems(T* dst, const T* src, uint64_t b, uint64_t e, bool strong) {
  constexpr int kVecElems = 16 / static_cast<int>(sizeof(T));
  for (uint64_t i = b * kVecElems + threadIdx.x; i < e * kVecElems; i += blockDim.x) dst[i] = strong ? LdScalarStrong<T>(src + i) : src[i];
}

template <typename T, bool kMultimem>
__device__ void StagedBody(const NvlsParams& p, uint64_t seq, int& s_stop) {
  using A = typename Acc<T>::type;
  constexpr int kVecElems = 16 / static_cast<int>(sizeof(T));
  const int pairs = static_cast<int>(gridDim.x / 2);
  const bool is_mover = static_cast<int>(blockIdx.x) >= pairs;
  const int b = static_cast<int>(blockIdx.x) % pairs;
  WaitCtx w;
  w.peers = &p.peers;
  w.status = p.status;
  w.doorbell = p.doorbell;
  w.seq = seq;
  w.timeout_ns = p.timeout_ns;
  w.rank = p.rank;
  w.world_size = p.world_size;
  w.channel = b;
  ControlPage* const me = Ctl(p.peers, p.rank);
  const uint64_t base = seq << 32;
  const T* sendbuf = static_cast<const T*>(p.sendbuf);
  T* recvbuf = static_cast<T*>(p.recvbuf);
  const uint64_t nwin = (p.len_elements + p.window_elems - 1) / p.window_elems;
  const bool do_scale = p.scale != 1.0;

  auto win_len = [&](uint64_t wi) -> uint64_t {
    const uint64_t w0 = wi * p.window_elems;
    return p.len_elements - w0 < p.window_elems ? p.len_elements - w0 : p.window_elems;
  };
  // Local wait of one CTA on a counter its partner CTA publishes.
  auto wait_local = [&](const uint64_t* flag, uint64_t count, int what) -> bool {
    if (threadIdx.x == 0 && !WaitGE(flag, base | count, w, kWaitData, p.rank, what)) s_stop = 1;
    __syncthreads();
    return s_stop == 0;
  };
  auto publish = [&](uint64_t* flag, uint64_t count) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();  // the window is read by the peers (or the switch) next
      StRelaxedSys(flag, base | count);
    }
  };

  if (is_mover) {
    for (uint64_t wi = 0; wi <= nwin; ++wi) {
      if (wi < nwin) {
        // The input window is free once window wi-2 has been reduced everywhere.
        if (wi >= 2 && !wait_local(&me->stage_out_ready[b], wi - 1, 100)) return;
        const uint64_t w0 = wi * p.window_elems, wn = win_len(wi), nvec = wn / kVecElems;
        unsigned char* in_win = p.local_in + (wi & 1) * p.window_stride;
        const uint4* src = reinterpret_cast<const uint4*>(sendbuf + w0);
        const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
        for (int s = 0; s < p.world_size; ++s) {
          uint64_t sb, se, vb, ve;
          SubRange(0, nvec, s, p.world_size, &sb, &se);
          SubRange(sb, se, b, pairs, &vb, &ve);
          if (aligned) CopyVectors<false>(reinterpret_cast<uint4*>(in_win), src, vb, ve);
          else CopyElems<T>(reinterpret_cast<T*>(in_win), sendbuf + w0, vb, ve, false);
        }
        if (b == 0) {
          T* dt = reinterpret_cast<T*>(in_win);
          for (uint64_t i = nvec * kVecElems + threadIdx.x; i < wn; i += blockDim.x) dt[i] = sendbuf[w0 + i];
        }
        publish(&me->stage_in_ready[b], wi + 1);
      }
      if (wi >= 1) {
        const uint64_t wo = wi - 1;
        if (!wait_local(&me->stage_out_ready[b], wo + 1, 101)) return;
        const uint64_t w0 = wo * p.window_elems, wn = win_len(wo), nvec = wn / kVecElems;
        const unsigned char* out_win = p.local_out + (wo & 1) * p.window_stride;
        uint4* dst = reinterpret_cast<uint4*>(recvbuf + w0);
        const bool aligned = (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
        for (int s = 0; s < p.world_size; ++s) {
          uint64_t sb, se, vb, ve;
          SubRange(0, nvec, s, p.world_size, &sb, &se);
          SubRange(sb, se, b, pairs, &vb, &ve);
          if (aligned) CopyVectors<true>(dst, reinterpret_cast<const uint4*>(out_win), vb, ve);
          else CopyElems<T>(recvbuf + w0, reinterpret_cast<const T*>(out_win), vb, ve, true);
        }
        publish(&me->stage_out_consumed[b], wo + 1);
      }
    }
    return;
  }

  // ---- reducer ----
  uint32_t phase = 0;
  if (!wait_local(&me->stage_in_ready[b], 1, 102)) return;
  if (!CrossRankBarrier(p, w, b, ++phase, &s_stop)) return;
  for (uint64_t wi = 0; wi < nwin; ++wi) {
    const uint64_t w0 = wi * p.window_elems, wn = win_len(wi), nvec = wn / kVecElems, tail0 = nvec * kVecElems;
    const uint64_t off = (wi & 1) * p.window_stride;
    {
      uint64_t sb, se, vb, ve;
      SubRange(0, nvec, p.rank, p.world_size, &sb, &se);
      SubRange(sb, se, b, pairs, &vb, &ve);
      if (kMultimem) {
        const unsigned char* mi = p.mc_in + off;
        unsigned char* mo = p.mc_out + off;
        constexpr int U = 4;
        for (uint64_t i = vb + threadIdx.x; i < ve; i += static_cast<uint64_t>(blockDim.x) * U) {
          uint4 v[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint64_t idx = i + static_cast<uint64_t>(u) * blockDim.x;
            if (idx < ve) v[u] = Multimem<T>::LdReduce(mi + idx * 16);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint64_t idx = i + static_cast<uint64_t>(u) * blockDim.x;
            if (idx < ve) {
              if (do_scale) {
                A acc[kVecElems];
                VecIO<T>::Load(v[u], acc);
#pragma unroll
                for (int k = 0; k < kVecElems; ++k) acc[k] = ScaleAcc<A>(acc[k], p.scale);
                v[u] = VecIO<T>::Store(acc);
              }
              Multimem<T>::St(mo + idx * 16, v[u]);
            }
          }
        }
      } else {
        const int ws = p.world_size;
        for (uint64_t i = vb + threadIdx.x; i < ve; i += blockDim.x) {
          uint4 v[kMaxRanks];
#pragma unroll
          for (int q = 0; q < kMaxRanks; ++q)
            if (q < ws) v[q] = Ld16Strong(p.peer_in[q] + off + i * 16);
          A acc[kVecElems];
          VecIO<T>::Load(v[0], acc);
#pragma unroll
          for (int q = 1; q < kMaxRanks; ++q)
            if (q < ws) VecIO<T>::Add(v[q], acc);
          if (do_scale) {
#pragma unroll
            for (int k = 0; k < kVecElems; ++k) acc[k] = ScaleAcc<A>(acc[k], p.scale);
          }
          const uint4 r = VecIO<T>::Store(acc);
#pragma unroll
          for (int q = 0; q < kMaxRanks; ++q)
            if (q < ws) St16(p.peer_out[q] + off + i * 16, r);
        }
      }
    }
    // Ragged end (< 16 bytes, last window only): summed from the peers'
    // input windows in rank order and written straight to recvbuf.
    if (b == 0 && tail0 + threadIdx.x < wn) {
      const uint64_t i = tail0 + threadIdx.x;
      A acc = A(0);
      for (int q = 0; q < p.world_size; ++q) acc += ToAcc<A, T>(LdScalarStrong<T>(reinterpret_cast<const T*>(p.peer_in[q] + off) + i));
      if (do_scale) acc = ScaleAcc<A>(acc, p.scale);
      recvbuf[w0 + i] = FromAcc<T, A>(acc);
    }
    // One barrier per window: "my stores of window wi are done" and "my input
    // of window wi+1 is in place and my output window wi+1 is free".
    if (wi + 1 < nwin) {
      if (!wait_local(&me->stage_in_ready[b], wi + 2, 103)) return;
      if (wi >= 1 && !wait_local(&me->stage_out_consumed[b], wi, 104)) return;
    }
    if (!CrossRankBarrier(p, w, b, ++phase, &s_stop)) return;
    publish(&me->stage_out_ready[b], wi + 1);
  }
}

template <typename T, bool kMultimem>
__global__ void __launch_bounds__(kNvlsThreads, 1)
StagedTwoShotKernel(const __grid_constant__ NvlsParams p0, const NvlsParams* __restrict__ emu) {
  __shared__ NvlsParams p;
  __shared__ int s_stop;
  __shared__ uint64_t s_seq;
  {
    const uint32_t* src = (emu != nullptr) ? reinterpret_cast<const uint32_t*>(emu + blockIdx.y) : reinterpret_cast<const uint32_t*>(&p0);
    for (unsigned i = threadIdx.x; i < sizeof(NvlsParams) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(&p)[i] = src[i];
    if (threadIdx.x == 0) s_stop = 0;
  }
  __syncthreads();
  const uint64_t seq = BeginCollective(p.peers, p.rank, &s_seq);
  StagedBody<T, kMultimem>(p, seq, s_stop);
  EndCollective(p.peers, p.rank, seq, gridDim.x);
}

}  // namespace dev

template <typename T, bool kMultimem>
static cudaError_t LaunchStagedU(const NvlsParams& p, const NvlsParams* emu, int emu_ranks, int pairs, cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>(2 * pairs), static_cast<unsigned>(emu != nullptr ? emu_ranks : 1));
  // Movers and reducers of one rank wait on each other: the launch must be
  // cooperative so that all of them are resident (or the launch is refused).
  void* args[] = {const_cast<NvlsParams*>(&p), &emu};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(dev::StagedTwoShotKernel<T, kMultimem>), grid, dim3(dev::kNvlsThreads), args, 0, stream);
}

template <typename T>
static cudaError_t LaunchStagedTyped(const NvlsParams& p, const NvlsParams* emu, int emu_ranks, int pairs, cudaStream_t stream) {
  if (!p.use_multimem) return LaunchStagedU<T, false>(p, emu, emu_ranks, pairs, stream);
  if constexpr (dev::HasMultimem<T>::value) {
    return LaunchStagedU<T, true>(p, emu, emu_ranks, pairs, stream);
  } else {
    return cudaErrorInvalidValue;
  }
}

cudaError_t LaunchStagedTwoShotKernel(const NvlsParams& p, const NvlsParams* emu, int emu_ranks, int pairs, cudaStream_t stream) {
  switch (static_cast<DType>(p.dtype)) {
    case DType::kFloat32: return LaunchStagedTyped<float>(p, emu, emu_ranks, pairs, stream);
    case DType::kFloat16: return LaunchStagedTyped<__half>(p, emu, emu_ranks, pairs, stream);
    case DType::kBFloat16: return LaunchStagedTyped<__nv_bfloat16>(p, emu, emu_ranks, pairs, stream);
    case DType::kFloat64: return LaunchStagedTyped<double>(p, emu, emu_ranks, pairs, stream);
    case DType::kInt32: return LaunchStagedTyped<int>(p, emu, emu_ranks, pairs, stream);
    case DType::kInt64: return LaunchStagedTyped<long long>(p, emu, emu_ranks, pairs, stream);
  }
  return cudaErrorInvalidValue;
}

int StagedTwoShotMaxPairs(int device) {
  int per_sm = 0, sms = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dev::StagedTwoShotKernel<float, true>, dev::kNvlsThreads, 0) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  return per_sm * sms / 2;
}

}  // namespace ibcomm
