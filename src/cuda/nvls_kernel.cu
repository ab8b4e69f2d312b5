// Two-shot allreduce in the NVSwitch (NVLS): every rank owns 1/world_size of
// the message; for its shard it issues `multimem.ld_reduce` (the switch reads
// the same address on every GPU and returns the sum), applies the scale, and
// `multimem.st` (the switch writes the result to every GPU).  Per GPU that is
// about S*(1+1/ws) bytes in each NVLink direction instead of the ring's
// 2*S*(ws-1)/ws.  The reference has no counterpart (it has no intra-node
// path, README.md:66).
//
// Buffers must be bound to a multicast object.  Buffers inside a symmetric
// allocation are used in place; others are staged through the arena's pool
// window by window inside this same kernel (copy in -> barrier -> reduce ->
// barrier -> copy out), with the copies of CTA b on every rank covering
// exactly what CTA b of the other ranks reduces, so the barriers are per CTA.
//
// The same kernel without multimem is the "direct" two-shot algorithm: a rank
// loads its shard from every peer's buffer over NVLink (plain 16-byte peer
// loads, summed in rank order), scales it and stores it into every peer's
// output buffer.  It needs no multicast (and can therefore be emulated with
// several ranks on one GPU), moves 2*S*(ws-1)/ws per direction like the ring
// but in two synchronisation steps instead of 2*(ws-1), and supports every
// element type.
#include <cooperative_groups.h>

#include <cstdlib>

#include "flags.cuh"
#include "ibcomm/communicator.h"
#include "ibcomm/tunables.h"
#include "kernels.h"
#include "twoshot_common.cuh"
#include "vec_ops.cuh"

namespace ibcomm {
namespace dev {

// Body of the two-shot kernel for one CTA; returns early when a barrier gave up.
template <typename T, int U, bool kMultimem, int kR>
__device__ void TwoShotBody(const NvlsParams& p, uint64_t seq, int& s_stop) {
  using A = typename Acc<T>::type;
  constexpr int kVecElems = 16 / static_cast<int>(sizeof(T));
  const int cta = blockIdx.x, ncta = gridDim.x;
  WaitCtx w;
  w.peers = &p.peers;
  w.status = p.status;
  w.doorbell = p.doorbell;
  w.seq = seq;
  w.timeout_ns = p.timeout_ns;
  w.rank = p.rank;
  w.world_size = p.world_size;
  w.channel = cta;

  const T* sendbuf = static_cast<const T*>(p.sendbuf);
  T* recvbuf = static_cast<T*>(p.recvbuf);
  const bool do_scale = p.scale != 1.0;
  uint32_t phase = 0;
  const uint64_t full_nvec = (p.window_elems + kVecElems - 1) / kVecElems;

  for (uint64_t w0 = 0; w0 < p.len_elements; w0 += p.window_elems) {
    const uint64_t wn = (p.len_elements - w0 < p.window_elems) ? p.len_elements - w0 : p.window_elems;
    const uint64_t nvec = wn / kVecElems;  // whole 16-byte vectors in the window
    const uint64_t tail0 = nvec * kVecElems;
    const uint64_t win_bytes_off = p.stage_in ? 0 : w0 * sizeof(T);
    const uint64_t wout_bytes_off = p.stage_out ? 0 : w0 * sizeof(T);

    // (1) stage in: CTA `cta` copies part `cta` of every shard.
    if (p.stage_in) {
      const uint4* src = reinterpret_cast<const uint4*>(sendbuf + w0);
      uint4* dst = reinterpret_cast<uint4*>(p.local_in);
      const bool src_aligned = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
      for (int s = 0; s < p.world_size; ++s) {
        uint64_t b, e;
        WindowPart(full_nvec, nvec, s, p.world_size, cta, ncta, &b, &e);
        if (src_aligned) {
          CopyVectors<false>(dst, src, b, e);
        } else {
          // A user buffer that is only element-aligned: element by element.
          T* dt = reinterpret_cast<T*>(p.local_in);
          for (uint64_t i = b * kVecElems + threadIdx.x; i < e * kVecElems; i += blockDim.x) dt[i] = sendbuf[w0 + i];
        }
      }
      if (cta == 0) {
        T* dt = reinterpret_cast<T*>(p.local_in + p.tail_in_off);
        for (uint64_t i = tail0 + threadIdx.x; i < wn; i += blockDim.x) dt[i - tail0] = sendbuf[w0 + i];
      }
    }
    if (!CrossRankBarrier(p.peers, w, cta, ++phase, &s_stop)) return;

    // (2) reduce my shard in the switch and broadcast it.
    {
      uint64_t b, e;
      WindowPart(full_nvec, nvec, p.rank, p.world_size, cta, ncta, &b, &e);
      const unsigned char* mi = p.mc_in + win_bytes_off;
      unsigned char* mo = p.mc_out + wout_bytes_off;
      if (kMultimem) {
        for (uint64_t i = b + threadIdx.x; i < e; i += static_cast<uint64_t>(blockDim.x) * U) {
          uint4 v[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint64_t idx = i + static_cast<uint64_t>(u) * blockDim.x;
            if (idx < e) v[u] = Multimem<T>::LdReduce(mi + idx * 16);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint64_t idx = i + static_cast<uint64_t>(u) * blockDim.x;
            if (idx < e) {
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
        // Direct variant: 16-byte loads from every peer, several in flight per
        // thread; the sum runs in rank order, so whoever reduces a shard, the
        // bits are the same.  The result goes to every rank's output window.
        const int ws = p.world_size;
        unsigned char* const* outs = p.peer_out;
        PeerReduce<T, kR>(p.peer_in, ws, win_bytes_off, b, e, do_scale, p.scale, [&](uint64_t idx, uint4 r) {
#pragma unroll
          for (int q = 0; q < kMaxRanks; ++q)
            if (q < ws) St16(outs[q] + wout_bytes_off + idx * 16, r);
        });
      }
    }
    // Ragged end (< 16 bytes): every rank sums it itself from the peers'
    // windows, in rank order.  The value is written after the barrier, since
    // with in-place buffers the peers are still reading this rank's input.
    A tail_acc = A(0);
    const bool has_tail = cta == 0 && tail0 + threadIdx.x < wn;
    if (has_tail) {
      const uint64_t i = tail0 + threadIdx.x;
      for (int q = 0; q < p.world_size; ++q) {
        const T* src = p.stage_in ? reinterpret_cast<const T*>(p.peer_in[q] + p.tail_in_off) + (i - tail0)
                                  : reinterpret_cast<const T*>(p.peer_in[q] + win_bytes_off) + i;
        tail_acc += ToAcc<A, T>(LdScalarStrong<T>(src));
      }
      if (do_scale) tail_acc = ScaleAcc<A>(tail_acc, p.scale);
    }
    if (!CrossRankBarrier(p.peers, w, cta, ++phase, &s_stop)) return;
    if (has_tail) {
      const uint64_t i = tail0 + threadIdx.x;
      if (p.stage_out) recvbuf[w0 + i] = FromAcc<T, A>(tail_acc);
      else reinterpret_cast<T*>(p.local_out + wout_bytes_off)[i] = FromAcc<T, A>(tail_acc);
    }

    // (3) stage out.
    if (p.stage_out) {
      const uint4* src = reinterpret_cast<const uint4*>(p.local_out);
      uint4* dst = reinterpret_cast<uint4*>(recvbuf + w0);
      const bool dst_aligned = (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
      for (int s = 0; s < p.world_size; ++s) {
        uint64_t b, e;
        WindowPart(full_nvec, nvec, s, p.world_size, cta, ncta, &b, &e);
        if (dst_aligned) {
          CopyVectors<true>(dst, src, b, e);
        } else {
          const T* st = reinterpret_cast<const T*>(p.local_out);
          for (uint64_t i = b * kVecElems + threadIdx.x; i < e * kVecElems; i += blockDim.x) recvbuf[w0 + i] = LdScalarStrong<T>(st + i);
        }
      }
    }
  }
}

template <typename T, int U, bool kMultimem, int kR>
__global__ void __launch_bounds__(kNvlsThreads, 1) NvlsKernel(const __grid_constant__ NvlsParams p0, const NvlsParams* __restrict__ emu) {
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
  TwoShotBody<T, U, kMultimem, kR>(p, seq, s_stop);
  EndCollective(p.peers, p.rank, seq, gridDim.x);
}

}  // namespace dev

template <typename T, int U, bool kMultimem, int kR>
static cudaError_t LaunchNvlsU(const NvlsParams& p, const NvlsParams* emu, int emu_ranks, int blocks, int threads, cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(emu != nullptr ? emu_ranks : 1));
  if (emu != nullptr) {
    void* args[] = {const_cast<NvlsParams*>(&p), &emu};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(dev::NvlsKernel<T, U, kMultimem, kR>), grid, dim3(threads), args, 0, stream);
  }
  dev::NvlsKernel<T, U, kMultimem, kR><<<grid, threads, 0, stream>>>(p, nullptr);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t LaunchNvlsTyped(const NvlsParams& p, const NvlsParams* emu, int emu_ranks, int blocks, cudaStream_t stream) {
  // Tuning knobs for experiments: loads in flight per thread and CTA size.
  const int unroll = Tunable("IBCOMM_NVLS_UNROLL", 4);
  const int threads_env = Tunable("IBCOMM_NVLS_THREADS", dev::kNvlsThreads);
  const int threads = (threads_env >= 64 && threads_env <= dev::kNvlsThreads && threads_env % 32 == 0) ? threads_env : dev::kNvlsThreads;
  if (!p.use_multimem) {
    // Direct variant: compiled per world-size class (loads in flight per rank).
    switch (dev::RankClass(p.world_size)) {
      case 2: return LaunchNvlsU<T, 4, false, 2>(p, emu, emu_ranks, blocks, threads, stream);
      case 4: return LaunchNvlsU<T, 4, false, 4>(p, emu, emu_ranks, blocks, threads, stream);
      default: return LaunchNvlsU<T, 4, false, kMaxRanks>(p, emu, emu_ranks, blocks, threads, stream);
    }
  }
  if constexpr (dev::HasMultimem<T>::value) {
    if (unroll == 8) return LaunchNvlsU<T, 8, true, kMaxRanks>(p, emu, emu_ranks, blocks, threads, stream);
    if (unroll == 2) return LaunchNvlsU<T, 2, true, kMaxRanks>(p, emu, emu_ranks, blocks, threads, stream);
    return LaunchNvlsU<T, 4, true, kMaxRanks>(p, emu, emu_ranks, blocks, threads, stream);
  } else {
    return cudaErrorInvalidValue;
  }
}

int TwoShotKernelMaxCoResidentBlocks(int device) {
  int per_sm = 0, sms = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dev::NvlsKernel<float, 4, false, kMaxRanks>, dev::kNvlsThreads, 0) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  return per_sm * sms;
}

cudaError_t LaunchNvlsKernel(const NvlsParams& p, const NvlsParams* emu, int emu_ranks, int blocks, cudaStream_t stream) {
  const DType t = static_cast<DType>(p.dtype);
  if (p.use_multimem && !(t == DType::kFloat32 || t == DType::kFloat16 || t == DType::kBFloat16)) return cudaErrorInvalidValue;
  switch (t) {
    case DType::kFloat32: return LaunchNvlsTyped<float>(p, emu, emu_ranks, blocks, stream);
    case DType::kFloat16: return LaunchNvlsTyped<__half>(p, emu, emu_ranks, blocks, stream);
    case DType::kBFloat16: return LaunchNvlsTyped<__nv_bfloat16>(p, emu, emu_ranks, blocks, stream);
    case DType::kFloat64: return LaunchNvlsTyped<double>(p, emu, emu_ranks, blocks, stream);
    case DType::kInt32: return LaunchNvlsTyped<int>(p, emu, emu_ranks, blocks, stream);
    case DType::kInt64: return LaunchNvlsTyped<long long>(p, emu, emu_ranks, blocks, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace ibcomm
