// Hybrid two-shot allreduce for buffers in symmetric memory: one part of the
// message is reduced in the NVSwitch (multimem.ld_reduce / multimem.st), the
// rest by the direct algorithm (peer loads summed in rank order, peer stores),
// at the same time, in ONE kernel: CTAs [0, nvls_ctas) run the switch part,
// the other CTAs the direct part.
//
// Why: per direction and GPU the switch path moves 1 + 1/ws of its bytes and
// the direct path 2 (ws-1)/ws of its bytes, but the switch path has measured
// at 0.67 of the link roofline (it is bound by the reduction in the switch,
// not by the links), so the links have room for direct traffic next to it.
// With a fraction f in the switch the time is about max(f * t_switch,
// (1.125 f + 1.75 (1 - f)) * S / link bandwidth) at 8 ranks.
//
// Opt-in (IBCOMM_NVLS_HYBRID = percentage of the message that goes direct):
// the split has to be tuned on the machine.  Zero-copy only; the element
// types of the switch path (fp32, fp16, bf16).  The reference has no
// counterpart (no intra-node path, README.md:66).
#include <cooperative_groups.h>

#include "flags.cuh"
#include "ibcomm/communicator.h"
#include "kernels.h"
#include "twoshot_common.cuh"
#include "vec_ops.cuh"

namespace ibcomm {
namespace dev {

template <typename T, int kR>
__global__ void __launch_bounds__(kNvlsThreads, 1) HybridKernel(const __grid_constant__ HybridParams h0) {
  using A = typename Acc<T>::type;
  constexpr int kVecElems = 16 / static_cast<int>(sizeof(T));
  __shared__ HybridParams h;
  __shared__ int s_stop;
  __shared__ uint64_t s_seq;
  for (unsigned i = threadIdx.x; i < sizeof(HybridParams) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(&h)[i] = reinterpret_cast<const uint32_t*>(&h0)[i];
  if (threadIdx.x == 0) s_stop = 0;
  __syncthreads();
  const NvlsParams& p = h.base;
  const uint64_t seq = BeginCollective(p.peers, p.rank, &s_seq);

  const int bar_index = blockIdx.x;  // one barrier slot per CTA of the grid, whatever its role
  const bool switch_role = static_cast<int>(blockIdx.x) < h.nvls_ctas;
  const int cta = switch_role ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x) - h.nvls_ctas;
  const int ncta = switch_role ? h.nvls_ctas : static_cast<int>(gridDim.x) - h.nvls_ctas;
  WaitCtx w;
  w.peers = &p.peers;
  w.status = p.status;
  w.doorbell = p.doorbell;
  w.seq = seq;
  w.timeout_ns = p.timeout_ns;
  w.rank = p.rank;
  w.world_size = p.world_size;
  w.channel = bar_index;

  const uint64_t nvec = p.len_elements / kVecElems, tail0 = nvec * kVecElems;
  // Vectors [0, split) go through the switch, [split, nvec) direct; inside a
  // part, rank r owns shard r and CTA `cta` of the role part `cta` of it.
  const uint64_t split = h.split_vec < nvec ? h.split_vec : nvec;
  uint64_t sb, se, b, e;
  SubRange(switch_role ? 0 : split, switch_role ? split : nvec, p.rank, p.world_size, &sb, &se);
  SubRange(sb, se, cta, ncta, &b, &e);
  const bool do_scale = p.scale != 1.0;

  // Every rank's input is ready, every rank's output may be written.
  bool alive = CrossRankBarrier(p.peers, w, bar_index, 1, &s_stop);
  A tail_acc = A(0);
  const bool has_tail = alive && !switch_role && cta == 0 && tail0 + threadIdx.x < p.len_elements;
  if (alive) {
    if (switch_role) {
      constexpr int kU = 4;
      for (uint64_t i = b + threadIdx.x; i < e; i += static_cast<uint64_t>(blockDim.x) * kU) {
        uint4 v[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint64_t idx = i + static_cast<uint64_t>(u) * blockDim.x;
          if (idx < e) v[u] = Multimem<T>::LdReduce(p.mc_in + idx * 16);
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint64_t idx = i + static_cast<uint64_t>(u) * blockDim.x;
          if (idx < e) {
            if (do_scale) {
              A acc[kVecElems];
              VecIO<T>::Load(v[u], acc);
#pragma unroll
              for (int k = 0; k < kVecElems; ++k) acc[k] = ScaleAcc<A>(acc[k], p.scale);
              v[u] = VecIO<T>::Store(acc);
            }
            Multimem<T>::St(p.mc_out + idx * 16, v[u]);
          }
        }
      }
    } else {
      const int ws = p.world_size;
      unsigned char* const* outs = p.peer_out;
      PeerReduce<T, kR>(p.peer_in, ws, 0, b, e, do_scale, p.scale, [&](uint64_t idx, uint4 r) {
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q)
          if (q < ws) St16(outs[q] + idx * 16, r);
      });
    }
    // The ragged end (< 16 bytes): summed by every rank itself, written after
    // the barrier (in place, the peers are still reading this rank's input).
    if (has_tail) {
      const uint64_t i = tail0 + threadIdx.x;
      for (int q = 0; q < p.world_size; ++q) tail_acc += ToAcc<A, T>(LdScalarStrong<T>(reinterpret_cast<const T*>(p.peer_in[q]) + i));
      if (do_scale) tail_acc = ScaleAcc<A>(tail_acc, p.scale);
    }
    alive = CrossRankBarrier(p.peers, w, bar_index, 2, &s_stop);
    if (alive && has_tail) reinterpret_cast<T*>(p.local_out)[tail0 + threadIdx.x] = FromAcc<T, A>(tail_acc);
  }
  EndCollective(p.peers, p.rank, seq, gridDim.x);
}

}  // namespace dev

template <typename T>
static cudaError_t LaunchHybridTyped(const HybridParams& h, int blocks, cudaStream_t stream) {
  switch (dev::RankClass(h.base.world_size)) {
    case 2: dev::HybridKernel<T, 2><<<blocks, dev::kNvlsThreads, 0, stream>>>(h); break;
    case 4: dev::HybridKernel<T, 4><<<blocks, dev::kNvlsThreads, 0, stream>>>(h); break;
    default: dev::HybridKernel<T, kMaxRanks><<<blocks, dev::kNvlsThreads, 0, stream>>>(h); break;
  }
  return cudaGetLastError();
}

cudaError_t LaunchHybridKernel(const HybridParams& h, int blocks, cudaStream_t stream) {
  if (h.nvls_ctas < 1 || h.nvls_ctas >= blocks || !h.base.use_multimem || h.base.stage_in || h.base.stage_out)
    return cudaErrorInvalidValue;
  switch (static_cast<DType>(h.base.dtype)) {
    case DType::kFloat32: return LaunchHybridTyped<float>(h, blocks, stream);
    case DType::kFloat16: return LaunchHybridTyped<__half>(h, blocks, stream);
    case DType::kBFloat16: return LaunchHybridTyped<__nv_bfloat16>(h, blocks, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace ibcomm
