// Two-sided device messaging (Send/Recv of device buffers) without the host
// in the data path.  The sender's kernel stores the payload piece by piece
// into its mailbox inside the RECEIVER's arena over NVLink and publishes a
// piece counter; the receiver's kernel waits for the counter, copies the piece
// into the user buffer and returns a credit so the slot can be reused.
// Counters are cumulative per ordered rank pair, so messages are matched in
// FIFO order without tags, like the reference's queue pairs
// (ibcomm/ibverbs_communicator.cpp:371-527), which bounce device data through
// pinned host memory instead.
//
// The two kernels run on DIFFERENT GPUs.  (Both ends on one GPU are served by a
// plain device-to-device copy in the host code.)
#include "flags.cuh"
#include "kernels.h"
#include "vec_ops.cuh"

namespace ibcomm {
namespace dev {

constexpr int kP2pThreads = 1024;

__device__ __forceinline__ void CopyBytes(unsigned char* dst, const unsigned char* src, uint64_t bytes, bool strong_src) {
  const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  uint64_t done = 0;
  if (aligned) {
    const uint64_t nvec = bytes / 16;
    for (uint64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 v = strong_src ? Ld16Strong(src + i * 16) : Ld16(src + i * 16);
      St16(dst + i * 16, v);
    }
    done = nvec * 16;
  }
  for (uint64_t i = done + threadIdx.x; i < bytes; i += blockDim.x)
    dst[i] = strong_src ? *reinterpret_cast<const volatile unsigned char*>(src + i) : src[i];
}

__global__ void __launch_bounds__(kP2pThreads, 1) P2pKernel(const __grid_constant__ P2pParams p) {
  __shared__ int s_stop;
  if (threadIdx.x == 0) s_stop = 0;
  __syncthreads();
  WaitCtx w;
  w.peers = &p.peers;
  w.status = p.status;
  w.doorbell = p.doorbell;
  w.seq = p.seq;
  w.timeout_ns = p.timeout_ns;
  w.rank = p.rank;
  w.world_size = p.world_size;
  w.channel = 0;
  ControlPage* mine = Ctl(p.peers, p.rank);
  ControlPage* theirs = Ctl(p.peers, p.peer);
  const uint64_t pieces = (p.bytes + p.slot_bytes - 1) / p.slot_bytes;
  for (uint64_t j = 0; j < pieces; ++j) {
    const uint64_t k = p.first_piece + j;  // cumulative piece number of this pair
    const uint64_t off = j * p.slot_bytes;
    const uint64_t len = (p.bytes - off < p.slot_bytes) ? p.bytes - off : p.slot_bytes;
    const uint64_t slot = k % p.slots;
    if (p.is_send) {
      // The slot is free once the receiver consumed piece k - slots.
      if (threadIdx.x == 0 && k >= p.slots) {
        if (!WaitGE(&mine->p2p_credit[p.peer], k - p.slots + 1, w, kWaitP2p, p.peer, static_cast<int>(j))) s_stop = 1;
      }
      __syncthreads();
      if (s_stop) return;
      unsigned char* dst = p.peers.arena[p.peer] + p.mailbox_offset +
                           (static_cast<uint64_t>(p.rank) * p.slots + slot) * p.slot_bytes;
      CopyBytes(dst, static_cast<const unsigned char*>(p.src) + off, len, false);
      __syncthreads();
      if (threadIdx.x == 0) {
        FenceSys();
        StRelaxedSys(&theirs->p2p_flag[p.rank], k + 1);
      }
    } else {
      if (threadIdx.x == 0) {
        if (!WaitGE(&mine->p2p_flag[p.peer], k + 1, w, kWaitP2p, p.peer, static_cast<int>(j))) s_stop = 1;
      }
      __syncthreads();
      if (s_stop) return;
      const unsigned char* src = p.peers.arena[p.rank] + p.mailbox_offset +
                                 (static_cast<uint64_t>(p.peer) * p.slots + slot) * p.slot_bytes;
      CopyBytes(static_cast<unsigned char*>(p.dst) + off, src, len, true);
      __syncthreads();
      if (threadIdx.x == 0) StRelaxedSys(&theirs->p2p_credit[p.rank], k + 1);
    }
  }
}

}  // namespace dev

cudaError_t LaunchP2pKernel(const P2pParams& p, cudaStream_t stream) {
  dev::P2pKernel<<<1, dev::kP2pThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace ibcomm
