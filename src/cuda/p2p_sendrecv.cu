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
// A message is moved by kP2pCtas CTAs.  CTA c owns a fixed part of every
// mailbox slot (bytes [c, c + 1) * slot_bytes / kP2pCtas), whatever the
// message, so its flags and credits cover exactly the bytes it touches and
// the CTAs never synchronise with each other; every CTA counts every piece,
// also those that leave its part empty.  Inside a CTA the work is
// warp-specialised like the op executor: a waiter thread runs ahead and waits
// for the next pieces' credits (sender) or flags (receiver), the data warps
// copy piece after piece, and a poster thread fences each piece's stores and
// publishes its flag (sender) or credit (receiver), so the NVLink round trip
// of a fence overlaps the next piece's data.
//
// The message length travels with the first piece (ControlPage::p2p_len), and
// a receive posted for another length reports "length mismatch" (the host
// transport's "Message length mismatch"), instead of reading stale bytes.
//
// The two kernels run on DIFFERENT GPUs.  (Both ends on one GPU are served by a
// plain device-to-device copy in the host code.)
#include "flags.cuh"
#include "kernels.h"
#include "vec_ops.cuh"
#include "warp_roles.cuh"

namespace ibcomm {
namespace dev {

constexpr int kP2pThreads = 512;

// Copies [0, bytes) with `nthr` threads; 16-byte vectors, eight in flight per
// thread, when both sides are 16-byte aligned, bytes otherwise.
__device__ __forceinline__ void CopyBytes(unsigned char* dst, const unsigned char* src, uint64_t bytes, bool strong_src,
                                          unsigned tid, unsigned nthr) {
  const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  uint64_t done = 0;
  if (aligned) {
    constexpr int kU = 8;
    const uint64_t nvec = bytes / 16;
    for (uint64_t i = tid; i < nvec; i += static_cast<uint64_t>(nthr) * kU) {
      uint4 v[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const uint64_t idx = i + static_cast<uint64_t>(u) * nthr;
        if (idx < nvec) v[u] = strong_src ? Ld16Strong(src + idx * 16) : Ld16(src + idx * 16);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const uint64_t idx = i + static_cast<uint64_t>(u) * nthr;
        if (idx < nvec) St16(dst + idx * 16, v[u]);
      }
    }
    done = nvec * 16;
  }
  for (uint64_t i = done + tid; i < bytes; i += nthr)
    dst[i] = strong_src ? *reinterpret_cast<const volatile unsigned char*>(src + i) : src[i];
}

__global__ void __launch_bounds__(kP2pThreads, 1) P2pKernel(const __grid_constant__ P2pParams p) {
  __shared__ RoleSync sync;
  if (threadIdx.x == 0) {
    sync.ready = 0;
    sync.done = 0;
    sync.stop = 0;
  }
  __syncthreads();
  const int cta = blockIdx.x;
  WaitCtx w;
  w.peers = &p.peers;
  w.status = p.status;
  w.doorbell = p.doorbell;
  w.seq = p.seq;
  w.timeout_ns = p.timeout_ns;
  w.rank = p.rank;
  w.world_size = p.world_size;
  w.channel = cta;
  ControlPage* mine = Ctl(p.peers, p.rank);
  ControlPage* theirs = Ctl(p.peers, p.peer);
  const uint64_t pieces = p.bytes == 0 ? 1 : (p.bytes + p.slot_bytes - 1) / p.slot_bytes;
  // This CTA's part of a slot: a whole number of 16-byte vectors.
  const uint64_t part = p.slot_bytes / gridDim.x / 16 * 16;
  const uint64_t part_b = part * cta;
  const uint64_t part_e = (cta + 1 == static_cast<int>(gridDim.x)) ? p.slot_bytes : part_b + part;
  const int warps = static_cast<int>(blockDim.x) / 32, data_warps = warps - 2;
  const int warp = static_cast<int>(threadIdx.x) / 32, lane = static_cast<int>(threadIdx.x) % 32;
  volatile int* const stop = &sync.stop;

  if (warp < data_warps) {
    const unsigned nthr = static_cast<unsigned>(data_warps) * 32u;
    for (uint64_t j = 0; j < pieces; ++j) {
      int go = 1;
      if (lane == 0) go = SpinShared(&sync.ready, static_cast<unsigned>(j) + 1u, &sync, p.timeout_ns) ? 1 : 0;
      go = __shfl_sync(0xffffffffu, go, 0);
      if (!go) break;
      const uint64_t k = p.first_piece + j;
      const uint64_t off = j * p.slot_bytes;
      const uint64_t len = (p.bytes - off < p.slot_bytes) ? p.bytes - off : p.slot_bytes;
      const uint64_t b = part_b < len ? part_b : len, e = part_e < len ? part_e : len;
      const uint64_t slot = k % p.slots;
      if (p.is_send) {
        unsigned char* box = p.peers.arena[p.peer] + p.mailbox_offset + (static_cast<uint64_t>(p.rank) * p.slots + slot) * p.slot_bytes;
        CopyBytes(box + b, static_cast<const unsigned char*>(p.src) + off + b, e - b, false, threadIdx.x, nthr);
      } else {
        const unsigned char* box = p.peers.arena[p.rank] + p.mailbox_offset + (static_cast<uint64_t>(p.peer) * p.slots + slot) * p.slot_bytes;
        CopyBytes(static_cast<unsigned char*>(p.dst) + off + b, box + b, e - b, true, threadIdx.x, nthr);
      }
      __syncwarp();
      if (lane == 0) AddReleaseShared(&sync.done, 1u);
    }
  } else if (warp == data_warps) {
    if (lane == 0) {
      for (uint64_t j = 0; j < pieces && *stop == 0; ++j) {
        const uint64_t k = p.first_piece + j;
        bool ok = true;
        if (p.is_send) {
          // The slot is free once the receiver consumed piece k - slots.
          if (k >= p.slots) ok = WaitGE(&mine->p2p_credit[cta][p.peer], k - p.slots + 1, w, kWaitP2p, p.peer, static_cast<int>(j));
        } else {
          ok = WaitGE(&mine->p2p_flag[cta][p.peer], k + 1, w, kWaitP2p, p.peer, static_cast<int>(j));
          // CTA 0 carries the length check (its copy of the length word is the
          // only one the sender's CTA 0 rewrites, and only after this CTA's credit).
          if (ok && j == 0 && cta == 0) {
            const uint64_t sent = LdRelaxedSys(&mine->p2p_len[p.peer][k % p.slots]);
            if (sent != p.bytes) {
              ReportFailure(w, kStatusLengthMismatch, kWaitP2p, p.peer, 0, p.bytes, sent);
              BroadcastAbort(w);
              ok = false;
            }
          }
        }
        if (!ok) {
          *stop = 1;
          break;
        }
        StReleaseShared(&sync.ready, static_cast<unsigned>(j) + 1u);
      }
    }
  } else {
    if (lane == 0) {
      for (uint64_t j = 0; j < pieces; ++j) {
        if (!SpinShared(&sync.done, static_cast<unsigned>(data_warps) * (static_cast<unsigned>(j) + 1u), &sync, p.timeout_ns)) break;
        const uint64_t k = p.first_piece + j;
        if (p.is_send) {
          if (j == 0 && cta == 0) StRelaxedSys(&theirs->p2p_len[p.rank][k % p.slots], p.bytes);
          FenceSys();
          StRelaxedSys(&theirs->p2p_flag[cta][p.rank], k + 1);
        } else {
          StRelaxedSys(&theirs->p2p_credit[cta][p.rank], k + 1);
        }
      }
    }
  }
}

}  // namespace dev

cudaError_t LaunchP2pKernel(const P2pParams& p, cudaStream_t stream) {
  dev::P2pKernel<<<kP2pCtas, dev::kP2pThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace ibcomm
