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
// A message is moved by a fixed number of CTAs (96 by default: one SM sustains
// roughly 10 GB/s of stores to a peer, measured on B200, so a few CTAs cannot
// fill a link).  CTA c owns a fixed part of every mailbox slot (bytes
// [c, c + 1) * slot_bytes / CTAs), whatever the message, so its flags and credits cover exactly the bytes it touches and
// the CTAs never synchronise with each other; every CTA counts every piece,
// also those that leave its part empty.  Inside a CTA the work is
// warp-specialised like the op executor: a waiter thread runs ahead and waits
// for the next pieces' credits (sender) or flags (receiver), the data warps
// copy piece after piece, and a poster thread fences each piece's stores and
// publishes its flag (sender) or credit (receiver).  Before a piece can be
// published its stores must be acknowledged over NVLink (microseconds under
// load); the data warps form two groups that take the pieces in turn, so one
// group streams while the other waits.
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

// 256 threads and at most 128 registers: two CTAs per SM, so that the send and the receive kernel of a rank
// (96 CTAs each by default) are resident side by side.
constexpr int kP2pThreads = 256;

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

__global__ void __launch_bounds__(kP2pThreads, 2) P2pKernel(const __grid_constant__ P2pParams p) {
  __shared__ RoleSync sync;
  if (threadIdx.x == 0) RoleSyncInit(&sync);
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
    // Two groups of data warps (even and odd warps) take the pieces in turn:
    // while one waits for the acknowledgement of its stores (the release
    // below), the other streams the next piece.
    const int group = warp & 1;
    const unsigned nthr = static_cast<unsigned>((data_warps + 1 - group) / 2) * 32u;
    const unsigned gtid = static_cast<unsigned>(warp >> 1) * 32u + static_cast<unsigned>(lane);
    for (uint64_t j = static_cast<uint64_t>(group); j < pieces; j += 2) {
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
        CopyBytes(box + b, static_cast<const unsigned char*>(p.src) + off + b, e - b, false, gtid, nthr);
      } else {
        const unsigned char* box = p.peers.arena[p.rank] + p.mailbox_offset + (static_cast<uint64_t>(p.peer) * p.slots + slot) * p.slot_bytes;
        CopyBytes(static_cast<unsigned char*>(p.dst) + off + b, box + b, e - b, true, gtid, nthr);
      }
      __syncwarp();
      if (lane == 0) StReleaseShared(&sync.done[warp], static_cast<unsigned>(j) + 1u);
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
        // The warps of the group that moved piece j.
        bool all = true;
        for (int wi = static_cast<int>(j & 1); wi < data_warps && all; wi += 2)
          all = SpinShared(&sync.done[wi], static_cast<unsigned>(j) + 1u, &sync, p.timeout_ns);
        if (!all) break;
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


// ---- broadcast through the switch ----
__device__ __forceinline__ void MultimemSt16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// 16 bytes from an address with no alignment guarantee.
__device__ __forceinline__ uint4 LdBytes16(const unsigned char* p) {
  union {
    uint4 v;
    unsigned char b[16];
  } u;
#pragma unroll
  for (int i = 0; i < 16; ++i) u.b[i] = p[i];
  return u.v;
}
__device__ __forceinline__ void MultimemStU64(void* mc, uint64_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(mc), "l"(v) : "memory");
}

__global__ void __launch_bounds__(kP2pThreads, 2) BcastKernel(const __grid_constant__ BcastParams p) {
  __shared__ RoleSync sync;
  if (threadIdx.x == 0) RoleSyncInit(&sync);
  __syncthreads();
  const int cta = blockIdx.x;
  const bool root = p.rank == p.root;
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
  ControlPage* mc_page = reinterpret_cast<ControlPage*>(p.peers.mc_arena);
  const uint64_t pieces = (p.bytes + p.slot_bytes - 1) / p.slot_bytes;
  const uint64_t part = p.slot_bytes / gridDim.x / 16 * 16;
  const uint64_t part_b = part * cta;
  const uint64_t part_e = (cta + 1 == static_cast<int>(gridDim.x)) ? p.slot_bytes : part_b + part;
  const int warps = static_cast<int>(blockDim.x) / 32, data_warps = warps - 2;
  const int warp = static_cast<int>(threadIdx.x) / 32, lane = static_cast<int>(threadIdx.x) % 32;
  volatile int* const stop = &sync.stop;

  if (warp < data_warps) {
    // Two groups of data warps (even and odd warps) take the pieces in turn:
    // while one waits for the acknowledgement of its stores (the release
    // below), the other streams the next piece.
    const int group = warp & 1;
    const unsigned nthr = static_cast<unsigned>((data_warps + 1 - group) / 2) * 32u;
    const unsigned gtid = static_cast<unsigned>(warp >> 1) * 32u + static_cast<unsigned>(lane);
    for (uint64_t j = static_cast<uint64_t>(group); j < pieces; j += 2) {
      int go = 1;
      if (lane == 0) go = SpinShared(&sync.ready, static_cast<unsigned>(j) + 1u, &sync, p.timeout_ns) ? 1 : 0;
      go = __shfl_sync(0xffffffffu, go, 0);
      if (!go) break;
      const uint64_t k = p.first_piece + j;
      const uint64_t off = j * p.slot_bytes;
      const uint64_t len = (p.bytes - off < p.slot_bytes) ? p.bytes - off : p.slot_bytes;
      const uint64_t b = part_b < len ? part_b : len, e = part_e < len ? part_e : len;
      const uint64_t slot_off = p.ring_offset + (k % p.slots) * p.slot_bytes;
      if (root) {
        unsigned char* box = p.peers.mc_arena + slot_off;
        const unsigned char* src = static_cast<const unsigned char*>(p.buf) + off;
        constexpr int kU = 8;
        const uint64_t v0 = b / 16, v1 = e / 16;
        const bool src_aligned = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
        for (uint64_t i = v0 + gtid; i < v1; i += static_cast<uint64_t>(nthr) * kU) {
          uint4 v[kU];
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            const uint64_t idx = i + static_cast<uint64_t>(u) * nthr;
            if (idx < v1) v[u] = src_aligned ? Ld16(src + idx * 16) : LdBytes16(src + idx * 16);
          }
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            const uint64_t idx = i + static_cast<uint64_t>(u) * nthr;
            if (idx < v1) MultimemSt16(box + idx * 16, v[u]);
          }
        }
      } else {
        const unsigned char* box = p.peers.arena[p.rank] + slot_off;
        CopyBytes(static_cast<unsigned char*>(p.buf) + off + b, box + b, e - b, true, gtid, nthr);
      }
      __syncwarp();
      if (lane == 0) StReleaseShared(&sync.done[warp], static_cast<unsigned>(j) + 1u);
    }
  } else if (warp == data_warps) {
    if (lane == 0) {
      for (uint64_t j = 0; j < pieces && *stop == 0; ++j) {
        const uint64_t k = p.first_piece + j;
        bool ok = true;
        if (root) {
          // The slot is free once every receiver consumed piece k - slots.
          if (k >= p.slots)
            for (int q = 0; q < p.world_size && ok; ++q)
              if (q != p.root) ok = WaitGE(&mine->bcast_credit[cta][q], k - p.slots + 1, w, kWaitP2p, q, static_cast<int>(j));
        } else {
          ok = WaitGE(&mine->bcast_flag[cta], k + 1, w, kWaitP2p, p.root, static_cast<int>(j));
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
        // The warps of the group that moved piece j.
        bool all = true;
        for (int wi = static_cast<int>(j & 1); wi < data_warps && all; wi += 2)
          all = SpinShared(&sync.done[wi], static_cast<unsigned>(j) + 1u, &sync, p.timeout_ns);
        if (!all) break;
        const uint64_t k = p.first_piece + j;
        if (root) {
          FenceSys();
          MultimemStU64(&mc_page->bcast_flag[cta], k + 1);
          // The root counts as a consumer of its own pieces: a later root waits
          // for the credits of every other rank, this one included.
          for (int q = 0; q < p.world_size; ++q) StRelaxedSys(&Ctl(p.peers, q)->bcast_credit[cta][p.rank], k + 1);
        } else {
          for (int q = 0; q < p.world_size; ++q) StRelaxedSys(&Ctl(p.peers, q)->bcast_credit[cta][p.rank], k + 1);
        }
      }
    }
  }
}

}  // namespace dev

cudaError_t LaunchP2pKernel(const P2pParams& p, int ctas, cudaStream_t stream) {
  if (ctas < 1 || ctas > kP2pCtas) return cudaErrorInvalidValue;
  dev::P2pKernel<<<ctas, dev::kP2pThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace ibcomm

namespace ibcomm {

cudaError_t LaunchBcastKernel(const BcastParams& p, int ctas, cudaStream_t stream) {
  if (ctas < 1 || ctas > kP2pCtas) return cudaErrorInvalidValue;
  if (p.peers.mc_arena == nullptr || p.bytes % 16 != 0 || p.bytes == 0) return cudaErrorInvalidValue;
  dev::BcastKernel<<<ctas, dev::kP2pThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace ibcomm
