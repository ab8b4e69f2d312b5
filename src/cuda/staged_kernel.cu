// Pipelined two-shot allreduce through the pool, for buffers the peers cannot
// map (the caller's ordinary device memory - the reference's contract,
// ibcomm/ibverbs_communicator.h:102-114) and for fp32 buffers that travel as
// bf16 or fp16.
//
// The message moves in windows.  A window lives in two pool buffers: the
// input window, which this rank fills from `sendbuf` and which every rank
// reads (its own shard of it, from every rank: `multimem.ld_reduce` in the
// NVSwitch, or peer loads summed in rank order), and the output window, which
// every rank writes (`multimem.st` / peer stores of its reduced, scaled
// shard) and which this rank copies to `recvbuf`.  There are three buffers of
// each kind, and the 16 warps of a CTA are four groups that work on up to four
// windows at the same time:
//
//   loader     sendbuf -> input window k+2                    local HBM traffic
//   reducer A  input windows k   -> output windows k   (even k)   NVLink traffic
//   reducer B  input windows k+1 -> output windows k+1 (odd k)    NVLink traffic
//   storer     output window k-1 -> recvbuf                   local HBM traffic
//
// so the links stay busy while the copies run, where the sequential kernel
// (nvls_kernel.cu) leaves them idle during its copy phases.  Two reducer
// groups because a window can only be published once its stores have been
// acknowledged over NVLink, which takes microseconds: while one group waits
// for that, the other streams the next window.  When the wire type equals the
// buffer type the copies are bulk asynchronous copies (TMA, `cp.async.bulk`,
// global -> shared -> global, no multicast, this GPU's memory only) driven by
// one thread of the loader warp and one of the storer warp through six-deep
// rings of 16 KiB shared-memory stages (the other 14 warps reduce); with a
// 16-bit wire the loader and the storer (three warps each) convert in
// registers instead (fp32 accumulation in the reducers either way).
//
// Synchronisation is per CTA index across ranks, with rows of the control
// page (values (call << 32) | window + 1, growing only):
//   inflag[b][q]              rank q's CTA b has filled its input window k
//   bar[b][q], bar[b+128][q]  rank q's CTA b has reduced its part of window k
//                             (even k / odd k: the two reducer groups finish
//                             their windows independently of each other)
//   credit[b][q]              rank q's CTA b has copied output window k out
// loader k waits for "reduced" >= k-2 (input buffer free again), reducer k for
// inflag >= k+1 and credit >= k-2, storer k for "reduced" >= k+1.  CTA b
// touches the same bytes of a window on every rank (part b of every shard),
// so no CTA-to-CTA synchronisation is needed.  Every wait is bounded.
//
// Requirements (the host falls back to the sequential kernel otherwise):
// 16-byte aligned buffers and a length that is a whole number of 16-byte
// wire vectors.  The reference has no counterpart (it stages through pinned
// host memory with one copy, one kernel and one copy per chunk,
// ibcomm/allreduce_cuda_impl.h:129-135).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "flags.cuh"
#include "ibcomm/communicator.h"
#include "kernels.h"
#include "tma_stage.cuh"
#include "twoshot_common.cuh"
#include "vec_ops.cuh"

namespace ibcomm {
namespace dev {

constexpr int kStagedThreads = 512;
// Warps per group.  With bulk copies one thread drives each copy group, so
// the loader and the storer are one warp each and 14 warps reduce; with
// copies in registers (16-bit wire) the split is 3 / 3 / 10.
constexpr int kLoadWarpsBulk = 1, kStoreWarpsBulk = 1;
constexpr int kLoadWarpsRegs = 3, kStoreWarpsRegs = 3;
constexpr int kBarLoad = 1, kBarStore = 2, kBarReduce = 3;  // named barriers of the groups (0 is __syncthreads); reducer B uses kBarReduce + 1
constexpr int kStagedMaxCtas = 128;   // the odd windows' "reduced" flags live in bar[cta + 128]
constexpr uint32_t kBulkChunk = 16384;  // bytes per bulk copy
constexpr int kBulkDepth = 6;           // stages per copy group
constexpr size_t kStagedSmemBytes = 2ull * kBulkDepth * kBulkChunk;

enum StagedRole : int { kRoleLoad = 0, kRoleStore = 1, kRoleReduce = 2 /* and 3 for reducer B */ };
enum StagedRow : int { kRowInReady = 0, kRowReduced = 1, kRowOutFree = 2 };

__device__ __forceinline__ void GroupSync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// `window` selects the row of the "reduced" flags (even or odd windows).
__device__ __forceinline__ uint64_t* FlagRow(ControlPage* page, int row, int cta, uint64_t window) {
  return row == kRowInReady ? page->inflag[cta]
                            : (row == kRowReduced ? page->bar[cta + ((window & 1) != 0 ? kStagedMaxCtas : 0)] : page->credit[cta]);
}

// State every thread of a warp group shares.
struct RoleCtx {
  WaitCtx w;
  int tid;       // 0 .. nthr - 1 inside the group
  int nthr;      // threads of the group that take part (1 when one thread drives bulk copies)
  int bar_id;
  int role;
  int cta;
  volatile int* stop;            // set by whoever gives up; the call is over
  volatile int (*role_stop)[2];  // [role][round & 1]: the group's own, uniform view of `stop`
  uint32_t round;
};

// Waits until every rank's word in `row` has reached `value`.  All `nthr`
// threads of the group call it and get the same answer: false when the call
// is over (a wait ran out here or elsewhere).
__device__ __forceinline__ bool RoleWait(RoleCtx& c, int row, uint64_t flag_window, uint64_t value, uint32_t kind, int window) {
  uint64_t* words = FlagRow(Ctl(*c.w.peers, c.w.rank), row, c.cta, flag_window);
  const int slot = static_cast<int>(c.round & 1u);
  ++c.round;
  if (c.nthr == 1) {
    bool ok = *c.stop == 0;
    for (int q = 0; q < c.w.world_size && ok; ++q) ok = WaitGE(words + q, value, c.w, kind, q, window);
    if (!ok) *c.stop = 1;
    return ok;
  }
  bool mine = true;
  if (c.tid < c.w.world_size) mine = WaitGE(words + c.tid, value, c.w, kind, c.tid, window);
  if (!mine) *c.stop = 1;
  if (!mine || (c.tid == 0 && *c.stop != 0)) c.role_stop[c.role][slot] = 1;
  GroupSync(c.bar_id, c.nthr);
  return c.role_stop[c.role][slot] == 0;
}

// Publishes `value` in `row` at every rank (this rank included).  Everything
// the group wrote before is ordered ahead of the flag.
__device__ __forceinline__ void RolePost(RoleCtx& c, int row, uint64_t flag_window, uint64_t value) {
  if (c.nthr == 1) {
    // One fence for all ranks' flags (a release per flag would wait for the
    // previous flag's acknowledgement every time).
    FenceSys();
    for (int q = 0; q < c.w.world_size; ++q) StRelaxedSys(FlagRow(Ctl(*c.w.peers, q), row, c.cta, flag_window) + c.w.rank, value);
    return;
  }
  GroupSync(c.bar_id, c.nthr);
  if (c.tid < c.w.world_size) StReleaseSys(FlagRow(Ctl(*c.w.peers, c.tid), row, c.cta, flag_window) + c.w.rank, value);
}

// ---- copies in registers (with the conversion between buffer and wire type) ----
// Wire vectors [b, e) of a window; `user` and `wire` point at the window's first element.
template <typename T, typename W>
__device__ __forceinline__ void CastIn(uint4* wire, const uint4* user, uint64_t b, uint64_t e, int tid, int nthr) {
  using A = typename Acc<T>::type;
  constexpr int P = 16 / static_cast<int>(sizeof(W));
  constexpr int VT = P * static_cast<int>(sizeof(T)) / 16;
  constexpr int U = VT == 1 ? 8 : 4;
  for (uint64_t i = b + tid; i < e; i += static_cast<uint64_t>(nthr) * U) {
    uint4 q[U][VT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t idx = i + static_cast<uint64_t>(u) * nthr;
      if (idx < e) {
#pragma unroll
        for (int v = 0; v < VT; ++v) q[u][v] = Ld16(user + idx * VT + v);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t idx = i + static_cast<uint64_t>(u) * nthr;
      if (idx < e) {
        if constexpr (sizeof(T) == sizeof(W)) {
          St16(wire + idx, q[u][0]);
        } else {
          A acc[P];
#pragma unroll
          for (int v = 0; v < VT; ++v) VecIO<T>::Load(q[u][v], acc + v * VecIO<T>::kN);
          St16(wire + idx, VecIO<W>::Store(acc));
        }
      }
    }
  }
}

template <typename T, typename W>
__device__ __forceinline__ void CastOut(uint4* user, const uint4* wire, uint64_t b, uint64_t e, int tid, int nthr) {
  using A = typename Acc<T>::type;
  constexpr int P = 16 / static_cast<int>(sizeof(W));
  constexpr int VT = P * static_cast<int>(sizeof(T)) / 16;
  constexpr int U = 8;
  for (uint64_t i = b + tid; i < e; i += static_cast<uint64_t>(nthr) * U) {
    uint4 q[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t idx = i + static_cast<uint64_t>(u) * nthr;
      if (idx < e) q[u] = Ld16Strong(wire + idx);  // written by the peers
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t idx = i + static_cast<uint64_t>(u) * nthr;
      if (idx < e) {
        if constexpr (sizeof(T) == sizeof(W)) {
          St16(user + idx, q[u]);
        } else {
          A acc[P];
          VecIO<W>::Load(q[u], acc);
#pragma unroll
          for (int v = 0; v < VT; ++v) St16(user + idx * VT + v, VecIO<T>::Store(acc + v * VecIO<T>::kN));
        }
      }
    }
  }
}

// ---- copies by the bulk copy engine: global -> shared -> global, one thread ----
struct BulkRing {
  unsigned char* smem;  // kBulkDepth stages of kBulkChunk bytes
  uint64_t* full;       // one mbarrier per stage
  uint32_t count;       // chunks moved so far: stage = count % depth, phase parity = (count / depth) & 1
};

// Copies `npieces` contiguous pieces (16-byte aligned, sizes multiples of 16).
// Loads run up to kBulkDepth - 1 chunks ahead of the stores.  Returns false
// when a load did not arrive within the limit; the stores issued so far are
// complete either way when this returns.
__device__ inline bool BulkCopyPieces(BulkRing& ring, unsigned char* const* dst, const unsigned char* const* src,
                                      const uint64_t* bytes, int npieces) {
  uint32_t total = 0;
  for (int s = 0; s < npieces; ++s) total += static_cast<uint32_t>((bytes[s] + kBulkChunk - 1) / kBulkChunk);
  int ls = 0, ss = 0;
  uint64_t loff = 0, soff = 0;
  uint32_t ld = 0;
  auto issue_load = [&]() {
    while (ls < npieces && loff >= bytes[ls]) {
      ++ls;
      loff = 0;
    }
    const uint64_t left = bytes[ls] - loff;
    const uint32_t n = left < kBulkChunk ? static_cast<uint32_t>(left) : kBulkChunk;
    const uint32_t stage = (ring.count + ld) % kBulkDepth;
    MbarExpectTx(&ring.full[stage], n);
    BulkLoad(ring.smem + static_cast<size_t>(stage) * kBulkChunk, src[ls] + loff, n, &ring.full[stage]);
    loff += n;
    ++ld;
  };
  while (ld < total && ld < static_cast<uint32_t>(kBulkDepth - 1)) issue_load();
  bool ok = true;
  for (uint32_t st = 0; st < total; ++st) {
    const uint32_t use = ring.count + st;
    const uint32_t stage = use % kBulkDepth;
    if (!MbarWait(&ring.full[stage], (use / kBulkDepth) & 1u)) {
      ok = false;
      break;
    }
    while (ss < npieces && soff >= bytes[ss]) {
      ++ss;
      soff = 0;
    }
    const uint64_t left = bytes[ss] - soff;
    const uint32_t n = left < kBulkChunk ? static_cast<uint32_t>(left) : kBulkChunk;
    BulkStore(dst[ss] + soff, ring.smem + static_cast<size_t>(stage) * kBulkChunk, n);
    BulkCommit();
    soff += n;
    // All stores but this one have read their stage: the previous chunk's
    // stage is free for the load that runs depth - 1 ahead.
    BulkWaitRead<1>();
    if (ld < total) issue_load();
  }
  BulkWaitAll();
  ring.count += total;
  return ok;
}

template <typename T, typename W, bool kMultimem, int kR>
__global__ void __launch_bounds__(kStagedThreads, 1)
StagedKernel(const __grid_constant__ StagedParams p0, const StagedParams* __restrict__ emu) {
  static_assert(sizeof(W) <= sizeof(T), "the wire type is never wider than the buffer type");
  using AW = typename Acc<W>::type;
  constexpr int P = 16 / static_cast<int>(sizeof(W));                // elements per wire vector
  constexpr int VT = P * static_cast<int>(sizeof(T)) / 16;           // user vectors per wire vector
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ StagedParams p;
  __shared__ uint64_t s_seq;
  __shared__ int s_stop;
  __shared__ int s_role_stop[4][2];
  __shared__ uint64_t s_full[2][kBulkDepth];
  {
    const uint32_t* src = (emu != nullptr) ? reinterpret_cast<const uint32_t*>(emu + blockIdx.y) : reinterpret_cast<const uint32_t*>(&p0);
    for (unsigned i = threadIdx.x; i < sizeof(StagedParams) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(&p)[i] = src[i];
    if (threadIdx.x == 0) {
      s_stop = 0;
      for (int r = 0; r < 4; ++r) s_role_stop[r][0] = s_role_stop[r][1] = 0;
      for (int r = 0; r < 2; ++r)
        for (int s = 0; s < kBulkDepth; ++s) MbarInit(&s_full[r][s], 1);
      MbarInitFence();
    }
  }
  __syncthreads();
  const uint64_t seq = BeginCollective(p.peers, p.rank, &s_seq);

  const int cta = blockIdx.x, ncta = gridDim.x;
  const int ws = p.world_size, me = p.rank;
  const uint64_t total_nv = p.len_elements / P;
  const uint64_t full_nv = p.window_elems / P;
  const uint64_t windows = full_nv == 0 ? 0 : (total_nv + full_nv - 1) / full_nv;
  const bool tma = p.use_tma != 0 && sizeof(T) == sizeof(W);
  const uint64_t base = seq << 32;
  // Input windows, and output windows, in the pool: at least three (two being
  // reduced, one being filled or emptied); more give the copies more time.
  const uint64_t kStagedBuffers = static_cast<uint64_t>(p.buffers < 3 ? 3 : (p.buffers > kStagedMaxBuffers ? kStagedMaxBuffers : p.buffers));

  RoleCtx c;
  c.w.peers = &p.peers;
  c.w.status = p.status;
  c.w.doorbell = p.doorbell;
  c.w.seq = seq;
  c.w.timeout_ns = p.timeout_ns;
  c.w.rank = me;
  c.w.world_size = ws;
  c.w.channel = cta;
  c.cta = cta;
  c.stop = &s_stop;
  c.role_stop = s_role_stop;
  c.round = 0;

  const int warp = threadIdx.x / 32;
  const int load_warps = tma ? kLoadWarpsBulk : kLoadWarpsRegs;
  const int store_warps = tma ? kStoreWarpsBulk : kStoreWarpsRegs;
  if (warp < load_warps) {
    // ------------------------------------------------------------ loader
    c.role = kRoleLoad;
    c.bar_id = kBarLoad;
    c.tid = threadIdx.x;
    // With bulk copies lane 0 moves the data; the other lanes of the warp share the flag waits and posts.
    c.nthr = 32 * load_warps;
    const bool mover = !tma || c.tid == 0;
    {
      BulkRing ring{smem, s_full[0], 0};
      for (uint64_t k = 0; k < windows; ++k) {
        const int j = static_cast<int>(k % kStagedBuffers);
        const uint64_t v0 = k * full_nv;
        const uint64_t nv = total_nv - v0 < full_nv ? total_nv - v0 : full_nv;
        // The input buffer is free once every rank has reduced the window that used it before.
        if (k >= kStagedBuffers &&
            !RoleWait(c, kRowReduced, k - kStagedBuffers, base | (k - kStagedBuffers + 1), kWaitBarrier, static_cast<int>(k)))
          break;
        unsigned char* win = p.stage[me] + p.in_off[j];
        const unsigned char* user = static_cast<const unsigned char*>(p.sendbuf) + v0 * 16 * VT;
        if (tma && mover) {
          unsigned char* dst[kMaxRanks];
          const unsigned char* src[kMaxRanks];
          uint64_t bytes[kMaxRanks];
          for (int s = 0; s < ws; ++s) {
            uint64_t b, e;
            WindowPart(full_nv, nv, s, ws, cta, ncta, &b, &e);
            dst[s] = win + b * 16;
            src[s] = user + b * 16;
            bytes[s] = (e - b) * 16;
          }
          FenceProxyAsyncAll();
          if (!BulkCopyPieces(ring, dst, src, bytes, ws)) {
            // Reported here; the warp leaves together at its next wait.
            ReportFailure(c.w, kStatusWaitTimeout, kWaitData, me, static_cast<int>(k), 0, 0);
            BroadcastAbort(c.w);
            s_stop = 1;
          }
          FenceProxyAsyncAll();
        } else if (!tma) {
          for (int s = 0; s < ws; ++s) {
            uint64_t b, e;
            WindowPart(full_nv, nv, s, ws, cta, ncta, &b, &e);
            CastIn<T, W>(reinterpret_cast<uint4*>(win), reinterpret_cast<const uint4*>(user), b, e, c.tid, c.nthr);
          }
        }
        RolePost(c, kRowInReady, k, base | (k + 1));
      }
    }
  } else if (warp < load_warps + store_warps) {
    // ------------------------------------------------------------ storer
    c.role = kRoleStore;
    c.bar_id = kBarStore;
    c.tid = threadIdx.x - 32 * load_warps;
    c.nthr = 32 * store_warps;
    const bool mover = !tma || c.tid == 0;
    {
      BulkRing ring{smem + static_cast<size_t>(kBulkDepth) * kBulkChunk, s_full[1], 0};
      for (uint64_t k = 0; k < windows; ++k) {
        const int j = static_cast<int>(k % kStagedBuffers);
        const uint64_t v0 = k * full_nv;
        const uint64_t nv = total_nv - v0 < full_nv ? total_nv - v0 : full_nv;
        if (!RoleWait(c, kRowReduced, k, base | (k + 1), kWaitBarrier, static_cast<int>(k))) break;
        const unsigned char* win = p.stage[me] + p.out_off[j];
        unsigned char* user = static_cast<unsigned char*>(p.recvbuf) + v0 * 16 * VT;
        if (tma && mover) {
          unsigned char* dst[kMaxRanks];
          const unsigned char* src[kMaxRanks];
          uint64_t bytes[kMaxRanks];
          for (int s = 0; s < ws; ++s) {
            uint64_t b, e;
            WindowPart(full_nv, nv, s, ws, cta, ncta, &b, &e);
            dst[s] = user + b * 16;
            src[s] = win + b * 16;
            bytes[s] = (e - b) * 16;
          }
          // The window was written by ordinary stores of the peers (made
          // visible by the flags just acquired); the copy engine reads it.
          FenceProxyAsyncAll();
          if (!BulkCopyPieces(ring, dst, src, bytes, ws)) {
            // Reported here; the warp leaves together at its next wait.
            ReportFailure(c.w, kStatusWaitTimeout, kWaitData, me, static_cast<int>(k), 0, 0);
            BroadcastAbort(c.w);
            s_stop = 1;
          }
          FenceProxyAsyncAll();
        } else if (!tma) {
          for (int s = 0; s < ws; ++s) {
            uint64_t b, e;
            WindowPart(full_nv, nv, s, ws, cta, ncta, &b, &e);
            CastOut<T, W>(reinterpret_cast<uint4*>(user), reinterpret_cast<const uint4*>(win), b, e, c.tid, c.nthr);
          }
        }
        RolePost(c, kRowOutFree, k, base | (k + 1));
      }
    }
  } else {
    // ----------------------------------------------------------- reducer
    // Two groups (even and odd warps of the reducers) take the windows in turn.
    const int rwarp = warp - load_warps - store_warps, rwarps = kStagedThreads / 32 - load_warps - store_warps;
    const int sub = rwarp & 1;
    const int reduce_threads = 32 * ((rwarps + 1 - sub) / 2);
    c.role = kRoleReduce + sub;
    c.bar_id = kBarReduce + sub;
    c.tid = (rwarp >> 1) * 32 + static_cast<int>(threadIdx.x % 32);
    c.nthr = reduce_threads;
    const bool do_scale = p.scale != 1.0;
    DeviceTraceRec* trace = (p.trace != nullptr && p.trace_capacity > 0) ? p.trace + static_cast<size_t>(cta) * p.trace_capacity : nullptr;
    for (uint64_t k = static_cast<uint64_t>(sub); k < windows; k += 2) {
      const int j = static_cast<int>(k % kStagedBuffers);
      const uint64_t v0 = k * full_nv;
      const uint64_t nv = total_nv - v0 < full_nv ? total_nv - v0 : full_nv;
      // Every rank's input window k is filled (which also says that every rank
      // runs this call, hence is done with whatever used the pool before) ...
      if (!RoleWait(c, kRowInReady, k, base | (k + 1), kWaitData, static_cast<int>(k))) break;
      // ... and every rank has emptied the output buffer this window reuses.
      if (k >= kStagedBuffers &&
          !RoleWait(c, kRowOutFree, k - kStagedBuffers, base | (k - kStagedBuffers + 1), kWaitCredit, static_cast<int>(k)))
        break;
      if (trace != nullptr && c.tid == 0 && k < static_cast<uint64_t>(p.trace_capacity)) trace[k].t_wait_done = GlobalTimerNs();
      uint64_t b, e;
      WindowPart(full_nv, nv, me, ws, cta, ncta, &b, &e);
      if constexpr (kMultimem) {
        constexpr int kU = 4;
        const unsigned char* mi = p.mc_stage + p.in_off[j];
        unsigned char* mo = p.mc_stage + p.out_off[j];
        for (uint64_t i = b + c.tid; i < e; i += static_cast<uint64_t>(reduce_threads) * kU) {
          uint4 v[kU];
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            const uint64_t idx = i + static_cast<uint64_t>(u) * reduce_threads;
            if (idx < e) v[u] = Multimem<W>::LdReduce(mi + idx * 16);
          }
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            const uint64_t idx = i + static_cast<uint64_t>(u) * reduce_threads;
            if (idx < e) {
              if (do_scale) {
                AW acc[P];
                VecIO<W>::Load(v[u], acc);
#pragma unroll
                for (int x = 0; x < P; ++x) acc[x] = ScaleAcc<AW>(acc[x], p.scale);
                v[u] = VecIO<W>::Store(acc);
              }
              Multimem<W>::St(mo + idx * 16, v[u]);
            }
          }
        }
      } else {
        unsigned char* const* arenas = p.stage;
        const uint64_t out_off = p.out_off[j];
        PeerReduceGroup<W, kR>(arenas, ws, p.in_off[j], b, e, do_scale, p.scale,
                               [&](uint64_t idx, uint4 r) {
#pragma unroll
                                 for (int q = 0; q < kMaxRanks; ++q)
                                   if (q < ws) St16(arenas[q] + out_off + idx * 16, r);
                               },
                               static_cast<unsigned>(c.tid), static_cast<unsigned>(reduce_threads));
      }
      RolePost(c, kRowReduced, k, base | (k + 1));
      if (trace != nullptr && c.tid == 0 && k < static_cast<uint64_t>(p.trace_capacity)) trace[k].t_done = GlobalTimerNs();
    }
  }
  EndCollective(p.peers, p.rank, seq, gridDim.x);
}

}  // namespace dev

template <typename T, typename W, bool kMultimem, int kR>
static cudaError_t LaunchStagedOne(const StagedParams& p, const StagedParams* emu, int emu_ranks, int blocks, cudaStream_t stream) {
  auto kernel = dev::StagedKernel<T, W, kMultimem, kR>;
  // Per (function, device); cheap, so made on every launch.
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dev::kStagedSmemBytes));
  if (e != cudaSuccess) return e;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(emu != nullptr ? emu_ranks : 1));
  if (emu != nullptr) {
    void* args[] = {const_cast<StagedParams*>(&p), &emu};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), grid, dim3(dev::kStagedThreads), args, dev::kStagedSmemBytes, stream);
  }
  kernel<<<grid, dev::kStagedThreads, dev::kStagedSmemBytes, stream>>>(p, nullptr);
  return cudaGetLastError();
}

template <typename T, typename W>
static cudaError_t LaunchStagedTyped(const StagedParams& p, const StagedParams* emu, int emu_ranks, int blocks, cudaStream_t stream) {
  if (p.use_multimem) {
    if constexpr (dev::HasMultimem<W>::value) {
      return LaunchStagedOne<T, W, true, kMaxRanks>(p, emu, emu_ranks, blocks, stream);
    } else {
      return cudaErrorInvalidValue;
    }
  }
  switch (dev::RankClass(p.world_size)) {
    case 2: return LaunchStagedOne<T, W, false, 2>(p, emu, emu_ranks, blocks, stream);
    case 4: return LaunchStagedOne<T, W, false, 4>(p, emu, emu_ranks, blocks, stream);
    default: return LaunchStagedOne<T, W, false, kMaxRanks>(p, emu, emu_ranks, blocks, stream);
  }
}

cudaError_t LaunchStagedKernel(const StagedParams& p, const StagedParams* emu, int emu_ranks, int blocks, cudaStream_t stream) {
  const DType t = static_cast<DType>(p.dtype), w = static_cast<DType>(p.wire);
  if (t == DType::kFloat32 && w == DType::kBFloat16) return LaunchStagedTyped<float, __nv_bfloat16>(p, emu, emu_ranks, blocks, stream);
  if (t == DType::kFloat32 && w == DType::kFloat16) return LaunchStagedTyped<float, __half>(p, emu, emu_ranks, blocks, stream);
  if (t != w) return cudaErrorInvalidValue;
  switch (t) {
    case DType::kFloat32: return LaunchStagedTyped<float, float>(p, emu, emu_ranks, blocks, stream);
    case DType::kFloat16: return LaunchStagedTyped<__half, __half>(p, emu, emu_ranks, blocks, stream);
    case DType::kBFloat16: return LaunchStagedTyped<__nv_bfloat16, __nv_bfloat16>(p, emu, emu_ranks, blocks, stream);
    case DType::kFloat64: return LaunchStagedTyped<double, double>(p, emu, emu_ranks, blocks, stream);
    case DType::kInt32: return LaunchStagedTyped<int, int>(p, emu, emu_ranks, blocks, stream);
    case DType::kInt64: return LaunchStagedTyped<long long, long long>(p, emu, emu_ranks, blocks, stream);
  }
  return cudaErrorInvalidValue;
}

int StagedKernelMaxCoResidentBlocks(int device) {
  int per_sm = 0, sms = 0;
  auto kernel = dev::StagedKernel<float, float, false, kMaxRanks>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dev::kStagedSmemBytes)) != cudaSuccess) return 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, dev::kStagedThreads, dev::kStagedSmemBytes) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  return per_sm * sms;
}

}  // namespace ibcomm
