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
// shard) and which this rank copies to `recvbuf`.  There are `buffers` (3 to
// 6) windows of each kind, and three roles work on different windows at the
// same time:
//
//   loader    sendbuf -> input window k+2 ...                 local HBM traffic
//   reducers  input window k -> output window k               NVLink traffic
//   storer    output window k-1 -> recvbuf                    local HBM traffic
//
// so the links stay busy while the copies run, where the sequential kernel
// (nvls_kernel.cu) leaves them idle during its copy phases.  A role can be
// several groups of warps that take the windows in turn (window k belongs to
// group k mod groups): a window can only be published once its stores have
// been acknowledged over NVLink, which takes microseconds, and while one
// reducer group waits for that, the other streams the next window.
//
// Where the roles run:
//   * every block runs all of them (one loader, one storer, two reducer
//     groups: 1 + 1 + 14 warps with bulk copies, 3 + 3 + 10 with copies in
//     registers), or
//   * split (the default where twice the blocks are co-resident): blocks
//     [0, n) only reduce, blocks [n, 2n) only copy, block n + b serving the
//     same part of every window as block b.  A release at system scope waits
//     for every store the SM has in flight; next to reducers that made a
//     loader's hand-over cost an NVLink round trip under load (9-12 us per
//     window for 32 KiB of local copying, measured with the per-role stamps
//     below).  In split mode the roles can have up to four groups each and the
//     reducer groups optional poster warps that fence and publish behind the
//     data warps (both off by default: within a few percent on 2 B200).
//
// When the wire type equals the buffer type the copies are bulk asynchronous
// copies (TMA, `cp.async.bulk`, global -> shared -> global, no multicast, this
// GPU's memory only) driven by one thread per copy group through a ring of
// shared-memory stages; with a 16-bit wire the copy groups convert in
// registers instead (fp32 accumulation in the reducers either way).
//
// Synchronisation is per block index across ranks, with rows of the control
// page (values (call << 32) | window + 1, growing only; group g of a role
// owns the rows b + g * n, so groups publish independently):
//   inflag[..][q]   rank q's loader has filled its input window k
//   bar[..][q]      rank q has reduced its part of window k
//   credit[..][q]   rank q's storer has copied output window k out
// loader k waits for "reduced" of window k - buffers (input buffer free
// again), reducer k for "filled" of window k and "copied out" of window
// k - buffers, storer k for "reduced" of window k.  Block b touches the same
// bytes of a window on every rank (part b of every shard), so no
// block-to-block synchronisation is needed.  Every wait is bounded.
//
// With tracing on, block 0 stamps %globaltimer per window and role
// (StagedParams::trace_roles; Communicator.staged_timeline() in Python).
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
#include "warp_roles.cuh"

namespace ibcomm {
namespace dev {

constexpr int kStagedThreads = 512;
// Warps per group.  With bulk copies one thread drives each copy group, so
// the loader and the storer are one warp each and 14 warps reduce; with
// copies in registers (16-bit wire) the split is 3 / 3 / 10.
constexpr int kLoadWarpsRegs = 3;
constexpr int kStagedMaxCtas = 128;   // blocks that reduce (and, unsplit, copy too)
constexpr int kStagedMaxGroups = 4;   // groups of one role that work on different windows at the same time
constexpr uint32_t kBulkChunk = 8192;   // bytes per bulk copy
constexpr int kBulkMaxDepth = 12;       // stages per ring at most (a lane and an mbarrier each)
constexpr int kBulkMaxRings = 2 * kStagedMaxGroups;
constexpr size_t kStagedSmemBytes = 192u << 10;

enum StagedRow : int { kRowInReady = 0, kRowReduced = 1, kRowOutFree = 2 };

__device__ __forceinline__ void GroupSync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Window k's word row of one kind: the groups of a role finish their windows
// independently of each other, so each group has rows of its own (window k
// belongs to group k % groups) and the values of a row only grow.
__device__ __forceinline__ uint64_t* FlagRow(ControlPage* page, int row, int cta, int ncta, uint64_t window, int groups) {
  const int r = cta + static_cast<int>(window % static_cast<uint64_t>(groups)) * ncta;
  return row == kRowInReady ? page->inflag[r] : (row == kRowReduced ? page->bar[r] : page->credit[r]);
}

// State every thread of a warp group shares.
struct RoleCtx {
  WaitCtx w;
  int tid;       // 0 .. nthr - 1 inside the group
  int nthr;      // threads of the group
  int bar_id;    // the group's named barrier
  int slot;      // the group's row in `role_stop`
  int cta, ncta;
  volatile int* stop;            // set by whoever gives up in this block; the call is over
  volatile int (*role_stop)[2];  // [slot][round & 1]: the group's own, uniform view of `stop`
  uint32_t round;
};

// Waits until every rank's word for `flag_window` in `row` (a role with
// `groups` groups) has reached `value`.  All threads of the group call it and
// get the same answer: false when the call is over (a wait ran out here or
// elsewhere).
__device__ __forceinline__ bool RoleWait(RoleCtx& c, int row, uint64_t flag_window, int groups, uint64_t value, uint32_t kind, int window) {
  uint64_t* words = FlagRow(Ctl(*c.w.peers, c.w.rank), row, c.cta, c.ncta, flag_window, groups);
  const int slot = static_cast<int>(c.round & 1u);
  ++c.round;
  bool mine = true;
  if (c.tid < c.w.world_size) mine = WaitGE(words + c.tid, value, c.w, kind, c.tid, window);
  if (!mine) *c.stop = 1;
  if (!mine || (c.tid == 0 && *c.stop != 0)) c.role_stop[c.slot][slot] = 1;
  GroupSync(c.bar_id, c.nthr);
  return c.role_stop[c.slot][slot] == 0;
}

// Publishes `value` for `flag_window` in `row` at every rank (this rank
// included).  Everything the group wrote before is ordered ahead of the flag.
__device__ __forceinline__ void RolePost(RoleCtx& c, int row, uint64_t flag_window, int groups, uint64_t value) {
  GroupSync(c.bar_id, c.nthr);
  if (c.tid < c.w.world_size) StReleaseSys(FlagRow(Ctl(*c.w.peers, c.tid), row, c.cta, c.ncta, flag_window, groups) + c.w.rank, value);
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
  unsigned char* smem;  // `depth` stages of `chunk` bytes
  uint64_t* full;       // one mbarrier per stage
  uint32_t chunk;       // bytes per bulk copy (a multiple of 16)
  uint32_t depth;       // stages
  uint32_t count;       // chunks moved so far: stage = count % depth, phase parity = (count / depth) & 1
};

// Copies `npieces` contiguous pieces (16-byte aligned, sizes multiples of 16).
// Loads run up to depth - 1 chunks ahead of the stores.  Returns false when a
// load did not arrive within the limit; the stores issued so far are complete
// either way when this returns.  (Measured alternatives that were slower on
// two B200 under the reducers' traffic: half the stages for loads and half for
// stores in flight, and a lane per stage, each with its own load-store chain.)
__device__ inline bool BulkCopyPieces(BulkRing& ring, unsigned char* const* dst, const unsigned char* const* src,
                                      const uint64_t* bytes, int npieces) {
  const uint32_t chunk = ring.chunk, depth = ring.depth;
  uint32_t total = 0;
  for (int s = 0; s < npieces; ++s) total += static_cast<uint32_t>((bytes[s] + chunk - 1) / chunk);
  int ls = 0, ss = 0;
  uint64_t loff = 0, soff = 0;
  uint32_t ld = 0;
  auto issue_load = [&]() {
    while (ls < npieces && loff >= bytes[ls]) {
      ++ls;
      loff = 0;
    }
    const uint64_t left = bytes[ls] - loff;
    const uint32_t n = left < chunk ? static_cast<uint32_t>(left) : chunk;
    const uint32_t stage = (ring.count + ld) % depth;
    MbarExpectTx(&ring.full[stage], n);
    BulkLoad(ring.smem + static_cast<size_t>(stage) * chunk, src[ls] + loff, n, &ring.full[stage]);
    loff += n;
    ++ld;
  };
  while (ld < total && ld < depth - 1) issue_load();
  bool ok = true;
  for (uint32_t st = 0; st < total; ++st) {
    const uint32_t use = ring.count + st;
    const uint32_t stage = use % depth;
    if (!MbarWait(&ring.full[stage], (use / depth) & 1u)) {
      ok = false;
      break;
    }
    while (ss < npieces && soff >= bytes[ss]) {
      ++ss;
      soff = 0;
    }
    const uint64_t left = bytes[ss] - soff;
    const uint32_t n = left < chunk ? static_cast<uint32_t>(left) : chunk;
    BulkStore(dst[ss] + soff, ring.smem + static_cast<size_t>(stage) * chunk, n);
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
  __shared__ int s_role_stop[3 * kStagedMaxGroups][2];
  __shared__ uint64_t s_full[kBulkMaxRings][kBulkMaxDepth];
  __shared__ RoleSync s_sync;  // reducing blocks in split mode: done[g] = windows whose stores group g has issued
  {
    const uint32_t* src = (emu != nullptr) ? reinterpret_cast<const uint32_t*>(emu + blockIdx.y) : reinterpret_cast<const uint32_t*>(&p0);
    for (unsigned i = threadIdx.x; i < sizeof(StagedParams) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(&p)[i] = src[i];
    if (threadIdx.x == 0) {
      s_stop = 0;
      RoleSyncInit(&s_sync);
      for (int r = 0; r < 3 * kStagedMaxGroups; ++r) s_role_stop[r][0] = s_role_stop[r][1] = 0;
      for (int r = 0; r < kBulkMaxRings; ++r)
        for (int s = 0; s < kBulkMaxDepth; ++s) MbarInit(&s_full[r][s], 1);
      MbarInitFence();
    }
  }
  __syncthreads();
  const uint64_t seq = BeginCollective(p.peers, p.rank, &s_seq);

  // Roles share a block, or - `split_ctas` - live in blocks of their own:
  // blocks [0, n) reduce with all 16 warps, blocks [n, 2n) copy (block n + b
  // serves the same part of every window as block b).  The roles only talk
  // through the flag rows, so nothing else changes; what changes is what a
  // hand-over costs.  A release at system scope waits for every store the SM
  // has in flight, and next to reducers that is a round trip over NVLink under
  // load (measured 9-12 us per window for a loader that had copied 32 KiB of
  // local memory).  Even without that, one pass of a role over a window is a
  // chain of five or six memory round trips (flags, copy, completion, fence,
  // flags): about 10 us on busy GPUs whatever the size.  So in split mode a
  // role is several groups that take the windows in turn (window k belongs to
  // group k mod groups): their chains overlap.
  const bool split = p.split_ctas != 0;
  const int ncta = split ? static_cast<int>(gridDim.x / 2) : static_cast<int>(gridDim.x);
  const bool copy_cta = split && static_cast<int>(blockIdx.x) >= ncta;
  const int cta = copy_cta ? static_cast<int>(blockIdx.x) - ncta : static_cast<int>(blockIdx.x);
  const int ws = p.world_size, me = p.rank;
  const uint64_t total_nv = p.len_elements / P;
  const uint64_t full_nv = p.window_elems / P;
  const uint64_t windows = full_nv == 0 ? 0 : (total_nv + full_nv - 1) / full_nv;
  const bool tma = p.use_tma != 0 && sizeof(T) == sizeof(W);
  const uint64_t base = seq << 32;
  // Input windows, and output windows, in the pool: at least three (two being
  // reduced, one being filled or emptied); more give the copies more time.
  const uint64_t kStagedBuffers = static_cast<uint64_t>(p.buffers < 3 ? 3 : (p.buffers > kStagedMaxBuffers ? kStagedMaxBuffers : p.buffers));
  auto clamp_groups = [](int g) { return g < 1 ? 1 : (g > kStagedMaxGroups ? kStagedMaxGroups : g); };
  // Groups per role.  Unsplit: one loader, one storer, two reducer groups.
  const int LG = split ? clamp_groups(p.load_groups) : 1;
  const int SG = split ? clamp_groups(p.store_groups) : 1;
  const int RG = split ? clamp_groups(p.reduce_groups) : 2;

  constexpr int kWarps = kStagedThreads / 32;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  // Warps of a copy group: one when a thread drives the copy engine, otherwise
  // 3 (unsplit) or as many as fit into half a block (split).
  const int copy_warps = tma ? 1 : (split ? kWarps / 2 / (LG > SG ? LG : SG) : kLoadWarpsRegs);
  // role: 0 loader, 1 storer, 2 reducer, -1 none; group inside the role; thread inside the group.
  int role = -1, group = 0, gthreads = 0, gtid = 0;
  if (!split) {
    if (warp < copy_warps) {
      role = 0, gthreads = 32 * copy_warps, gtid = threadIdx.x;
    } else if (warp < 2 * copy_warps) {
      role = 1, gthreads = 32 * copy_warps, gtid = threadIdx.x - 32 * copy_warps;
    } else {
      const int rwarp = warp - 2 * copy_warps, rwarps = kWarps - 2 * copy_warps;
      role = 2, group = rwarp % RG, gthreads = 32 * ((rwarps - group + RG - 1) / RG), gtid = (rwarp / RG) * 32 + lane;
    }
  } else if (copy_cta) {
    const int half = kWarps / 2, w2 = warp % half;
    const int groups = warp < half ? LG : SG;
    if (w2 < groups * copy_warps) role = warp < half ? 0 : 1, group = w2 / copy_warps, gthreads = 32 * copy_warps, gtid = (w2 % copy_warps) * 32 + lane;
  } else {
    // Reducing block: RG groups of data warps and, behind each, a poster warp
    // that fences the group's stores and publishes the window while the group
    // is already on its next one (the fence waits for the acknowledgements of
    // the stores over NVLink, 8-15 us under load).
    const int data_warps = p.posters != 0 ? kWarps - RG : kWarps;
    if (warp < data_warps) {
      role = 2, group = warp % RG, gthreads = 32 * ((data_warps - group + RG - 1) / RG), gtid = (warp / RG) * 32 + lane;
    } else {
      role = 3, group = warp - data_warps, gthreads = 32, gtid = lane;
    }
  }
  const bool has_poster = split && !copy_cta && p.posters != 0;

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
  c.ncta = ncta;
  c.stop = &s_stop;
  c.role_stop = s_role_stop;
  c.round = 0;
  c.tid = gtid;
  c.nthr = gthreads;
  c.slot = (role < 0 || role > 2 ? 0 : role) * kStagedMaxGroups + group;
  c.bar_id = 1 + c.slot;  // named barriers 1 .. 12 (0 is __syncthreads); posters are single warps and need none

  DeviceTraceRec* const trace = (p.trace != nullptr && p.trace_capacity > 0) ? p.trace + static_cast<size_t>(cta) * p.trace_capacity : nullptr;
  // Stamps of the other roles (see StagedParams::trace_roles).
  const uint64_t role_w = (trace != nullptr && p.trace_roles > 0) ? static_cast<uint64_t>(p.trace_roles) : 0;
  // The copy groups' rings share the dynamic shared memory: 2 rings of 6 x 16 KiB, 4 of 6 x 8 KiB, 6 of 4 x 8 KiB, 8 of 3 x 8 KiB.
  const int rings = split ? LG + SG : 2;
  const uint32_t ring_chunk = rings <= 2 ? 2 * kBulkChunk : kBulkChunk;
  const uint32_t ring_bytes = static_cast<uint32_t>(kStagedSmemBytes / static_cast<size_t>(rings)) / ring_chunk * ring_chunk;
  const uint32_t ring_depth = ring_bytes / ring_chunk < 6u ? ring_bytes / ring_chunk : 6u;
  const int ring_index = role == 0 ? group : LG + group;
  BulkRing ring{smem + static_cast<size_t>(ring_index) * ring_bytes, s_full[ring_index % kBulkMaxRings], ring_chunk, ring_depth, 0};
  const bool mover = !tma || gtid == 0;
  if (role == 0) {
    // ------------------------------------------------------------ loader
    for (uint64_t k = static_cast<uint64_t>(group); k < windows; k += static_cast<uint64_t>(LG)) {
      const int j = static_cast<int>(k % kStagedBuffers);
      const uint64_t v0 = k * full_nv;
      const uint64_t nv = total_nv - v0 < full_nv ? total_nv - v0 : full_nv;
      // The input buffer is free once every rank has reduced the window that used it before.
      if (k >= kStagedBuffers &&
          !RoleWait(c, kRowReduced, k - kStagedBuffers, RG, base | (k - kStagedBuffers + 1), kWaitBarrier, static_cast<int>(k)))
        break;
      if (role_w != 0 && gtid == 0) trace[role_w + k].t_wait_done = GlobalTimerNs();
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
          // Reported here; the group leaves together at its next wait.
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
      RolePost(c, kRowInReady, k, LG, base | (k + 1));
      if (role_w != 0 && gtid == 0) trace[role_w + k].t_done = GlobalTimerNs();
    }
  } else if (role == 1) {
    // ------------------------------------------------------------ storer
    for (uint64_t k = static_cast<uint64_t>(group); k < windows; k += static_cast<uint64_t>(SG)) {
      const int j = static_cast<int>(k % kStagedBuffers);
      const uint64_t v0 = k * full_nv;
      const uint64_t nv = total_nv - v0 < full_nv ? total_nv - v0 : full_nv;
      if (!RoleWait(c, kRowReduced, k, RG, base | (k + 1), kWaitBarrier, static_cast<int>(k))) break;
      if (role_w != 0 && gtid == 0) trace[2 * role_w + k].t_wait_done = GlobalTimerNs();
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
          // Reported here; the group leaves together at its next wait.
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
      RolePost(c, kRowOutFree, k, SG, base | (k + 1));
      if (role_w != 0 && gtid == 0) trace[2 * role_w + k].t_done = GlobalTimerNs();
    }
  } else if (role == 2) {
    // ----------------------------------------------------------- reducer
    const int reduce_threads = gthreads;
    const bool do_scale = p.scale != 1.0;
    bool finished = windows <= static_cast<uint64_t>(group);
    for (uint64_t k = static_cast<uint64_t>(group); k < windows; k += static_cast<uint64_t>(RG)) {
      const int j = static_cast<int>(k % kStagedBuffers);
      const uint64_t v0 = k * full_nv;
      const uint64_t nv = total_nv - v0 < full_nv ? total_nv - v0 : full_nv;
      // Every rank's input window k is filled (which also says that every rank
      // runs this call, hence is done with whatever used the pool before) ...
      if (!RoleWait(c, kRowInReady, k, LG, base | (k + 1), kWaitData, static_cast<int>(k))) break;
      // ... and every rank has emptied the output buffer this window reuses.
      if (k >= kStagedBuffers &&
          !RoleWait(c, kRowOutFree, k - kStagedBuffers, SG, base | (k - kStagedBuffers + 1), kWaitCredit, static_cast<int>(k)))
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
      if (role_w != 0 && c.tid == 0) trace[3 * role_w + k].t_wait_done = GlobalTimerNs();
      if (has_poster) {
        // Hand the window to the poster: every thread's stores are issued (the
        // barrier), and the release makes them part of what the poster's fence orders.
        GroupSync(c.bar_id, c.nthr);
        if (c.tid == 0) StReleaseShared(&s_sync.done[group], static_cast<unsigned>(k / static_cast<uint64_t>(RG)) + 1u);
      } else {
        RolePost(c, kRowReduced, k, RG, base | (k + 1));
        if (trace != nullptr && c.tid == 0 && k < static_cast<uint64_t>(p.trace_capacity)) trace[k].t_done = GlobalTimerNs();
      }
      finished = k + static_cast<uint64_t>(RG) >= windows;
    }
    // Left early (a wait ran out): the poster must not wait for windows that will not come.
    if (has_poster && !finished && c.tid == 0) *reinterpret_cast<volatile int*>(&s_sync.stop) = 1;
  } else if (role == 3) {
    // ------------------------------------------------------------ poster
    for (uint64_t k = static_cast<uint64_t>(group); k < windows; k += static_cast<uint64_t>(RG)) {
      int ok = 1;
      if (lane == 0) ok = SpinShared(&s_sync.done[group], static_cast<unsigned>(k / static_cast<uint64_t>(RG)) + 1u, &s_sync, p.timeout_ns) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      __syncwarp();  // lane 0's acquire is ordered before the other lanes' releases
      if (lane < ws) StReleaseSys(FlagRow(Ctl(p.peers, lane), kRowReduced, cta, ncta, k, RG) + me, base | (k + 1));
      if (trace != nullptr && lane == 0 && k < static_cast<uint64_t>(p.trace_capacity)) trace[k].t_done = GlobalTimerNs();
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
