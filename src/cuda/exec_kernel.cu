// Generic executor of op programs (ring and Rabenseifner allreduce).
//
// One CTA per channel.  A CTA walks the rank's program; for every op it waits
// (bounded) for the peer's data flag and for slot credit, streams its slice of
// the chunk through registers as 16-byte vectors
//     staging slot / sendbuf / recvbuf  (+ sendbuf|recvbuf) (* scale) (cast)
//         -> recvbuf and/or the next peer's staging slot over NVLink,
// then publishes the data flag to the receiver and returns the credit to the
// sender.  No host round trip and no separate reduce, cast or scale kernel.
//
// The CTA is warp-specialised so that the synchronisation of one op overlaps
// the data of its neighbours: one thread (the "waiter") runs ahead through
// the program and waits for the flags of the coming ops; the data warps
// stream op after op without a CTA-wide barrier, in two groups that take the
// ops in turn; another thread (the "poster") follows behind, and once the
// warps of an op's group have had their stores acknowledged it publishes the
// op's flags.  The parties hand over through counters in shared memory (ops
// ready; per data warp, ops done).
// Counterpart of the reference's host event loop around _reduce_inplace_cuda
// (ibcomm/allreduce_cuda_impl.h:24-33, 103-299, 470-707).
//
// With `emu` non-null the grid is (channels, ranks): blockIdx.y selects the
// rank whose parameters to use, so that several ranks that share one GPU run
// as ONE cooperative launch (CTAs that wait on each other are co-resident).
#include <cooperative_groups.h>

#include <cstdlib>

#include "flags.cuh"
#include "ibcomm/communicator.h"
#include "ibcomm/tunables.h"
#include "kernels.h"
#include "vec_ops.cuh"
#include "warp_roles.cuh"

namespace ibcomm {
namespace dev {

template <typename T, typename W>
struct ExecTraits {
  using A = typename Acc<T>::type;
  static constexpr int kMinBytes = sizeof(T) < sizeof(W) ? sizeof(T) : sizeof(W);
  static constexpr int P = 16 / kMinBytes;                       // elements per pack
  static constexpr int U = 64 / (P * static_cast<int>(sizeof(T))) > 0 ? 64 / (P * static_cast<int>(sizeof(T))) : 1;
};

// Vector path of one op: packs of P elements, U packs in flight per thread,
// all loads of an iteration issued before any use.  The op's shape (which
// sources, which destinations) is uniform over the CTA, so the branches below
// are predicates on registers, not divergence.
template <typename T, typename W>
__device__ __forceinline__ void VecLoop(const uint4* __restrict__ a_base, bool a_is_stage, const uint4* __restrict__ b_base,
                                        uint4* l_base, uint4* r_base, uint64_t npacks, bool do_scale, double scale, bool round_wire,
                                        unsigned tid, unsigned nthr) {
  using Tr = ExecTraits<T, W>;
  using A = typename Tr::A;
  constexpr int P = Tr::P;
  constexpr int U = Tr::U;
  constexpr int VT = P / VecIO<T>::kN;  // 16-byte vectors per pack in the user type
  constexpr int VW = P / VecIO<W>::kN;  // ... in the wire type
  const int va = a_is_stage ? VW : VT;
  const uint64_t stride = nthr;
  for (uint64_t i = tid; i < npacks; i += stride * U) {
    uint4 qa[U][VT];
    uint4 qb[U][VT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t idx = i + static_cast<uint64_t>(u) * stride;
      if (idx < npacks) {
        if (a_is_stage) {
#pragma unroll
          for (int v = 0; v < VW; ++v) qa[u][v] = Ld16Strong(a_base + idx * VW + v);
        } else {
#pragma unroll
          for (int v = 0; v < VT; ++v) qa[u][v] = Ld16(a_base + idx * VT + v);
        }
        if (b_base != nullptr) {
#pragma unroll
          for (int v = 0; v < VT; ++v) qb[u][v] = Ld16(b_base + idx * VT + v);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t idx = i + static_cast<uint64_t>(u) * stride;
      if (idx < npacks) {
        A acc[P];
        if (a_is_stage) {
#pragma unroll
          for (int v = 0; v < VW; ++v) VecIO<W>::Load(qa[u][v], acc + v * VecIO<W>::kN);
        } else {
#pragma unroll
          for (int v = 0; v < VT; ++v) VecIO<T>::Load(qa[u][v], acc + v * VecIO<T>::kN);
        }
        if (b_base != nullptr) {
#pragma unroll
          for (int v = 0; v < VT; ++v) VecIO<T>::Add(qb[u][v], acc + v * VecIO<T>::kN);
        }
        if (do_scale) {
#pragma unroll
          for (int e = 0; e < P; ++e) acc[e] = ScaleAcc<A>(acc[e], scale);
        }
        uint4 wq[VW];
        if (r_base != nullptr || round_wire) {
#pragma unroll
          for (int v = 0; v < VW; ++v) wq[v] = VecIO<W>::Store(acc + v * VecIO<W>::kN);
        }
        if (r_base != nullptr) {
#pragma unroll
          for (int v = 0; v < VW; ++v) St16(r_base + idx * VW + v, wq[v]);
        }
        if (l_base != nullptr) {
          if (round_wire && sizeof(W) != sizeof(T)) {
#pragma unroll
            for (int v = 0; v < VW; ++v) VecIO<W>::Load(wq[v], acc + v * VecIO<W>::kN);
          }
#pragma unroll
          for (int v = 0; v < VT; ++v) St16(l_base + idx * VT + v, VecIO<T>::Store(acc + v * VecIO<T>::kN));
        }
      }
    }
  }
  (void)va;
}

// Element-at-a-time path for chunks that do not start on a 16-byte boundary
// and for the few elements after the last whole pack.
template <typename T, typename W>
__device__ void ScalarLoop(const Op& op, const T* sendbuf, T* recvbuf, const W* stage_in, W* stage_out, uint64_t lo,
                           uint64_t hi, double scale, unsigned tid, unsigned nthr) {
  using A = typename Acc<T>::type;
  for (uint64_t k = lo + tid; k < hi; k += nthr) {
    const uint64_t g = op.cell_begin + k;
    A v;
    if (op.src_a == kSrcStage) v = ToAcc<A, W>(LdScalarStrong<W>(stage_in + k));
    else if (op.src_a == kSrcSend) v = ToAcc<A, T>(sendbuf[g]);
    else v = ToAcc<A, T>(recvbuf[g]);
    if (op.src_b == kSrcSend) v += ToAcc<A, T>(sendbuf[g]);
    else if (op.src_b == kSrcRecv) v += ToAcc<A, T>(recvbuf[g]);
    if (op.flags & kOpScale) v = ScaleAcc<A>(v, scale);
    if ((op.flags & kOpRoundWire) && sizeof(W) != sizeof(T)) v = ToAcc<A, W>(FromAcc<W, A>(v));
    if (op.flags & kOpStoreLocal) recvbuf[g] = FromAcc<T, A>(v);
    if (op.flags & kOpStoreRemote) stage_out[k] = FromAcc<W, A>(v);
  }
}

template <typename T, typename W>
__device__ void RunOpData(const Op& op, const ExecParams& p, int ch, int nch, unsigned tid, unsigned nthr) {
  using Tr = ExecTraits<T, W>;
  uint64_t lo, hi;
  ChannelSlice(op.elem_begin - op.cell_begin, op.elem_count, p.stage.slot_bytes / sizeof(W), nch, ch, &lo, &hi);
  if (lo >= hi) return;
  const T* sendbuf = static_cast<const T*>(p.sendbuf);
  T* recvbuf = static_cast<T*>(p.recvbuf);
  const StageLayout& st = p.stage;
  const W* stage_in = nullptr;
  W* stage_out = nullptr;
  if (op.src_a == kSrcStage)
    stage_in = reinterpret_cast<const W*>(p.peers.arena[p.rank] + st.offset +
                                          (static_cast<uint64_t>(op.region_in) * st.slots + op.slot_in) * st.slot_bytes);
  if (op.flags & kOpStoreRemote)
    stage_out = reinterpret_cast<W*>(p.peers.arena[op.peer_out] + st.offset +
                                     (static_cast<uint64_t>(op.region_out) * st.slots + op.slot_out) * st.slot_bytes);
  const uint64_t g0 = op.cell_begin + lo;
  const bool uses_send = op.src_a == kSrcSend || op.src_b == kSrcSend;
  const bool uses_recv = op.src_a == kSrcRecv || op.src_b == kSrcRecv || (op.flags & kOpStoreLocal);
  bool aligned = true;
  if (uses_send) aligned &= (reinterpret_cast<uintptr_t>(sendbuf + g0) & 15u) == 0;
  if (uses_recv) aligned &= (reinterpret_cast<uintptr_t>(recvbuf + g0) & 15u) == 0;
  // The place inside a staging slot follows the cell, not the user buffer: a
  // range that starts in the middle of a cell (Rabenseifner pieces, 16-bit
  // wire) can be 16-byte aligned on the user side and not in the slot.
  if (stage_in != nullptr) aligned &= (reinterpret_cast<uintptr_t>(stage_in + lo) & 15u) == 0;
  if (stage_out != nullptr) aligned &= (reinterpret_cast<uintptr_t>(stage_out + lo) & 15u) == 0;
  if (!aligned) {
    ScalarLoop<T, W>(op, sendbuf, recvbuf, stage_in, stage_out, lo, hi, p.scale, tid, nthr);
    return;
  }
  const uint64_t npacks = (hi - lo) / Tr::P;
  {
    const bool a_is_stage = op.src_a == kSrcStage;
    const uint4* a_base = a_is_stage ? reinterpret_cast<const uint4*>(stage_in + lo)
                          : (op.src_a == kSrcSend) ? reinterpret_cast<const uint4*>(sendbuf + g0)
                                                   : reinterpret_cast<const uint4*>(recvbuf + g0);
    const uint4* b_base = (op.src_b == kSrcSend)   ? reinterpret_cast<const uint4*>(sendbuf + g0)
                          : (op.src_b == kSrcRecv) ? reinterpret_cast<const uint4*>(recvbuf + g0)
                                                   : nullptr;
    uint4* l_base = (op.flags & kOpStoreLocal) ? reinterpret_cast<uint4*>(recvbuf + g0) : nullptr;
    uint4* r_base = (op.flags & kOpStoreRemote) ? reinterpret_cast<uint4*>(stage_out + lo) : nullptr;
    VecLoop<T, W>(a_base, a_is_stage, b_base, l_base, r_base, npacks, (op.flags & kOpScale) != 0, p.scale,
                  (op.flags & kOpRoundWire) != 0, tid, nthr);
  }
  const uint64_t done = lo + npacks * Tr::P;
  if (done < hi) ScalarLoop<T, W>(op, sendbuf, recvbuf, stage_in, stage_out, done, hi, p.scale, tid, nthr);
}

// Body of the executor for one CTA; returns when the program is done or a wait gave up.
// Self-check of an op before any of its addresses is formed: the message
// range, the place inside the staging slot and the slot, region and peer
// indices.  A failing op is reported (status "bad program") and the call
// stops; nothing is accessed out of range and nothing traps.
template <typename W>
__device__ __forceinline__ bool OpInBounds(const Op& op, const ExecParams& p) {
  if (op.elem_begin > p.len_elements || op.elem_count > p.len_elements - op.elem_begin) return false;
  if (op.cell_begin > op.elem_begin) return false;
  const bool reads_stage = op.src_a == kSrcStage || op.src_b == kSrcStage;
  const bool writes_stage = (op.flags & kOpStoreRemote) != 0;
  if (reads_stage || writes_stage) {
    if ((op.elem_begin - op.cell_begin + op.elem_count) * sizeof(W) > p.stage.slot_bytes) return false;
  }
  if (reads_stage && (op.region_in >= p.stage.regions || op.slot_in >= p.stage.slots)) return false;
  if (writes_stage && (op.region_out >= p.stage.regions || op.slot_out >= p.stage.slots || op.peer_out < 0 ||
                       op.peer_out >= p.world_size))
    return false;
  if ((op.wait_in != 0 || op.post_credit != 0) && (op.peer_in < 0 || op.peer_in >= p.world_size)) return false;
  if ((op.wait_credit != 0 || op.post_out != 0) && (op.peer_out < 0 || op.peer_out >= p.world_size)) return false;
  return true;
}

// Body of the executor for one CTA: warps [0, data_warps) move data, lane 0 of
// the next warp is the waiter, lane 0 of the last warp the poster.
template <typename T, typename W>
__device__ void ExecBody(const ExecParams& p, uint64_t seq, RoleSync* sync) {
  const int ch = blockIdx.x, nch = gridDim.x;
  WaitCtx w;
  w.peers = &p.peers;
  w.status = p.status;
  w.doorbell = p.doorbell;
  w.seq = seq;
  w.timeout_ns = p.timeout_ns;
  w.rank = p.rank;
  w.world_size = p.world_size;
  w.channel = ch;
  const uint64_t base = seq << 32;
  ControlPage* const me = Ctl(p.peers, p.rank);
  volatile int* const stop = &sync->stop;

  // Entry barrier per channel: every peer's channel `ch` has started this
  // call, hence finished the previous one, so staging slots are free.
  if (threadIdx.x < p.world_size && threadIdx.x != p.rank) {
    StReleaseSys(&Ctl(p.peers, threadIdx.x)->bar[ch][p.rank], base | 1u);
    if (!WaitGE(&me->bar[ch][threadIdx.x], base | 1u, w, kWaitBarrier, threadIdx.x, -1)) *stop = 1;
  }
  __syncthreads();
  if (*stop) return;

  DeviceTraceRec* trace = (p.trace != nullptr && p.trace_capacity > 0) ? p.trace + static_cast<size_t>(ch) * p.trace_capacity : nullptr;
  const int warps = static_cast<int>(blockDim.x) / 32;
  const int data_warps = warps - 2;
  const int warp = static_cast<int>(threadIdx.x) / 32, lane = static_cast<int>(threadIdx.x) % 32;

  if (warp < data_warps) {
    // Two groups of data warps (even and odd warps) take the ops in turn.
    // After its stores a group waits until they are acknowledged over NVLink
    // (the release below) before the poster may publish the op; meanwhile the
    // other group loads and stores the next op, so the link does not idle
    // during the hand-over.  Consecutive ops are independent of each other
    // (different chains of the ring, different pieces of a halving step) with
    // one exception, handled by the barrier below.
    const int group = warp & 1;
    const unsigned all_threads = static_cast<unsigned>(data_warps) * 32u;
    const unsigned nthr = static_cast<unsigned>((data_warps + 1 - group) / 2) * 32u;
    const unsigned gtid = static_cast<unsigned>(warp >> 1) * 32u + static_cast<unsigned>(lane);
    bool alive = true;
    for (int oi = 0; oi < p.num_ops; ++oi) {
      const Op op = p.ops[oi];
      // No barrier separates consecutive ops, and an element need not map to
      // the same thread in two ops that cover different ranges.  An op that
      // reads recvbuf (Rabenseifner's running partial sums, written by earlier
      // ops) therefore first waits until every data warp, of both groups, has
      // finished the ops before it.  Every data warp walks the whole program
      // and meets these barriers, also after the call was stopped.
      // Overwrites need no such barrier: a range is overwritten only by data
      // that a peer derived from this rank's own transfer of the range, which
      // the poster published after all warps of the op's group had read it.
      if (op.src_a == kSrcRecv || op.src_b == kSrcRecv) asm volatile("bar.sync 1, %0;" ::"r"(all_threads) : "memory");
      if ((oi & 1) != group || !alive) continue;
      int go = 1;
      if (lane == 0) go = SpinShared(&sync->ready, static_cast<unsigned>(oi) + 1u, sync, p.timeout_ns) ? 1 : 0;
      go = __shfl_sync(0xffffffffu, go, 0);
      if (!go) {
        alive = false;
        continue;
      }
      RunOpData<T, W>(op, p, ch, nch, gtid, nthr);
      __syncwarp();
      if (lane == 0) StReleaseShared(&sync->done[warp], static_cast<unsigned>(oi) + 1u);
    }
  } else if (warp == data_warps) {
    if (lane == 0) {
      // Waiter: bounds check, then the op's data flag and slot credit.
      for (int oi = 0; oi < p.num_ops && *stop == 0; ++oi) {
        const Op op = p.ops[oi];
        bool ok = OpInBounds<W>(op, p);
        if (!ok) {
          ReportFailure(w, kStatusBadProgram, 0, -1, oi, op.elem_begin, op.elem_count);
          BroadcastAbort(w);
        }
        if (ok && op.wait_in != 0) ok = WaitGE(&me->inflag[ch][op.peer_in], base | op.wait_in, w, kWaitData, op.peer_in, oi);
        if (ok && op.wait_credit != 0)
          ok = WaitGE(&me->credit[ch][op.peer_out], base | op.wait_credit, w, kWaitCredit, op.peer_out, oi);
        if (!ok) {
          *stop = 1;
          break;
        }
        if (trace != nullptr && oi < p.trace_capacity) trace[oi].t_wait_done = GlobalTimerNs();
        StReleaseShared(&sync->ready, static_cast<unsigned>(oi) + 1u);
      }
    }
  } else {
    if (lane == 0) {
      // Poster: when all data warps have issued the op's stores, make them
      // visible system-wide and publish the op's flags.
      for (int oi = 0; oi < p.num_ops; ++oi) {
        // The warps of the group that ran op oi.
        bool all = true;
        for (int wi = oi & 1; wi < data_warps && all; wi += 2)
          all = SpinShared(&sync->done[wi], static_cast<unsigned>(oi) + 1u, sync, p.timeout_ns);
        if (!all) break;
        const Op op = p.ops[oi];
        if (op.post_out != 0) {
          FenceSys();
          StRelaxedSys(&Ctl(p.peers, op.peer_out)->inflag[ch][p.rank], base | op.post_out);
        }
        if (op.post_credit != 0) StRelaxedSys(&Ctl(p.peers, op.peer_in)->credit[ch][p.rank], base | op.post_credit);
        if (trace != nullptr && oi < p.trace_capacity) trace[oi].t_done = GlobalTimerNs();
      }
    }
  }
}

template <typename T, typename W>
__global__ void __launch_bounds__(kExecThreads, 1)
ExecKernel(const __grid_constant__ ExecParams p0, const ExecParams* __restrict__ emu) {
  __shared__ ExecParams p;
  __shared__ RoleSync s_sync;
  __shared__ uint64_t s_seq;
  {
    const uint32_t* src = (emu != nullptr) ? reinterpret_cast<const uint32_t*>(emu + blockIdx.y)
                                           : reinterpret_cast<const uint32_t*>(&p0);
    for (unsigned i = threadIdx.x; i < sizeof(ExecParams) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(&p)[i] = src[i];
    if (threadIdx.x == 0) RoleSyncInit(&s_sync);
  }
  __syncthreads();
  if (p.world_size <= 1) return;
  const uint64_t seq = BeginCollective(p.peers, p.rank, &s_seq);
  // num_ops <= 0: this rank sits the call out (test hook), but still counts it.
  if (p.num_ops > 0) ExecBody<T, W>(p, seq, &s_sync);
  EndCollective(p.peers, p.rank, seq, gridDim.x);
}

}  // namespace dev

static int ExecThreads() {
  const int v = Tunable("IBCOMM_EXEC_THREADS", 0);
  return (v >= 64 && v <= kExecThreads && v % 32 == 0) ? v : kExecThreads;
}

template <typename T, typename W>
static cudaError_t Launch(const ExecParams& p, const ExecParams* emu, int emu_ranks, int channels, cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>(channels), static_cast<unsigned>(emu != nullptr ? emu_ranks : 1));
  // Beyond one CTA per SM, two smaller CTAs share an SM: while one waits for a
  // flag, the other streams.
  const int kThreads = ExecKernelThreadsFor(channels);
  if (emu != nullptr) {
    // Ranks sharing one GPU wait on each other inside this launch: it must be
    // cooperative so the runtime refuses a grid that cannot be co-resident.
    void* args[] = {const_cast<ExecParams*>(&p), &emu};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(dev::ExecKernel<T, W>), grid, dim3(kThreads), args, 0, stream);
  }
  dev::ExecKernel<T, W><<<grid, kThreads, 0, stream>>>(p, nullptr);
  return cudaGetLastError();
}

cudaError_t LaunchExecKernel(const ExecParams& p, const ExecParams* emu, int emu_ranks, int channels, cudaStream_t stream) {
  const DType t = static_cast<DType>(p.dtype), w = static_cast<DType>(p.wire);
  if (t == DType::kFloat32 && w == DType::kFloat32) return Launch<float, float>(p, emu, emu_ranks, channels, stream);
  if (t == DType::kFloat32 && w == DType::kBFloat16) return Launch<float, __nv_bfloat16>(p, emu, emu_ranks, channels, stream);
  if (t == DType::kFloat32 && w == DType::kFloat16) return Launch<float, __half>(p, emu, emu_ranks, channels, stream);
  if (t == DType::kFloat64 && w == t) return Launch<double, double>(p, emu, emu_ranks, channels, stream);
  if (t == DType::kInt32 && w == t) return Launch<int, int>(p, emu, emu_ranks, channels, stream);
  if (t == DType::kInt64 && w == t) return Launch<long long, long long>(p, emu, emu_ranks, channels, stream);
  if (t == DType::kFloat16 && w == t) return Launch<__half, __half>(p, emu, emu_ranks, channels, stream);
  if (t == DType::kBFloat16 && w == t) return Launch<__nv_bfloat16, __nv_bfloat16>(p, emu, emu_ranks, channels, stream);
  return cudaErrorInvalidValue;
}

int ExecKernelThreadsFor(int channels) { return (channels > 148 && ExecThreads() > 256) ? 256 : ExecThreads(); }

int ExecKernelMaxCoResidentBlocks(int device, int threads) {
  int per_sm = 0, sms = 0;
  if (threads <= 0) threads = kExecThreads;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dev::ExecKernel<float, float>, threads, 0) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  return per_sm * sms;
}

}  // namespace ibcomm
