#include "ibcomm/emu_world.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>

#include "engine.h"
#include "ibcomm/tunables.h"

namespace ibcomm {

struct EmuWorld::Impl {
  int ws = 1;
  int device = 0;
  ArenaLayout layout;
  unsigned char* arenas = nullptr;  // ws arenas back to back
  std::vector<StatusBlock> status;
  std::vector<RankResources> ranks;
  ProgramCache cache;
  void* d_params = nullptr;  // parameter blocks of one launch
  size_t d_params_bytes = 0;
  int timeout_ms = env::kDefaultTimeoutMs;
  int max_blocks = 0;
  int last_channels = 0;
  int silent_rank = -1;
  int bad_program_rank = -1;
  int direct_staging = 0;  // 0 in place, 1 staged window by window, 2 staged through the pipelined kernel
  int staged_max_blocks = 0;
  uint32_t last_status = 0;
  DeviceStatus last_report{};

  void* Params(size_t bytes) {
    if (bytes > d_params_bytes) {
      if (d_params != nullptr) CUDACHECK(cudaFree(d_params));
      CUDACHECK(cudaMalloc(&d_params, bytes));
      d_params_bytes = bytes;
    }
    return d_params;
  }
};

EmuWorld::EmuWorld(int num_ranks, size_t pool_bytes, size_t work_bytes) : ws_(num_ranks), impl_(new Impl()) {
  if (num_ranks < 1 || num_ranks > kMaxRanks)
    IBCOMM_FAIL(NOT_SUPPORTED, "EmuWorld supports 1..%d ranks (got %d).\n", kMaxRanks, num_ranks);
  Impl& m = *impl_;
  m.ws = num_ranks;
  CUDACHECK(cudaGetDevice(&m.device));
  m.timeout_ms = env::ReadTimeoutMs();
  m.layout = MakeArenaLayout(pool_bytes ? pool_bytes : env::ReadPreAllocSize(), work_bytes ? work_bytes : env::ReadWorkGpuMemorySize(), num_ranks);
  const size_t total = static_cast<size_t>(m.layout.total_bytes) * static_cast<size_t>(num_ranks);
  CUDACHECK(cudaMalloc(&m.arenas, total));
  CUDACHECK(cudaMemset(m.arenas, 0, total));
  m.status.resize(static_cast<size_t>(num_ranks));
  m.ranks.resize(static_cast<size_t>(num_ranks));
  for (int r = 0; r < num_ranks; ++r) {
    m.status[static_cast<size_t>(r)].Create();
    RankResources& rr = m.ranks[static_cast<size_t>(r)];
    rr.rank = r;
    rr.world_size = num_ranks;
    rr.layout = m.layout;
    for (int q = 0; q < num_ranks; ++q) rr.peers.arena[q] = m.arenas + static_cast<size_t>(q) * m.layout.total_bytes;
    rr.peers.mc_arena = nullptr;
    rr.d_status = m.status[static_cast<size_t>(r)].d_status;
    rr.h_doorbell = m.status[static_cast<size_t>(r)].h_doorbell;
    rr.d_doorbell = m.status[static_cast<size_t>(r)].d_doorbell;
  }
  m.max_blocks = ExecKernelMaxCoResidentBlocks(m.device, 0);
  m.staged_max_blocks = StagedKernelMaxCoResidentBlocks(m.device);
  CUDACHECK(cudaDeviceSynchronize());
}

EmuWorld::~EmuWorld() {
  Impl& m = *impl_;
  cudaDeviceSynchronize();
  m.cache.Clear();
  for (StatusBlock& s : m.status) s.Destroy();
  if (m.arenas != nullptr) cudaFree(m.arenas);
  if (m.d_params != nullptr) cudaFree(m.d_params);
  (void)cudaGetLastError();
}

void EmuWorld::SetSilentRank(int r) { impl_->silent_rank = r; }
void EmuWorld::SetBadProgramRank(int r) { impl_->bad_program_rank = r; }
void EmuWorld::SetDirectStaging(int mode) { impl_->direct_staging = mode; }
void EmuWorld::SetTimeoutMs(int ms) { impl_->timeout_ms = ms > 0 ? ms : env::ReadTimeoutMs(); }
int EmuWorld::last_channels() const { return impl_->last_channels; }

uint32_t EmuWorld::LastStatus(DeviceStatus* report) const {
  if (report != nullptr) *report = impl_->last_report;
  return impl_->last_status;
}

void EmuWorld::Allreduce(Algo algo, DType dtype, const std::vector<const void*>& sendbufs, const std::vector<void*>& recvbufs,
                         size_t n, double scale, DType wire, int channels, void* stream_v, bool async) {
  Impl& m = *impl_;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (static_cast<int>(sendbufs.size()) != m.ws || static_cast<int>(recvbufs.size()) != m.ws)
    IBCOMM_FAIL(INVALID_ARGUMENT, "EmuWorld::Allreduce needs one buffer pair per rank.\n");
  for (int r = 0; r < m.ws; ++r)
    if (sendbufs[static_cast<size_t>(r)] == nullptr || recvbufs[static_cast<size_t>(r)] == nullptr)
      IBCOMM_FAIL(INVALID_ARGUMENT, "EmuWorld::Allreduce: null buffer.\n");
  if (dtype != DType::kFloat32) wire = dtype;
  const size_t esize = DTypeSize(dtype);
  const size_t bytes = n * esize;
  m.last_status = 0;

  if (m.ws == 1) {
    CopyParams cp{sendbufs[0], recvbufs[0], n, static_cast<int32_t>(dtype), static_cast<int32_t>(dtype), scale};
    if (!(sendbufs[0] == recvbufs[0] && scale == 1.0)) CUDACHECK(LaunchCopyKernel(cp, kCopyDefaultBlocks, stream));
    m.last_channels = 0;
    if (!async) CUDACHECK(cudaStreamSynchronize(stream));
    return;
  }

  if (algo == Algo::kAuto) algo = ChooseAlgorithm(bytes, m.ws, false, false, kMaxChannels).algo;
  if (algo == Algo::kNvls)
    IBCOMM_FAIL(NOT_SUPPORTED, "Algorithm 'nvls' needs NVSwitch multicast between GPUs; it cannot be emulated on one GPU.\n");
  const uint64_t timeout_ns = static_cast<uint64_t>(m.timeout_ms) * 1000000ull;
  const int cap = std::max(1, m.max_blocks / m.ws);

  bool all_aligned = true;
  for (int q = 0; q < m.ws; ++q)
    all_aligned = all_aligned && ((reinterpret_cast<uintptr_t>(sendbufs[static_cast<size_t>(q)]) | reinterpret_cast<uintptr_t>(recvbufs[static_cast<size_t>(q)])) & 15u) == 0;
  const size_t wsize = DTypeSize(wire);
  if (algo == Algo::kDirect && (wire != dtype || m.direct_staging == 2)) {
    // The pipelined staged kernel (what ordinary buffers and 16-bit wires get on several GPUs).
    // Copy roles in blocks of their own: twice the blocks, all of them co-resident with every rank's.
    const bool split = Tunable("IBCOMM_STAGED_SPLIT", 1) != 0 && m.staged_max_blocks / m.ws >= 2;
    int buffers = Tunable("IBCOMM_STAGED_BUFFERS", 3);
    buffers = std::max(3, std::min(buffers, kStagedMaxBuffers));
    const uint64_t quarter = (m.layout.pool_bytes + m.layout.work_bytes) / static_cast<uint64_t>(2 * buffers) / 4096 * 4096;
    if (!all_aligned || (n * wsize) % 16 != 0 || quarter < 4096)
      IBCOMM_FAIL(NOT_SUPPORTED, "The pipelined staged two-shot needs 16-byte aligned buffers of whole 16-byte wire vectors.\n");
    int ch = channels > 0 ? channels : ChooseChannels(Algo::kDirect, n * wsize, m.ws, kMaxChannels);
    ch = std::max(1, std::min(std::min(ch, 128), std::max(1, m.staged_max_blocks / m.ws)));
    if (split) ch = std::max(1, std::min(ch, m.staged_max_blocks / m.ws / 2));
    std::vector<StagedParams> ps(static_cast<size_t>(m.ws));
    for (int r = 0; r < m.ws; ++r) {
      StagedParams& p = ps[static_cast<size_t>(r)];
      memset(&p, 0, sizeof(p));
      const RankResources& rr = m.ranks[static_cast<size_t>(r)];
      p.rank = r;
      p.world_size = m.ws;
      p.dtype = static_cast<int32_t>(dtype);
      p.wire = static_cast<int32_t>(wire);
      p.use_multimem = 0;
      p.use_tma = (wire == dtype && Tunable("IBCOMM_STAGED_TMA", 1) != 0) ? 1 : 0;
      p.peers = rr.peers;
      p.sendbuf = sendbufs[static_cast<size_t>(r)];
      p.recvbuf = recvbufs[static_cast<size_t>(r)];
      p.len_elements = n;
      p.scale = scale;
      p.window_elems = TwoShotWindowElems(n, quarter / wsize, wsize, m.ws, ch);
      p.buffers = buffers;
      p.split_ctas = split ? 1 : 0;
      p.load_groups = std::max(1, std::min(Tunable("IBCOMM_STAGED_LOAD_GROUPS", 1), 4));
      p.reduce_groups = std::max(1, std::min(Tunable("IBCOMM_STAGED_REDUCE_GROUPS", 2), 4));
      p.store_groups = std::max(1, std::min(Tunable("IBCOMM_STAGED_STORE_GROUPS", 1), 4));
      p.posters = Tunable("IBCOMM_STAGED_POSTERS", 0) != 0 ? 1 : 0;
      for (int q = 0; q < m.ws; ++q) p.stage[q] = rr.peers.arena[q];
      p.mc_stage = nullptr;
      for (int j = 0; j < buffers; ++j) {
        p.in_off[j] = m.layout.pool_offset + static_cast<uint64_t>(j) * quarter;
        p.out_off[j] = m.layout.pool_offset + static_cast<uint64_t>(buffers + j) * quarter;
      }
      p.timeout_ns = timeout_ns;
      p.status = rr.d_status;
      p.doorbell = rr.d_doorbell;
      if (r == m.silent_rank) p.len_elements = 0;  // takes no part: no window, no flag
    }
    void* d = m.Params(ps.size() * sizeof(StagedParams));
    CUDACHECK(cudaMemcpyAsync(d, ps.data(), ps.size() * sizeof(StagedParams), cudaMemcpyHostToDevice, stream));
    CUDACHECK(LaunchStagedKernel(ps[0], static_cast<const StagedParams*>(d), m.ws, split ? 2 * ch : ch, stream));
    m.last_channels = ch;
  } else if (algo == Algo::kDirect) {
    // The two-shot kernel with peer loads and stores.  All ranks' buffers live
    // on this GPU, so they can be used in place; with `direct_staging` they
    // go through the pool windows like buffers the peers cannot map.
    const uint64_t half = m.layout.pool_bytes / 2 / 4096 * 4096;
    int ch = channels > 0 ? channels : ChooseChannels(Algo::kDirect, bytes, m.ws, kMaxChannels);
    ch = std::min(ch, cap);
    std::vector<NvlsParams> ps(static_cast<size_t>(m.ws));
    for (int r = 0; r < m.ws; ++r) {
      NvlsParams& p = ps[static_cast<size_t>(r)];
      memset(&p, 0, sizeof(p));
      const RankResources& rr = m.ranks[static_cast<size_t>(r)];
      p.rank = r;
      p.world_size = m.ws;
      p.dtype = static_cast<int32_t>(dtype);
      p.use_multimem = 0;
      p.peers = rr.peers;
      p.sendbuf = sendbufs[static_cast<size_t>(r)];
      p.recvbuf = recvbufs[static_cast<size_t>(r)];
      p.len_elements = n;
      p.scale = scale;
      p.timeout_ns = timeout_ns;
      p.status = rr.d_status;
      p.doorbell = rr.d_doorbell;
      bool aligned = true;
      for (int q = 0; q < m.ws; ++q)
        aligned = aligned && ((reinterpret_cast<uintptr_t>(sendbufs[static_cast<size_t>(q)]) | reinterpret_cast<uintptr_t>(recvbufs[static_cast<size_t>(q)])) & 15u) == 0;
      const bool staged = m.direct_staging != 0 || !aligned;
      if (staged && half < 8192)
        IBCOMM_FAIL(NOT_SUPPORTED, "Two-shot allreduce through the pool needs a pool of at least 16 KiB.\n");
      p.stage_in = staged ? 1 : 0;
      p.stage_out = staged ? 1 : 0;
      for (int q = 0; q < m.ws; ++q) {
        if (staged) {
          p.peer_in[q] = rr.peers.arena[q] + m.layout.pool_offset;
          p.peer_out[q] = rr.peers.arena[q] + m.layout.pool_offset + half;
        } else {
          p.peer_in[q] = static_cast<unsigned char*>(const_cast<void*>(sendbufs[static_cast<size_t>(q)]));
          p.peer_out[q] = static_cast<unsigned char*>(recvbufs[static_cast<size_t>(q)]);
        }
      }
      p.local_in = p.peer_in[r];
      p.local_out = p.peer_out[r];
      p.window_elems = staged ? TwoShotWindowElems(n, (half - 4096) / esize, esize, m.ws, ch) : std::max<uint64_t>(1, n);
      p.tail_in_off = half - 4096;  // the ragged end of a staged message lives past every window
    }
    void* d = m.Params(ps.size() * sizeof(NvlsParams));
    CUDACHECK(cudaMemcpyAsync(d, ps.data(), ps.size() * sizeof(NvlsParams), cudaMemcpyHostToDevice, stream));
    CUDACHECK(LaunchNvlsKernel(ps[0], static_cast<const NvlsParams*>(d), m.ws, ch, stream));
    m.last_channels = ch;
  } else if (algo == Algo::kOneShot) {
    if (bytes > m.layout.oneshot_slot_bytes)
      IBCOMM_FAIL(INVALID_ARGUMENT, "One-shot allreduce handles at most %llu bytes (got %zu).\n",
                  static_cast<unsigned long long>(m.layout.oneshot_slot_bytes), bytes);
    std::vector<OneShotParams> ps;
    for (int r = 0; r < m.ws; ++r)
      ps.push_back(MakeOneShotParams(m.ranks[static_cast<size_t>(r)], dtype, sendbufs[static_cast<size_t>(r)],
                                     recvbufs[static_cast<size_t>(r)], n, scale, timeout_ns));
    int ch = channels > 0 ? channels : ChooseChannels(Algo::kOneShot, bytes, m.ws, kMaxChannels);
    ch = std::min(ch, cap);
    void* d = m.Params(ps.size() * sizeof(OneShotParams));
    CUDACHECK(cudaMemcpyAsync(d, ps.data(), ps.size() * sizeof(OneShotParams), cudaMemcpyHostToDevice, stream));
    CUDACHECK(LaunchOneShotKernel(ps[0], static_cast<const OneShotParams*>(d), m.ws, ch, stream));
    m.last_channels = ch;
  } else {
    // Validation (length, chunk size) happens while the first program is cut.
    std::vector<ExecParams> ps;
    for (int r = 0; r < m.ws; ++r) {
      const CachedProgram& cp = m.cache.Get(algo, r, m.ws, n, dtype, wire, m.layout, scale != 1.0, stream, false);
      ps.push_back(MakeExecParams(m.ranks[static_cast<size_t>(r)], cp, dtype, wire, sendbufs[static_cast<size_t>(r)],
                                  recvbufs[static_cast<size_t>(r)], n, scale, timeout_ns, nullptr, 0));
      if (r == m.silent_rank) ps.back().num_ops = 0;
      if (r == m.bad_program_rank) ps.back().len_elements = 1;
    }
    int ch = channels > 0 ? channels : ChooseChannels(algo, bytes, m.ws, kMaxChannels);
    ch = std::min(ch, cap);
    void* d = m.Params(ps.size() * sizeof(ExecParams));
    CUDACHECK(cudaMemcpyAsync(d, ps.data(), ps.size() * sizeof(ExecParams), cudaMemcpyHostToDevice, stream));
    CUDACHECK(LaunchExecKernel(ps[0], static_cast<const ExecParams*>(d), m.ws, ch, stream));
    m.last_channels = ch;
  }
  if (async) return;
  CUDACHECK(cudaStreamSynchronize(stream));
  m.cache.NoteSynchronized();
  for (int r = 0; r < m.ws; ++r) {
    DeviceStatus st;
    uint32_t code = m.status[static_cast<size_t>(r)].Consume(&st, stream);
    // The report of the rank that found the problem beats "aborted by a peer".
    if (code != 0 && (m.last_status == 0 || (m.last_status == kStatusPeerAbort && code != kStatusPeerAbort))) {
      m.last_status = code;
      m.last_report = st;
    }
  }
  if (m.last_status != 0) IBCOMM_FAIL(TRANSPORT_ERROR, "%s\n", DescribeStatus(m.last_report).c_str());
}

void EmuWorld::ReduceScatterOrAllGather(bool all_gather, DType dtype, const std::vector<const void*>& sendbufs,
                                        const std::vector<void*>& recvbufs, size_t block_elems, double scale, int channels,
                                        void* stream_v, bool async) {
  Impl& m = *impl_;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (static_cast<int>(sendbufs.size()) != m.ws || static_cast<int>(recvbufs.size()) != m.ws)
    IBCOMM_FAIL(INVALID_ARGUMENT, "EmuWorld::ReduceScatterOrAllGather needs one buffer pair per rank.\n");
  if (block_elems == 0) IBCOMM_FAIL(NOT_SUPPORTED, "EmuWorld::ReduceScatterOrAllGather: empty block.\n");
  const size_t esize = DTypeSize(dtype);
  const size_t block_bytes = block_elems * esize;
  m.last_status = 0;
  if (m.ws == 1) {
    CopyParams cp{sendbufs[0], recvbufs[0], block_elems, static_cast<int32_t>(dtype), static_cast<int32_t>(dtype), all_gather ? 1.0 : scale};
    CUDACHECK(LaunchCopyKernel(cp, kCopyDefaultBlocks, stream));
    if (!async) CUDACHECK(cudaStreamSynchronize(stream));
    return;
  }
  const bool vec = block_bytes % 16 == 0;
  bool aligned = vec;
  for (int q = 0; q < m.ws; ++q) {
    const void* remote = all_gather ? recvbufs[static_cast<size_t>(q)] : sendbufs[static_cast<size_t>(q)];
    aligned = aligned && (reinterpret_cast<uintptr_t>(remote) & 15u) == 0;
  }
  const bool staged = m.direct_staging != 0 || !aligned;
  const uint64_t sub = m.layout.pool_bytes / static_cast<uint64_t>(m.ws) / 4096 * 4096;
  if (staged && sub < 4096) IBCOMM_FAIL(NOT_SUPPORTED, "Reduce-scatter / all-gather through the pool need a larger pool.\n");
  const int cap = std::max(1, m.max_blocks / m.ws);
  int ch = channels > 0 ? channels : ChooseChannels(Algo::kDirect, block_bytes * static_cast<size_t>(m.ws), m.ws, kMaxChannels);
  ch = std::min(ch, cap);
  std::vector<RsAgParams> ps(static_cast<size_t>(m.ws));
  for (int r = 0; r < m.ws; ++r) {
    RsAgParams& p = ps[static_cast<size_t>(r)];
    memset(&p, 0, sizeof(p));
    const RankResources& rr = m.ranks[static_cast<size_t>(r)];
    p.rank = r;
    p.world_size = m.ws;
    p.dtype = static_cast<int32_t>(dtype);
    p.mode = all_gather ? kRsAgAllGather : kRsAgReduceScatter;
    p.staged = staged ? 1 : 0;
    p.peers = rr.peers;
    p.sendbuf = sendbufs[static_cast<size_t>(r)];
    p.recvbuf = recvbufs[static_cast<size_t>(r)];
    p.block_elems = block_elems;
    p.scale = all_gather ? 1.0 : scale;
    p.timeout_ns = static_cast<uint64_t>(m.timeout_ms) * 1000000ull;
    p.status = rr.d_status;
    p.doorbell = rr.d_doorbell;
    for (int q = 0; q < m.ws; ++q) {
      if (staged) {
        p.peer_buf[q] = rr.peers.arena[q] + m.layout.pool_offset;
      } else {
        p.peer_buf[q] = all_gather ? static_cast<unsigned char*>(recvbufs[static_cast<size_t>(q)])
                                   : static_cast<unsigned char*>(const_cast<void*>(sendbufs[static_cast<size_t>(q)]));
      }
    }
    if (staged) {
      p.sub_stride_bytes = sub;
      p.window_elems = TwoShotWindowElems(block_elems, sub / esize, esize, 1, ch);
      if (!vec) p.window_elems = std::min<uint64_t>(std::max<uint64_t>(p.window_elems, 1), sub / esize);
    } else {
      p.sub_stride_bytes = block_bytes;
      p.window_elems = block_elems;
    }
  }
  void* d = m.Params(ps.size() * sizeof(RsAgParams));
  CUDACHECK(cudaMemcpyAsync(d, ps.data(), ps.size() * sizeof(RsAgParams), cudaMemcpyHostToDevice, stream));
  CUDACHECK(LaunchRsAgKernel(ps[0], static_cast<const RsAgParams*>(d), m.ws, ch, stream));
  m.last_channels = ch;
  if (async) return;
  CUDACHECK(cudaStreamSynchronize(stream));
  for (int r = 0; r < m.ws; ++r) {
    DeviceStatus st;
    uint32_t code = m.status[static_cast<size_t>(r)].Consume(&st, stream);
    if (code != 0 && (m.last_status == 0 || (m.last_status == kStatusPeerAbort && code != kStatusPeerAbort))) {
      m.last_status = code;
      m.last_report = st;
    }
  }
  if (m.last_status != 0) IBCOMM_FAIL(TRANSPORT_ERROR, "%s\n", DescribeStatus(m.last_report).c_str());
}

void EmuWorld::AllreduceHostBuffers(Algo algo, DType dtype, const std::vector<const void*>& in, const std::vector<void*>& out,
                                    size_t n) {
  const size_t bytes = n * DTypeSize(dtype);
  std::vector<void*> d_in(in.size(), nullptr), d_out(out.size(), nullptr);
  std::vector<const void*> d_in_c;
  for (size_t r = 0; r < in.size(); ++r) {
    CUDACHECK(cudaMalloc(&d_in[r], std::max<size_t>(bytes, 16)));
    CUDACHECK(cudaMalloc(&d_out[r], std::max<size_t>(bytes, 16)));
    CUDACHECK(cudaMemcpy(d_in[r], in[r], bytes, cudaMemcpyHostToDevice));
    d_in_c.push_back(d_in[r]);
  }
  Allreduce(algo, dtype, d_in_c, d_out, n);
  for (size_t r = 0; r < in.size(); ++r) {
    CUDACHECK(cudaMemcpy(out[r], d_out[r], bytes, cudaMemcpyDeviceToHost));
    CUDACHECK(cudaFree(d_in[r]));
    CUDACHECK(cudaFree(d_out[r]));
  }
}

}  // namespace ibcomm
