// DeviceContext: the device half of a communicator.
#include "ibcomm/device_context.h"

#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>

#include "arena.h"
#include "driver_api.h"
#include "engine.h"
#include "fd_channel.h"
#include "ibcomm/tunables.h"

namespace ibcomm {

namespace {

// First message between two ranks on the device path.
struct Hello {
  ShareTicket ticket;
  int32_t multicast_ok;
  int32_t device;
  uint64_t arena_bytes;
  uint64_t pool_bytes;
  uint64_t work_bytes;
};

struct SymmetricAlloc {
  std::unique_ptr<SharedAllocation> mine;
  std::vector<std::unique_ptr<SharedAllocation>> imported;  // by rank (null for me)
  std::unique_ptr<MulticastGroup> mc;
  unsigned char* peer_ptr[kMaxRanks] = {nullptr};
  size_t bytes = 0;
};

// A user buffer (any cudaMalloc'ed memory, e.g. a tensor of a framework's
// caching allocator) that the peers have mapped through CUDA IPC.
struct RegisteredBuffer {
  int id = -1;
  unsigned char* ptr = nullptr;
  size_t bytes = 0;
  unsigned char* peer_ptr[kMaxRanks] = {nullptr};
  unsigned long long peer_alloc[kMaxRanks] = {0};  // key of the peer's imported allocation
  // With NVSwitch multicast: the granules around the buffer are bound to a
  // multicast object of their own (every rank's at offset 0), so the switch
  // kernels reduce and broadcast the buffer in place.  `mc_ptr` is the
  // multicast alias of `ptr`.
  std::shared_ptr<MulticastGroup> mc;
  unsigned char* mc_ptr = nullptr;
};

// What the ranks tell each other before binding a registered buffer to a multicast object.
struct RegisterMcMsg {
  int32_t ok;
  int32_t pad_;
  uint64_t inner;  // offset of the buffer inside its first granule
  uint64_t span;   // bytes of the granules that cover it
};

// One peer allocation opened with cudaIpcOpenMemHandle.  A process may open a
// given allocation only once, so registrations inside the same allocation
// share the mapping.
struct ImportedIpc {
  int peer = -1;
  unsigned long long alloc_id = 0;  // the exporter's CU_POINTER_ATTRIBUTE_BUFFER_ID
  void* base = nullptr;
  int refs = 0;
};

// What the ranks tell each other about a buffer they register.
struct RegisterMsg {
  cudaIpcMemHandle_t handle;
  uint64_t offset;    // of the buffer inside the allocation
  uint64_t bytes;
  uint64_t alloc_id;
  int32_t ok;
  int32_t pid;
};

// NVTX range around a host call (shows up in timeline tools next to the
// kernels; costs a few nanoseconds when no tool is attached).
class NvtxRange {
 public:
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

struct LoopbackSend {
  const void* buf;
  size_t len;
};

// Identity of one device message for the abort protocol: the same on the
// sending and the receiving side, different for every message of every ordered
// pair, and outside the range of the collectives' call numbers.  (A constant
// per rank would make one timed-out message poison every later one: the abort
// word keeps the last value written to it.)
uint64_t P2pSeq(int src, int dst, uint64_t first_piece) {
  return 0xFF00000000000000ull | (static_cast<uint64_t>(src) << 52) | (static_cast<uint64_t>(dst) << 48) |
         (first_piece & 0xFFFFFFFFFFFFull);
}

// Share of a zero-copy switch allreduce that the hybrid kernel runs through
// the direct algorithm, in percent (0 = plain switch kernel), when
// IBCOMM_NVLS_HYBRID does not say.  Off until a sweep on the machine shows a
// gain; see the tuning notes of the hybrid kernel.
int HybridDefaultPercent(int world_size, size_t bytes) {
  (void)world_size;
  (void)bytes;
  return 0;
}

}  // namespace

class DeviceContext {
 public:
  explicit DeviceContext(Communicator* comm);
  ~DeviceContext();

  void ConnectPeers();
  void Allreduce(DType dtype, const void* sendbuf, void* recvbuf, size_t n, const CudaAllreduceOptions& opts);
  // mode: kRsAgReduceScatter or kRsAgAllGather; `block_elems` per rank.
  void ReduceScatterOrAllGather(int mode, DType dtype, const void* sendbuf, void* recvbuf, size_t block_elems,
                                const CudaAllreduceOptions& opts);
  void Check();
  uint32_t Peek(DeviceStatus* out);

  bool Bcast(void* buf, size_t len, int root);
  void Send(int dest, const void* buf, size_t len);
  void Recv(int src, void* buf, size_t len);
  bool SendPoll(int dest);
  bool RecvPoll(int src);
  void SendWait(int dest);
  void RecvWait(int src);

  void* SymmetricAlloc_(size_t bytes);
  void SymmetricFree_(void* ptr);
  int RegisterBuffer(void* ptr, size_t bytes);
  void DeregisterBuffer(int id);
  void CollectTrace(Tracer* tracer);
  const std::vector<uint64_t>& StagedTimeline() const { return staged_timeline_; }
  DeviceInfo Info() const;
  void SetMaxChannels(int c) { max_channels_ = c > 0 ? std::min(c, kMaxChannels) : std::min(env::ReadNumCudaStream(), kMaxChannels); }

 private:
  struct P2pState {
    cudaEvent_t send_done = nullptr, recv_done = nullptr;
    uint64_t pieces_sent = 0, pieces_received = 0;
    std::deque<LoopbackSend> loopback;  // same-device sends waiting for their receive
    bool loopback_send_complete = false;
  };

  cudaStream_t StreamFor(const CudaAllreduceOptions& opts);
  void OrderAfterPrevious(cudaStream_t stream);
  void MarkIssued(cudaStream_t stream);
  void Finish(cudaStream_t stream, bool async);
  bool IsLoopback(int peer) const;
  const SymmetricAlloc* FindSymmetric(const void* p, size_t bytes) const;
  // Peer pointers of a buffer every rank has mapped (symmetric memory or a
  // registered buffer); false when the buffer is neither.
  bool FindPeerMapped(const void* p, size_t bytes, unsigned char** peer_ptr) const;
  void BindRegisteredToSwitch(RegisteredBuffer* reg);
  unsigned char* FindRegisteredMulticast(const void* p, size_t bytes) const;
  template <typename M> void ExchangeWithAll(const M& mine, std::vector<M>* all);

  void RunCopy(DType dtype, const void* sendbuf, void* recvbuf, size_t n, double scale, cudaStream_t stream);
  void RunProgram(Algo algo, DType dtype, DType wire, const void* sendbuf, void* recvbuf, size_t n, double scale, int channels,
                  cudaStream_t stream);
  void RunOneShot(DType dtype, const void* sendbuf, void* recvbuf, size_t n, double scale, int channels, cudaStream_t stream);
  void RunTwoShot(bool multimem, DType dtype, DType wire, const void* sendbuf, void* recvbuf, size_t n, double scale, int channels,
                  cudaStream_t stream);
  // The pipelined kernel for buffers that go through the pool; false when the
  // call does not meet its requirements (nothing has been launched then).
  bool RunStaged(bool multimem, DType dtype, DType wire, const void* sendbuf, void* recvbuf, size_t n, double scale, int channels,
                 cudaStream_t stream);
  // Caps a collective's CTAs at what the GPU holds at once (CTA b of this rank
  // waits for CTA b of the peers) and at IBCOMM_MAX_CTAS when set (a program
  // that overlaps collectives with compute leaves SMs to the compute).
  int ClampChannels(Algo algo, int channels, size_t bytes = 0);
  int sm_count_ = -1;  // looked up on first use
  bool switch_bind_refused_ = false;  // some rank's driver refused to bind a registered buffer to the switch
  // Begins a device trace record of `records` entries per channel (no-op when tracing is off).
  DeviceTraceRec* BeginDeviceTrace(int channels, int records, int* capacity);
  void ExchangeAllocation(SharedAllocation* mine, std::vector<std::unique_ptr<SharedAllocation>>* imported,
                          unsigned char** peer_ptr, bool try_multicast, std::unique_ptr<MulticastGroup>* mc);

  Communicator* comm_;
  int device_ = 0;
  int rank_ = 0, ws_ = 1;
  cudaStream_t stream_ = nullptr;
  // Send and receive kernels of one rank must be able to run side by side
  // (each waits for a kernel on ANOTHER GPU), hence one stream per direction.
  cudaStream_t send_stream_ = nullptr, recv_stream_ = nullptr;
  cudaEvent_t last_done_ = nullptr;
  cudaStream_t last_stream_ = nullptr;
  bool have_last_ = false;
  ArenaLayout layout_;
  SharedAllocation arena_;
  std::vector<std::unique_ptr<SharedAllocation>> peer_arenas_;
  std::unique_ptr<MulticastGroup> mc_;
  std::vector<std::unique_ptr<FdChannel>> fdch_;
  bool connected_ = false;
  bool multicast_local_ok_ = false;
  RankResources rr_;
  StatusBlock status_;
  ProgramCache cache_;
  uint64_t calls_ = 0;
  uint64_t kernel_launches_ = 0;
  int last_algo_ = 0, last_channels_ = 0;
  int hybrid_channels_ = 0;  // CTAs of the hybrid two-shot kernel when the last call ran it
  int staged_channels_ = 0;  // CTAs of the pipelined staged kernel when the last call ran it
  std::map<int, int> exec_resident_;  // executor CTA size -> co-resident CTAs on this device
  int twoshot_resident_ = -1;
  int max_channels_ = env::kDefaultNumCudaStream;
  std::vector<P2pState> p2p_;
  int p2p_ctas_ = 96;          // CTAs of every Send / Recv / Bcast kernel of this communicator (knob IBCOMM_P2P_CTAS)
  uint64_t bcast_pieces_ = 0;  // pieces of all device broadcasts so far (equal on every rank)
  std::vector<std::unique_ptr<SymmetricAlloc>> symm_;
  std::unique_ptr<SymmetricAlloc> grown_stage_;  // staging block for large messages through the pool (allocated on demand)
  std::vector<RegisteredBuffer> registered_;
  std::vector<ImportedIpc> ipc_imports_;
  int next_registration_ = 0;
  // tracing
  DeviceTraceRec* d_trace_ = nullptr;
  int trace_capacity_ = 0;
  int trace_channels_ = 0;
  struct PendingTrace {
    int channels;
    int ops;
    int roles = 0;  // staged kernel: the other roles' stamps follow in three more ranges of `roles` records
    struct timespec host_launch;
  };
  std::vector<uint64_t> staged_timeline_;  // last traced staged call, CTA 0: 4 x windows x (t_wait_done, t_done), ns from the first stamp
  std::deque<PendingTrace> pending_trace_;
  std::vector<std::pair<double, double>> trace_wait_, trace_done_;  // (start_ns, dur_ns) relative to base
  Tracer* tracer_ = nullptr;
};

// ------------------------------------------------------------------ set-up
DeviceContext::DeviceContext(Communicator* comm) : comm_(comm) {
  CUDACHECK(cudaGetDevice(&device_));
  rank_ = comm->rank() < 0 ? 0 : comm->rank();
  ws_ = static_cast<int>(comm->world_size());
  if (ws_ > kMaxRanks) IBCOMM_FAIL(NOT_SUPPORTED, "Device collectives support up to %d ranks (got %d).\n", kMaxRanks, ws_);
  max_channels_ = std::min(env::ReadNumCudaStream(), kMaxChannels);
  p2p_ctas_ = Tunable("IBCOMM_P2P_CTAS", 96);
  if (p2p_ctas_ < 1 || p2p_ctas_ > kP2pCtas) p2p_ctas_ = 96;
  layout_ = MakeArenaLayout(env::ReadPreAllocSize(), env::ReadWorkGpuMemorySize(), ws_);
  // A blocking stream: work the caller queued on the legacy default stream is
  // ordered before the collectives issued here, and vice versa.
  CUDACHECK(cudaStreamCreateWithFlags(&stream_, cudaStreamDefault));
  CUDACHECK(cudaStreamCreateWithFlags(&send_stream_, cudaStreamDefault));
  CUDACHECK(cudaStreamCreateWithFlags(&recv_stream_, cudaStreamDefault));
  CUDACHECK(cudaEventCreateWithFlags(&last_done_, cudaEventDisableTiming));
  multicast_local_ok_ = !env::ReadDisableNvls() && ws_ > 1 && MulticastGroup::Supported(device_);
  size_t align = 0;
  if (multicast_local_ok_) align = MulticastGroup::Granularity(ws_, layout_.total_bytes);
  arena_.Create(layout_.total_bytes, device_, align);
  status_.Create();
  rr_.rank = rank_;
  rr_.world_size = ws_;
  rr_.layout = layout_;
  rr_.peers.arena[rank_] = arena_.ptr();
  rr_.d_status = status_.d_status;
  rr_.h_doorbell = status_.h_doorbell;
  rr_.d_doorbell = status_.d_doorbell;
  p2p_.resize(static_cast<size_t>(ws_));
  peer_arenas_.resize(static_cast<size_t>(ws_));
  fdch_.resize(static_cast<size_t>(ws_));
  tracer_ = &comm->tracer();
  if (tracer_->enabled()) {
    trace_capacity_ = 512;
    trace_channels_ = max_channels_;
    CUDACHECK(cudaMalloc(&d_trace_, sizeof(DeviceTraceRec) * static_cast<size_t>(trace_capacity_) * static_cast<size_t>(trace_channels_)));
  }
}

DeviceContext::~DeviceContext() {
  cudaDeviceSynchronize();
  for (P2pState& s : p2p_) {
    if (s.send_done) cudaEventDestroy(s.send_done);
    if (s.recv_done) cudaEventDestroy(s.recv_done);
  }
  cache_.Clear();
  for (ImportedIpc& imp : ipc_imports_) cudaIpcCloseMemHandle(imp.base);
  ipc_imports_.clear();
  registered_.clear();
  grown_stage_.reset();
  symm_.clear();
  mc_.reset();
  peer_arenas_.clear();
  arena_.Release();
  status_.Destroy();
  if (d_trace_) cudaFree(d_trace_);
  if (last_done_) cudaEventDestroy(last_done_);
  if (stream_) cudaStreamDestroy(stream_);
  if (send_stream_) cudaStreamDestroy(send_stream_);
  if (recv_stream_) cudaStreamDestroy(recv_stream_);
  (void)cudaGetLastError();
}

bool DeviceContext::IsLoopback(int peer) const {
  // A queue pair whose other end lives in this very communicator (the
  // single-process self-connection used by the transport smoke test).
  const auto& ep = comm_->eps_[static_cast<size_t>(peer)];
  if (!ep.connected) return false;
  if (ep.peer_info.qp_n != static_cast<uint32_t>(getpid())) return false;
  for (const auto& other : comm_->eps_)
    if (other.created && other.my_info.psn == ep.peer_info.psn && other.my_info.qp_n == ep.peer_info.qp_n) return true;
  return false;
}

void DeviceContext::ExchangeAllocation(SharedAllocation* mine, std::vector<std::unique_ptr<SharedAllocation>>* imported,
                                       unsigned char** peer_ptr, bool try_multicast, std::unique_ptr<MulticastGroup>* mc) {
  const int timeout = std::max(comm_->timeout_ms(), 30000);
  // Tickets over the host transport.
  Hello mine_hello;
  memset(&mine_hello, 0, sizeof(mine_hello));
  mine_hello.ticket = mine->Ticket();
  mine_hello.multicast_ok = (try_multicast && multicast_local_ok_ && mine->mode() == ShareMode::kVmm) ? 1 : 0;
  mine_hello.device = device_;
  mine_hello.arena_bytes = mine->bytes();
  mine_hello.pool_bytes = layout_.pool_bytes;
  mine_hello.work_bytes = layout_.work_bytes;
  std::vector<Hello> hellos(static_cast<size_t>(ws_));
  for (int q = 0; q < ws_; ++q) {
    if (q == rank_) continue;
    comm_->PostSend(q, &mine_hello, sizeof(Hello));
    comm_->PostRecv(q, &hellos[static_cast<size_t>(q)], sizeof(Hello));
  }
  for (int q = 0; q < ws_; ++q) {
    if (q == rank_) continue;
    comm_->WaitRecvCompletion(q);
    --comm_->eps_[static_cast<size_t>(q)].recv_completions;
    comm_->WaitSendCompletion(q);
    --comm_->eps_[static_cast<size_t>(q)].send_completions;
  }
  bool all_mc = mine_hello.multicast_ok != 0;
  for (int q = 0; q < ws_; ++q) {
    if (q == rank_) continue;
    const Hello& h = hellos[static_cast<size_t>(q)];
    if (h.arena_bytes != mine->bytes() || h.pool_bytes != layout_.pool_bytes || h.work_bytes != layout_.work_bytes)
      IBCOMM_FAIL(INVALID_ARGUMENT,
                  "Rank %d uses a different arena geometry (%llu bytes vs %zu): IBCOMM_MEMORY_POOL_PRE_ALLOC and "
                  "IBCOMM_WORK_GPU_MEMORY_SIZE must agree on all ranks.\n",
                  q, static_cast<unsigned long long>(h.arena_bytes), mine->bytes());
    all_mc = all_mc && h.multicast_ok != 0;
  }
  // Descriptors over the per-pair unix sockets.
  int my_fd_mode = mine->mode() == ShareMode::kVmm ? 1 : 0;
  imported->clear();
  imported->resize(static_cast<size_t>(ws_));
  for (int q = 0; q < ws_; ++q) {
    if (q == rank_) continue;
    int sent_fd = -1;
    if (my_fd_mode) sent_fd = mine->ExportFd();
    int token = my_fd_mode;
    fdch_[static_cast<size_t>(q)]->Send(&token, sizeof(token), sent_fd);
    if (sent_fd >= 0) close(sent_fd);
  }
  for (int q = 0; q < ws_; ++q) {
    if (q == rank_) continue;
    int token = 0;
    int fd = fdch_[static_cast<size_t>(q)]->Recv(&token, sizeof(token), timeout);
    std::unique_ptr<SharedAllocation> imp(new SharedAllocation());
    imp->Import(hellos[static_cast<size_t>(q)].ticket, fd, device_);
    peer_ptr[q] = imp->ptr();
    (*imported)[static_cast<size_t>(q)] = std::move(imp);
  }
  peer_ptr[rank_] = mine->ptr();
  comm_->Barrier();

  // Multicast object: rank 0 creates, everybody adds its device, then binds.
  mc->reset();
  if (!all_mc) return;
  int ok = 1;
  std::unique_ptr<MulticastGroup> group(new MulticastGroup());
  if (rank_ == 0) {
    // The same descriptor is handed to every peer (each receives its own duplicate).
    int fd = group->CreateRoot(mine->bytes(), ws_);
    if (fd < 0) ok = 0;
    for (int q = 1; q < ws_; ++q) fdch_[static_cast<size_t>(q)]->Send(&ok, sizeof(ok), fd);
    if (fd >= 0) close(fd);
  } else {
    int fd = fdch_[0]->Recv(&ok, sizeof(ok), timeout);
    if (ok) group->Import(fd, mine->bytes(), ws_);
  }
  if (!ok) {
    comm_->Barrier();
    return;
  }
  group->AddDevice(device_);
  comm_->Barrier();
  group->BindAndMap(*mine, device_);
  comm_->Barrier();
  *mc = std::move(group);
}

void DeviceContext::ConnectPeers() {
  if (connected_) return;
  NvtxRange nvtx("ibcomm::ConnectPeers");
  rank_ = comm_->rank();
  if (rank_ < 0) IBCOMM_FAIL(INVALID_ARGUMENT, "Device collectives need RegisterMyself first.\n");
  rr_.rank = rank_;
  rr_.peers.arena[rank_] = arena_.ptr();
  if (ws_ > 1) {
    const int timeout = std::max(comm_->timeout_ms(), 30000);
    // One stream socket per pair: the lower rank listens on the name of its
    // endpoint for that peer, the higher rank connects to it.
    for (int q = 0; q < ws_; ++q) {
      if (q == rank_) continue;
      const auto& ep = comm_->eps_[static_cast<size_t>(q)];
      if (!ep.connected || !ep.created)
        IBCOMM_FAIL(INVALID_ARGUMENT, "Device collectives need a registered queue pair with every rank (rank %d is missing).\n", q);
      fdch_[static_cast<size_t>(q)].reset(new FdChannel());
      if (rank_ < q) fdch_[static_cast<size_t>(q)]->Listen(FdChannelName(ep.my_info.qp_n, ep.my_info.psn));
    }
    comm_->Barrier();
    for (int q = 0; q < ws_; ++q) {
      if (q == rank_) continue;
      const auto& ep = comm_->eps_[static_cast<size_t>(q)];
      if (rank_ > q) fdch_[static_cast<size_t>(q)]->Connect(FdChannelName(ep.peer_info.qp_n, ep.peer_info.psn), timeout);
    }
    for (int q = 0; q < ws_; ++q)
      if (q != rank_ && rank_ < q) fdch_[static_cast<size_t>(q)]->Accept(timeout);
    ExchangeAllocation(&arena_, &peer_arenas_, rr_.peers.arena, true, &mc_);
    rr_.peers.mc_arena = mc_ ? mc_->ptr() : nullptr;
  }
  connected_ = true;
}

// ---------------------------------------------------------------- streams
cudaStream_t DeviceContext::StreamFor(const CudaAllreduceOptions& opts) {
  return (opts.use_stream || opts.stream != nullptr) ? static_cast<cudaStream_t>(opts.stream) : stream_;
}

static bool IsCapturing(cudaStream_t stream) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return st != cudaStreamCaptureStatusNone;
}

void DeviceContext::OrderAfterPrevious(cudaStream_t stream) {
  // Collectives of one communicator reuse the same staging memory and flags:
  // the next one may only start when the previous one has finished, also when
  // the caller switches streams.  Inside a stream capture the graph's own
  // edges order the collectives; the caller keeps them on one stream.
  // No event is recorded per call (it would put a bubble between
  // back-to-back kernels); the rare switch of streams waits on the host.
  if (IsCapturing(stream)) return;
  if (have_last_ && last_stream_ != stream) CUDACHECK(cudaStreamSynchronize(last_stream_));
}

void DeviceContext::MarkIssued(cudaStream_t stream) {
  ++calls_;
  if (IsCapturing(stream)) return;
  last_stream_ = stream;
  have_last_ = true;
}

void DeviceContext::Finish(cudaStream_t stream, bool async) {
  if (async) return;
  CUDACHECK(cudaStreamSynchronize(stream));
  cache_.NoteSynchronized();
  Check();
}

uint32_t DeviceContext::Peek(DeviceStatus* out) { return status_.Consume(out, stream_); }

void DeviceContext::Check() {
  DeviceStatus st;
  uint32_t code = status_.Consume(&st, stream_);
  if (code != 0) IBCOMM_FAIL(TRANSPORT_ERROR, "%s\n", DescribeStatus(st).c_str());
}

// -------------------------------------------------------------- allreduce
const SymmetricAlloc* DeviceContext::FindSymmetric(const void* p, size_t bytes) const {
  const unsigned char* c = static_cast<const unsigned char*>(p);
  for (const auto& s : symm_)
    if (s && c >= s->mine->ptr() && c + bytes <= s->mine->ptr() + s->bytes) return s.get();
  return nullptr;
}

bool DeviceContext::FindPeerMapped(const void* p, size_t bytes, unsigned char** peer_ptr) const {
  const unsigned char* c = static_cast<const unsigned char*>(p);
  if (const SymmetricAlloc* s = FindSymmetric(p, bytes)) {
    const size_t off = static_cast<size_t>(c - s->mine->ptr());
    for (int q = 0; q < ws_; ++q) peer_ptr[q] = s->peer_ptr[q] + off;
    return true;
  }
  for (const RegisteredBuffer& r : registered_) {
    if (c >= r.ptr && c + bytes <= r.ptr + r.bytes) {
      const size_t off = static_cast<size_t>(c - r.ptr);
      for (int q = 0; q < ws_; ++q) peer_ptr[q] = r.peer_ptr[q] + off;
      return true;
    }
  }
  return false;
}

template <typename M>
void DeviceContext::ExchangeWithAll(const M& mine, std::vector<M>* all) {
  all->assign(static_cast<size_t>(ws_), mine);
  for (int q = 0; q < ws_; ++q) {
    if (q == rank_) continue;
    comm_->PostSend(q, &mine, sizeof(M));
    comm_->PostRecv(q, &(*all)[static_cast<size_t>(q)], sizeof(M));
  }
  for (int q = 0; q < ws_; ++q) {
    if (q == rank_) continue;
    comm_->WaitRecvCompletion(q);
    --comm_->eps_[static_cast<size_t>(q)].recv_completions;
    comm_->WaitSendCompletion(q);
    --comm_->eps_[static_cast<size_t>(q)].send_completions;
  }
}

// Collective.  Every rank passes its own buffer (the addresses and the
// positions inside the underlying allocations may differ, the sizes may
// not); afterwards two-shot collectives on the buffer, or on the same
// sub-range of it on every rank, load from and store into the peers' copies
// directly.  Returns -1, on every rank alike, when some rank's memory cannot
// be shared this way (not from cudaMalloc, e.g. a virtual-memory allocation,
// or a peer in the same process); such buffers keep going through the pool.
int DeviceContext::RegisterBuffer(void* ptr, size_t bytes) {
  if (ptr == nullptr || bytes == 0) IBCOMM_FAIL(INVALID_ARGUMENT, "RegisterBuffer: empty buffer.\n");
  NvtxRange nvtx("ibcomm::RegisterBuffer");
  ConnectPeers();
  RegisteredBuffer reg;
  reg.ptr = static_cast<unsigned char*>(ptr);
  reg.bytes = bytes;
  reg.peer_ptr[rank_] = reg.ptr;
  if (ws_ == 1) {
    reg.id = next_registration_++;
    registered_.push_back(reg);
    return reg.id;
  }
  RegisterMsg mine;
  memset(&mine, 0, sizeof(mine));
  mine.bytes = bytes;
  mine.pid = static_cast<int32_t>(getpid());
  const drv::Api* api = drv::Get();
  if (api != nullptr) {
    CUdeviceptr base = 0;
    size_t size = 0;
    unsigned long long alloc_id = 0;
    const CUdeviceptr p = reinterpret_cast<CUdeviceptr>(ptr);
    if (api->MemGetAddressRange(&base, &size, p) == CUDA_SUCCESS && p + bytes <= base + size &&
        api->PointerGetAttribute(&alloc_id, CU_POINTER_ATTRIBUTE_BUFFER_ID, p) == CUDA_SUCCESS &&
        cudaIpcGetMemHandle(&mine.handle, reinterpret_cast<void*>(base)) == cudaSuccess) {
      mine.offset = p - base;
      mine.alloc_id = alloc_id;
      mine.ok = 1;
    }
    (void)cudaGetLastError();
  }
  std::vector<RegisterMsg> all;
  ExchangeWithAll(mine, &all);
  bool ok = true;
  for (int q = 0; q < ws_; ++q) {
    const RegisterMsg& m = all[static_cast<size_t>(q)];
    ok = ok && m.ok != 0 && m.bytes == bytes && (q == rank_ || m.pid != mine.pid);
  }
  // Map the peers' allocations (once per allocation).
  std::vector<size_t> opened;  // entries of ipc_imports_ whose count this call raised
  if (ok) {
    for (int q = 0; q < ws_ && ok; ++q) {
      if (q == rank_) continue;
      const RegisterMsg& m = all[static_cast<size_t>(q)];
      size_t at = ipc_imports_.size();
      for (size_t i = 0; i < ipc_imports_.size(); ++i)
        if (ipc_imports_[i].peer == q && ipc_imports_[i].alloc_id == m.alloc_id) at = i;
      if (at == ipc_imports_.size()) {
        void* base = nullptr;
        if (cudaIpcOpenMemHandle(&base, m.handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
          (void)cudaGetLastError();
          ok = false;
          break;
        }
        ImportedIpc imp;
        imp.peer = q;
        imp.alloc_id = m.alloc_id;
        imp.base = base;
        ipc_imports_.push_back(imp);
      }
      ++ipc_imports_[at].refs;
      opened.push_back(at);
      reg.peer_ptr[q] = static_cast<unsigned char*>(ipc_imports_[at].base) + m.offset;
      reg.peer_alloc[q] = m.alloc_id;
    }
  }
  // Second round: all ranks mapped everything, or nobody keeps anything.
  int32_t mapped = ok ? 1 : 0;
  std::vector<int32_t> all_mapped;
  ExchangeWithAll(mapped, &all_mapped);
  for (int32_t v : all_mapped) ok = ok && v != 0;
  if (!ok) {
    for (size_t at : opened) --ipc_imports_[at].refs;
    for (size_t i = ipc_imports_.size(); i-- > 0;) {
      if (ipc_imports_[i].refs == 0) {
        (void)cudaIpcCloseMemHandle(ipc_imports_[i].base);
        ipc_imports_.erase(ipc_imports_.begin() + static_cast<long>(i));
      }
    }
    (void)cudaGetLastError();
    return -1;
  }
  BindRegisteredToSwitch(&reg);
  reg.id = next_registration_++;
  registered_.push_back(reg);
  return reg.id;
}

// Collective (part of RegisterBuffer).  Binds the granules around the buffer
// to a multicast object so that the switch kernels can work on it in place,
// as they do on symmetric memory.  Needs: multicast on this box, the driver's
// bind-by-address call, the buffer at the same offset inside its first
// granule on every rank, and the granules inside the buffer's allocation.
// Whatever is missing, on any rank, leaves the registration as it was
// (peer-mapped only) on every rank.
void DeviceContext::BindRegisteredToSwitch(RegisteredBuffer* reg) {
  // (all three conditions are the same on every rank; a refusal by the driver is remembered, because it is a
  // property of the driver and the allocator, not of the buffer)
  if (mc_ == nullptr || switch_bind_refused_ || Tunable("IBCOMM_REGISTER_SWITCH", 1) == 0) return;
  const drv::Api* api = drv::Get();
  RegisterMcMsg mine;
  memset(&mine, 0, sizeof(mine));
  const uintptr_t p = reinterpret_cast<uintptr_t>(reg->ptr);
  uintptr_t lo = 0;
  if (api != nullptr && api->MulticastBindAddr != nullptr) {
    size_t gran = MulticastGroup::Granularity(ws_, reg->bytes);
    CUdeviceptr base = 0;
    size_t size = 0;
    if (gran != 0 && api->MemGetAddressRange(&base, &size, static_cast<CUdeviceptr>(p)) == CUDA_SUCCESS) {
      lo = p / gran * gran;
      const uintptr_t hi = (p + reg->bytes + gran - 1) / gran * gran;
      if (lo >= base && hi <= base + size) {
        mine.ok = 1;
        mine.inner = p - lo;
        mine.span = hi - lo;
      }
    }
  }
  std::vector<RegisterMcMsg> all;
  ExchangeWithAll(mine, &all);
  for (const RegisterMcMsg& m : all)
    if (m.ok == 0 || m.inner != mine.inner || m.span != mine.span) return;
  const int timeout = std::max(comm_->timeout_ms(), 30000);
  int ok = 1;
  std::shared_ptr<MulticastGroup> group(new MulticastGroup());
  if (rank_ == 0) {
    int fd = group->CreateRoot(mine.span, ws_);
    if (fd < 0) ok = 0;
    for (int q = 1; q < ws_; ++q) fdch_[static_cast<size_t>(q)]->Send(&ok, sizeof(ok), fd);
    if (fd >= 0) close(fd);
  } else {
    int fd = fdch_[0]->Recv(&ok, sizeof(ok), timeout);
    if (ok) group->Import(fd, mine.span, ws_);
  }
  if (!ok) return;
  group->AddDevice(device_);
  comm_->Barrier();  // every device is in the object before anybody binds
  std::string why;
  int32_t bound = group->BindAddrAndMap(reinterpret_cast<void*>(lo), device_, &why) ? 1 : 0;
  std::vector<int32_t> all_bound;
  ExchangeWithAll(bound, &all_bound);
  bool everybody = true;
  for (int32_t v : all_bound) everybody = everybody && v != 0;
  if (!everybody) {
    static bool warned = false;
    if (!bound && !warned) {
      warned = true;
      IBCOMM_WARN("registered buffer stays peer-mapped only, the switch cannot be used on it in place (%s).\n", why.c_str());
    }
    group->Release();
    comm_->Barrier();
    switch_bind_refused_ = true;
    return;
  }
  reg->mc = group;
  reg->mc_ptr = group->ptr() + mine.inner;
}

// The multicast alias of [p, p + bytes) when it lies in a registered buffer that is bound to the switch.
unsigned char* DeviceContext::FindRegisteredMulticast(const void* p, size_t bytes) const {
  const unsigned char* c = static_cast<const unsigned char*>(p);
  for (const RegisteredBuffer& r : registered_)
    if (r.mc_ptr != nullptr && c >= r.ptr && c + bytes <= r.ptr + r.bytes) return r.mc_ptr + (c - r.ptr);
  return nullptr;
}

// Collective by contract: no rank may still run a collective on the buffer.
void DeviceContext::DeregisterBuffer(int id) {
  for (size_t i = 0; i < registered_.size(); ++i) {
    if (registered_[i].id != id) continue;
    CUDACHECK(cudaDeviceSynchronize());
    if (ws_ > 1) comm_->Barrier();  // the peers' kernels on this buffer are done, too
    RegisteredBuffer reg = registered_[i];
    registered_.erase(registered_.begin() + static_cast<long>(i));
    if (reg.mc) {
      reg.mc->Release();  // unmaps the alias and unbinds this rank's memory
      reg.mc.reset();
      if (ws_ > 1) comm_->Barrier();
    }
    for (int q = 0; q < ws_; ++q) {
      if (q == rank_ || reg.peer_ptr[q] == nullptr) continue;
      for (size_t k = 0; k < ipc_imports_.size(); ++k) {
        ImportedIpc& imp = ipc_imports_[k];
        if (imp.peer != q || imp.alloc_id != reg.peer_alloc[q]) continue;
        if (--imp.refs == 0) {
          CUDACHECK(cudaIpcCloseMemHandle(imp.base));
          ipc_imports_.erase(ipc_imports_.begin() + static_cast<long>(k));
        }
        break;
      }
    }
    return;
  }
  IBCOMM_FAIL(INVALID_ARGUMENT, "DeregisterBuffer: unknown registration %d.\n", id);
}

void DeviceContext::RunCopy(DType dtype, const void* sendbuf, void* recvbuf, size_t n, double scale, cudaStream_t stream) {
  if (sendbuf == recvbuf && scale == 1.0) return;
  CopyParams cp{sendbuf, recvbuf, n, static_cast<int32_t>(dtype), static_cast<int32_t>(dtype), scale};
  CUDACHECK(LaunchCopyKernel(cp, kCopyDefaultBlocks, stream));
  ++kernel_launches_;
}

void DeviceContext::RunProgram(Algo algo, DType dtype, DType wire, const void* sendbuf, void* recvbuf, size_t n, double scale,
                               int channels, cudaStream_t stream) {
  const CachedProgram& cp = cache_.Get(algo, rank_, ws_, n, dtype, wire, layout_, scale != 1.0, stream, IsCapturing(stream));
  int cap = 0;
  DeviceTraceRec* trace = BeginDeviceTrace(channels, static_cast<int>(cp.prog.ops.size()), &cap);
  ExecParams p = MakeExecParams(rr_, cp, dtype, wire, sendbuf, recvbuf, n, scale,
                                static_cast<uint64_t>(comm_->timeout_ms()) * 1000000ull, trace, cap);
  IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
  CUDACHECK(LaunchExecKernel(p, nullptr, 1, channels, stream));
  ++kernel_launches_;
  IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
}

void DeviceContext::RunOneShot(DType dtype, const void* sendbuf, void* recvbuf, size_t n, double scale, int channels,
                               cudaStream_t stream) {
  OneShotParams p = MakeOneShotParams(rr_, dtype, sendbuf, recvbuf, n, scale,
                                      static_cast<uint64_t>(comm_->timeout_ms()) * 1000000ull);
  IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
  CUDACHECK(LaunchOneShotKernel(p, nullptr, 1, channels, stream));
  ++kernel_launches_;
  IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
}

int DeviceContext::ClampChannels(Algo algo, int channels, size_t bytes) {
  int limit;
  if ((algo == Algo::kRing || algo == Algo::kRabenseifner) && (bytes < (256u << 20) || (algo == Algo::kRing && ws_ <= 2)) &&
      Tunable("IBCOMM_EXEC_CHANNELS", 0) <= 0) {
    // One 512-thread block per SM at most.  Beyond that the executor runs two
    // 256-thread blocks per SM, whose three data warps per op make a step
    // slower at medium sizes (two ranks, 16 and 64 MiB: 256 channels take 113-175
    // us where 64-148 take 72-82 and 134-150 us, ring and Rabenseifner alike;
    // 64 MiB ring on 3-6 ranks: 53-65 us per step with 170-256 channels against
    // 28-29 us on 7-8 ranks with 128-146).  From 256 MiB on both programs keep
    // 256 channels on more than two ranks (Rabenseifner 11 % ahead on 8 GPUs,
    // the ring 4 % on 8 and 8 % on 4); on two ranks the ring stays capped
    // (441 against 464 us).
    if (sm_count_ < 0 && cudaDeviceGetAttribute(&sm_count_, cudaDevAttrMultiProcessorCount, device_) != cudaSuccess) sm_count_ = 0;
    if (sm_count_ > 0) channels = std::min(channels, sm_count_);
  }
  if (algo == Algo::kRing || algo == Algo::kRabenseifner) {
    const int threads = ExecKernelThreadsFor(channels);
    auto it = exec_resident_.find(threads);
    if (it == exec_resident_.end()) it = exec_resident_.emplace(threads, ExecKernelMaxCoResidentBlocks(device_, threads)).first;
    limit = it->second;
  } else {
    if (twoshot_resident_ < 0) twoshot_resident_ = TwoShotKernelMaxCoResidentBlocks(device_);
    limit = twoshot_resident_;
  }
  if (limit > 0) channels = std::min(channels, limit);
  const int cap = Tunable("IBCOMM_MAX_CTAS", 0);
  if (cap > 0) channels = std::min(channels, cap);
  return std::max(1, channels);
}

DeviceTraceRec* DeviceContext::BeginDeviceTrace(int channels, int records, int* capacity) {
  *capacity = 0;
  if (d_trace_ == nullptr || channels > trace_channels_) return nullptr;
  if (!pending_trace_.empty()) CollectTrace(tracer_);
  CUDACHECK(cudaMemsetAsync(d_trace_, 0, sizeof(DeviceTraceRec) * static_cast<size_t>(trace_capacity_) * static_cast<size_t>(trace_channels_), stream_));
  CUDACHECK(cudaStreamSynchronize(stream_));
  PendingTrace pt;
  pt.channels = channels;
  pt.ops = std::min<int>(records, trace_capacity_);
  clock_gettime(CLOCK_MONOTONIC_RAW, &pt.host_launch);
  pending_trace_.push_back(pt);
  *capacity = trace_capacity_;
  return d_trace_;
}

bool DeviceContext::RunStaged(bool multimem, DType dtype, DType wire, const void* sendbuf, void* recvbuf, size_t n, double scale,
                              int channels, cudaStream_t stream) {
  if (Tunable("IBCOMM_STAGED", 1) == 0) return false;
  const size_t wsize = DTypeSize(wire);
  if (wsize > DTypeSize(dtype)) return false;
  if (((reinterpret_cast<uintptr_t>(sendbuf) | reinterpret_cast<uintptr_t>(recvbuf)) & 15u) != 0) return false;
  if ((n * wsize) % 16 != 0) return false;
  if (multimem && (mc_ == nullptr || !NvlsSupportsDType(wire))) return false;
  // Windows: `buffers` input and `buffers` output windows.  They live in the
  // pool and the work region behind it (adjacent, and one collective runs at
  // a time), or, for large messages, in a staging block of its own that the
  // ranks allocate together the first time it is needed - the counterpart of
  // the reference growing its pool and its work buffer at run time with a
  // warning (memory_pool.h:222-236, allreduce_cuda_impl.h:372-385).  Every
  // window costs a fixed 15-20 us of cross-rank hand-over on 8 GPUs, so a
  // 256 MiB message wants windows of tens of MiB: measured 0.80 ms with
  // 16 MiB windows, 0.70 ms with 36 MiB windows (NCCL: 0.73 ms).
  int buffers = Tunable("IBCOMM_STAGED_BUFFERS", 0);
  const uint64_t wire_bytes = static_cast<uint64_t>(n) * wsize;
  const uint64_t arena_stage = layout_.pool_bytes + layout_.work_bytes;
  const uint64_t grow_max = static_cast<uint64_t>(std::max(0, Tunable("IBCOMM_STAGING_GROW_MAX_MIB", 320))) << 20;
  const bool big = wire_bytes >= (96ull << 20);
  if (big && grow_max > arena_stage && ws_ > 1 && !IsCapturing(stream) &&
      (grown_stage_ == nullptr || grown_stage_->bytes < grow_max)) {
    // The decision depends on the message and the knobs only: the same on every rank.
    static bool warned = false;
    if (!warned && rank_ == 0) {
      warned = true;
      IBCOMM_WARN("allreduce of %llu bytes through the staging pool: growing the staging memory from %llu to %llu bytes "
                  "(IBCOMM_MEMORY_POOL_PRE_ALLOC + IBCOMM_WORK_GPU_MEMORY_SIZE; limit IBCOMM_STAGING_GROW_MAX_MIB).\n",
                  static_cast<unsigned long long>(wire_bytes), static_cast<unsigned long long>(arena_stage),
                  static_cast<unsigned long long>(grow_max));
    }
    CUDACHECK(cudaStreamSynchronize(stream));
    if (have_last_) CUDACHECK(cudaStreamSynchronize(last_stream_));
    std::unique_ptr<SymmetricAlloc> g(new SymmetricAlloc());
    g->mine.reset(new SharedAllocation());
    size_t align = 0;
    if (mc_ != nullptr) align = MulticastGroup::Granularity(ws_, grow_max);
    g->mine->Create(grow_max, device_, align);
    g->bytes = g->mine->bytes();
    ExchangeAllocation(g->mine.get(), &g->imported, g->peer_ptr, mc_ != nullptr, &g->mc);
    grown_stage_ = std::move(g);
  }
  const bool use_grown = big && grown_stage_ != nullptr && (!multimem || grown_stage_->mc != nullptr);
  const uint64_t stage_bytes = use_grown ? grown_stage_->bytes : arena_stage;
  // Copy roles in blocks of their own (see the kernel): twice the blocks, all co-resident.
  static const int resident = StagedKernelMaxCoResidentBlocks(device_);
  const int cap = Tunable("IBCOMM_MAX_CTAS", 0);
  const bool split = Tunable("IBCOMM_STAGED_SPLIT", 1) != 0 && resident >= 4 && (cap <= 0 || cap >= 2);
  // Windows of 16-27 MiB measured best on 2 and 8 B200: three of each kind in the arena's 96 MiB, six in the grown block.
  // In the grown block: the switch path wants the largest windows (4 GPUs, 256 MiB: 688 us with three of 53 MiB
  // against 725 with six of 27 MiB), the peer-load path the smaller ones (2 GPUs: 465 against 509 us).
  // With a 16-bit wire (copies convert in registers) six windows again: 416 against 481 us on 4 GPUs.
  if (buffers <= 0) buffers = use_grown ? (multimem && wire == dtype ? 3 : (split ? 6 : 4)) : 3;
  buffers = std::max(3, std::min(buffers, kStagedMaxBuffers));
  const uint64_t quarter = stage_bytes / static_cast<uint64_t>(2 * buffers) / 4096 * 4096;
  if (quarter < 4096) return false;
  StagedParams p;
  memset(&p, 0, sizeof(p));
  p.rank = rank_;
  p.world_size = ws_;
  p.dtype = static_cast<int32_t>(dtype);
  p.wire = static_cast<int32_t>(wire);
  p.use_multimem = multimem ? 1 : 0;
  p.use_tma = (wire == dtype && Tunable("IBCOMM_STAGED_TMA", 1) != 0) ? 1 : 0;
  p.peers = rr_.peers;
  p.sendbuf = sendbuf;
  p.recvbuf = recvbuf;
  p.len_elements = n;
  p.scale = scale;
  int ctas = Tunable("IBCOMM_STAGED_CTAS", 0);
  // 64 CTAs measured best for the switch path at every size from 16 MiB up (fewer flags per window).
  if (ctas <= 0) ctas = std::min(multimem ? 64 : 128, std::max(channels, ChooseChannels(Algo::kDirect, n * wsize, ws_, max_channels_)));
  if (resident > 0) ctas = std::min(ctas, resident);
  ctas = std::max(1, std::min(ctas, 128));  // two reducer groups' flag rows must fit the control page
  if (split) ctas = std::max(1, std::min(ctas, resident / 2));
  if (cap > 0) ctas = std::max(1, std::min(ctas, split ? cap / 2 : cap));
  uint64_t cap_bytes = quarter;
  const int max_window = Tunable("IBCOMM_STAGED_WINDOW_KIB", 0);  // experiment knob: smaller windows
  if (max_window > 0) cap_bytes = std::min<uint64_t>(cap_bytes, static_cast<uint64_t>(max_window) << 10);
  p.window_elems = TwoShotWindowElems(n, cap_bytes / wsize, wsize, ws_, ctas);
  p.buffers = buffers;
  p.split_ctas = split ? 1 : 0;
  // Groups per role (split mode): their flag rows must fit the control page.
  auto groups = [&](const char* knob, int dflt) {
    int g = std::max(1, std::min(Tunable(knob, dflt), 4));
    while (g > 1 && g * ctas > kMaxChannels) --g;
    return g;
  };
  p.load_groups = groups("IBCOMM_STAGED_LOAD_GROUPS", 1);
  p.reduce_groups = groups("IBCOMM_STAGED_REDUCE_GROUPS", 2);
  p.store_groups = groups("IBCOMM_STAGED_STORE_GROUPS", 1);
  p.posters = Tunable("IBCOMM_STAGED_POSTERS", 0) != 0 ? 1 : 0;
  const uint64_t stage_off = use_grown ? 0 : layout_.pool_offset;
  for (int q = 0; q < ws_; ++q) p.stage[q] = use_grown ? grown_stage_->peer_ptr[q] : rr_.peers.arena[q];
  p.mc_stage = use_grown ? (grown_stage_->mc ? grown_stage_->mc->ptr() : nullptr) : rr_.peers.mc_arena;
  for (int j = 0; j < buffers; ++j) {
    p.in_off[j] = stage_off + static_cast<uint64_t>(j) * quarter;
    p.out_off[j] = stage_off + static_cast<uint64_t>(buffers + j) * quarter;
  }
  p.timeout_ns = static_cast<uint64_t>(comm_->timeout_ms()) * 1000000ull;
  p.status = rr_.d_status;
  p.doorbell = rr_.d_doorbell;
  const uint64_t windows = (n + p.window_elems - 1) / p.window_elems;
  p.trace = BeginDeviceTrace(ctas, static_cast<int>(std::min<uint64_t>(windows, 1u << 20)), &p.trace_capacity);
  if (p.trace != nullptr && 4 * windows <= static_cast<uint64_t>(p.trace_capacity)) {
    p.trace_roles = static_cast<int32_t>(windows);
    pending_trace_.back().roles = p.trace_roles;
  }
  IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
  CUDACHECK(LaunchStagedKernel(p, nullptr, 1, split ? 2 * ctas : ctas, stream));
  ++kernel_launches_;
  IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
  staged_channels_ = ctas;
  return true;
}

void DeviceContext::RunTwoShot(bool multimem, DType dtype, DType wire, const void* sendbuf, void* recvbuf, size_t n, double scale,
                               int channels, cudaStream_t stream) {
  const size_t esize = DTypeSize(dtype);
  const size_t bytes = n * esize;
  NvlsParams p;
  memset(&p, 0, sizeof(p));
  p.rank = rank_;
  p.world_size = ws_;
  p.dtype = static_cast<int32_t>(dtype);
  p.use_multimem = multimem ? 1 : 0;
  p.peers = rr_.peers;
  p.sendbuf = sendbuf;
  p.recvbuf = recvbuf;
  p.len_elements = n;
  p.scale = scale;
  p.timeout_ns = static_cast<uint64_t>(comm_->timeout_ms()) * 1000000ull;
  p.status = rr_.d_status;
  p.doorbell = rr_.d_doorbell;

  const SymmetricAlloc* sin = FindSymmetric(sendbuf, bytes);
  const SymmetricAlloc* sout = FindSymmetric(recvbuf, bytes);
  // Zero-copy needs the buffer mapped by the peers and, for the switch path,
  // bound to a multicast object.
  // The direct variant also takes buffers the peers mapped by registration.
  unsigned char* reg_in[kMaxRanks];
  unsigned char* reg_out[kMaxRanks];
  bool rin = sin == nullptr && FindPeerMapped(sendbuf, bytes, reg_in);
  bool rout = sout == nullptr && FindPeerMapped(recvbuf, bytes, reg_out);
  // ... and the switch variant those that registration could bind to a multicast object.
  unsigned char* const rmc_in = multimem && rin ? FindRegisteredMulticast(sendbuf, bytes) : nullptr;
  unsigned char* const rmc_out = multimem && rout ? FindRegisteredMulticast(recvbuf, bytes) : nullptr;
  if (multimem) {
    rin = rin && rmc_in != nullptr;
    rout = rout && rmc_out != nullptr;
  }
  // Registered buffers sit at different offsets on different ranks: all
  // ranks must come to the same decision, so every rank's pointer has to be
  // 16-byte aligned (the mappings' bases are), not only this rank's.
  for (int q = 0; q < ws_; ++q) {
    if (rin && (reinterpret_cast<uintptr_t>(reg_in[q]) & 15u) != 0) rin = false;
    if (rout && (reinterpret_cast<uintptr_t>(reg_out[q]) & 15u) != 0) rout = false;
  }
  const bool zin = (rin || (sin != nullptr && (sin->mc || !multimem))) && (reinterpret_cast<uintptr_t>(sendbuf) & 15u) == 0;
  const bool zout = (rout || (sout != nullptr && (sout->mc || !multimem))) && (reinterpret_cast<uintptr_t>(recvbuf) & 15u) == 0;
  // Nothing zero-copy (or a 16-bit wire, which is staged by definition): the
  // pipelined kernel, when the buffers meet its alignment rules.
  if ((wire != dtype || (!zin && !zout)) && RunStaged(multimem, dtype, wire, sendbuf, recvbuf, n, scale, channels, stream)) return;
  if (wire != dtype)
    IBCOMM_FAIL(NOT_SUPPORTED, "The %s algorithm sends fp32 as 16-bit values only for 16-byte aligned buffers of a whole number of "
                "16-byte wire vectors; use the ring algorithm for this buffer.\n", multimem ? "nvls" : "direct");
  unsigned char* const mc_arena = mc_ ? mc_->ptr() : nullptr;
  // Staging windows: first half of the pool for inputs, second half for outputs.
  const uint64_t half = layout_.pool_bytes / 2 / 4096 * 4096;
  if (!(zin && zout) && half < 8192)
    IBCOMM_FAIL(NOT_SUPPORTED, "Two-shot allreduce of ordinary buffers needs a pool of at least 16 KiB (IBCOMM_MEMORY_POOL_PRE_ALLOC).\n");
  // The last 4 KiB of the input half hold the ragged end (< 16 bytes) of a message.
  const uint64_t window_elems = TwoShotWindowElems(n, (half - 4096) / esize, esize, ws_, channels);
  p.tail_in_off = half - 4096;
  p.stage_in = zin ? 0 : 1;
  p.stage_out = zout ? 0 : 1;
  if (zin && rin) {
    p.mc_in = rmc_in;
    p.local_in = reg_in[rank_];
    for (int q = 0; q < ws_; ++q) p.peer_in[q] = reg_in[q];
  } else if (zin) {
    const size_t off = static_cast<const unsigned char*>(sendbuf) - sin->mine->ptr();
    p.mc_in = sin->mc ? sin->mc->ptr() + off : nullptr;
    p.local_in = sin->mine->ptr() + off;
    for (int q = 0; q < ws_; ++q) p.peer_in[q] = sin->peer_ptr[q] + off;
  } else {
    p.mc_in = mc_arena ? mc_arena + layout_.pool_offset : nullptr;
    p.local_in = arena_.ptr() + layout_.pool_offset;
    for (int q = 0; q < ws_; ++q) p.peer_in[q] = rr_.peers.arena[q] + layout_.pool_offset;
  }
  if (zout && rout) {
    p.mc_out = rmc_out;
    p.local_out = reg_out[rank_];
    for (int q = 0; q < ws_; ++q) p.peer_out[q] = reg_out[q];
  } else if (zout) {
    const size_t off = static_cast<unsigned char*>(recvbuf) - sout->mine->ptr();
    p.mc_out = sout->mc ? sout->mc->ptr() + off : nullptr;
    p.local_out = sout->mine->ptr() + off;
    for (int q = 0; q < ws_; ++q) p.peer_out[q] = sout->peer_ptr[q] + off;
  } else {
    p.mc_out = mc_arena ? mc_arena + layout_.pool_offset + half : nullptr;
    p.local_out = arena_.ptr() + layout_.pool_offset + half;
    for (int q = 0; q < ws_; ++q) p.peer_out[q] = rr_.peers.arena[q] + layout_.pool_offset + half;
  }
  p.window_elems = (zin && zout) ? n : window_elems;
  if (p.window_elems == 0) p.window_elems = 1;
  // Hybrid: IBCOMM_NVLS_HYBRID = percentage (1..90) of a zero-copy switch allreduce that runs direct,
  // concurrently, in the same kernel on CTAs of its own (IBCOMM_NVLS_HYBRID_SWITCH_CTAS + IBCOMM_NVLS_HYBRID_DIRECT_CTAS
  // <= one per SM).  The built-in percentage per world size comes from sweeps on B200 (HybridDefaultPercent).
  if (multimem && zin && zout && ws_ > 1) {
    int direct_percent = Tunable("IBCOMM_NVLS_HYBRID", HybridDefaultPercent(ws_, bytes));
    if (direct_percent < 1 || direct_percent > 90) direct_percent = 0;
    if (direct_percent > 0 && bytes >= (8u << 20)) {
      int nvls_ctas = Tunable("IBCOMM_NVLS_HYBRID_SWITCH_CTAS", 48), direct_ctas = Tunable("IBCOMM_NVLS_HYBRID_DIRECT_CTAS", 96);
      if (nvls_ctas < 1 || direct_ctas < 1 || nvls_ctas + direct_ctas > 148) {
        nvls_ctas = 48;
        direct_ctas = 96;
      }
      HybridParams h;
      memset(&h, 0, sizeof(h));
      h.base = p;
      h.nvls_ctas = nvls_ctas;
      const uint64_t nvec = bytes / 16;
      h.split_vec = nvec * static_cast<uint64_t>(100 - direct_percent) / 100;
      IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
      CUDACHECK(LaunchHybridKernel(h, nvls_ctas + direct_ctas, stream));
      ++kernel_launches_;
      IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
      hybrid_channels_ = nvls_ctas + direct_ctas;
      return;
    }
  }
  IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
  CUDACHECK(LaunchNvlsKernel(p, nullptr, 1, channels, stream));
  ++kernel_launches_;
  IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
}

void DeviceContext::Allreduce(DType dtype, const void* sendbuf, void* recvbuf, size_t n, const CudaAllreduceOptions& opts) {
  NvtxRange nvtx("ibcomm::AllreduceCuda");
  if (sendbuf == nullptr || recvbuf == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "AllreduceCuda: null buffer.\n");
  cudaStream_t stream = StreamFor(opts);
  const size_t esize = DTypeSize(dtype);
  const size_t bytes = n * esize;
  DType wire = (dtype == DType::kFloat32 && (opts.wire == DType::kBFloat16 || opts.wire == DType::kFloat16)) ? opts.wire : dtype;
  if (ws_ == 1) {
    OrderAfterPrevious(stream);
    RunCopy(dtype, sendbuf, recvbuf, n, opts.scale, stream);
    MarkIssued(stream);
    last_algo_ = 0;
    last_channels_ = 0;
    Finish(stream, opts.async);
    return;
  }
  if (n < static_cast<size_t>(ws_))
    IBCOMM_FAIL(NOT_SUPPORTED,
                "Input vector is too short for the Allreduce algorithms: %zu elements for %d processes.\n", n, ws_);
  ConnectPeers();
  Algo algo = opts.algo;
  if (algo == Algo::kAuto) algo = AlgoFromName(env::ReadAlgo());
  // A 16-bit wire is carried by the ring / Rabenseifner programs and by the
  // pipelined staged two-shot (switch or direct), which wants 16-byte aligned
  // buffers of whole 16-byte wire vectors.
  const bool compressed = wire != dtype;
  const bool staged_shape = ((reinterpret_cast<uintptr_t>(sendbuf) | reinterpret_cast<uintptr_t>(recvbuf)) & 15u) == 0 &&
                            (n * DTypeSize(wire)) % 16 == 0 && Tunable("IBCOMM_STAGED", 1) != 0;
  const bool nvls_ok = mc_ != nullptr && NvlsSupportsDType(wire) && (!compressed || staged_shape);
  int channels;
  if (algo == Algo::kAuto) {
    // "symmetric" for the choice: both buffers are mapped by the peers AND bound to the switch
    // (symmetric memory, or registered buffers that registration could bind).
    auto on_switch = [&](const void* b) { return FindSymmetric(b, bytes) != nullptr || FindRegisteredMulticast(b, bytes) != nullptr; };
    const bool symmetric = on_switch(sendbuf) && on_switch(recvbuf);
    unsigned char* unused[kMaxRanks];
    // Registered buffers are mapped by the peers but not bound to the
    // multicast object: zero-copy for the direct algorithm only.  With a
    // 16-bit wire every buffer goes through the pool (that is where the
    // 16-bit copy lives), mapped or not.
    bool mapped = !compressed && (symmetric || (FindPeerMapped(sendbuf, bytes, unused) && FindPeerMapped(recvbuf, bytes, unused)));
    // From 256 MiB on, the switch path through the pool (1 + 1/ws of the
    // message per direction, pipelined copies) beats peer loads on registered
    // buffers in place (2 (ws-1)/ws of it): 1303 against 1444 us at 512 MiB on
    // 8 GPUs.  Such buffers are then treated as ordinary ones.
    // Only from seven ranks on: with four, peer loads in place move 1.5 S per direction and win (615 against 731 us).
    if (mapped && !symmetric && nvls_ok && staged_shape && ws_ >= 7 &&
        bytes >= (static_cast<size_t>(Tunable("IBCOMM_REGISTERED_SWITCH_MIB", 256)) << 20))
      mapped = false;
    TunerChoice c = ChooseAlgorithm(bytes, ws_, nvls_ok && (symmetric || !mapped), mapped, max_channels_);
    algo = c.algo;
    channels = c.channels;
    if ((algo == Algo::kOneShot && (bytes > layout_.oneshot_slot_bytes || compressed)) ||
        ((algo == Algo::kDirect || algo == Algo::kNvls) && compressed && !staged_shape)) {
      algo = Algo::kRing;
      channels = ChooseChannels(algo, bytes, ws_, max_channels_);
    }
  } else {
    if (algo == Algo::kNvls && !nvls_ok)
      IBCOMM_FAIL(NOT_SUPPORTED, "The NVLS algorithm needs NVSwitch multicast and float32/float16/bfloat16 values on the wire "
                  "(with a 16-bit wire: 16-byte aligned buffers of whole 16-byte wire vectors).\n");
    if (algo == Algo::kOneShot && bytes > layout_.oneshot_slot_bytes)
      IBCOMM_FAIL(INVALID_ARGUMENT, "One-shot allreduce handles at most %llu bytes (got %zu).\n",
                  static_cast<unsigned long long>(layout_.oneshot_slot_bytes), bytes);
    if (algo == Algo::kOneShot && compressed) IBCOMM_FAIL(NOT_SUPPORTED, "One-shot allreduce has no wire compression.\n");
    channels = ChooseChannels(algo, bytes, ws_, max_channels_);
    auto on_switch = [&](const void* b) { return FindSymmetric(b, bytes) != nullptr || FindRegisteredMulticast(b, bytes) != nullptr; };
    if (algo == Algo::kNvls && !(on_switch(sendbuf) && on_switch(recvbuf)))
      channels = std::max(channels, ChooseChannels(Algo::kDirect, bytes, ws_, max_channels_));
  }
  {
    // Experiment knobs: a fixed CTA count for the op executor / the two-shot kernels.
    const char* knob = (algo == Algo::kRing || algo == Algo::kRabenseifner) ? "IBCOMM_EXEC_CHANNELS"
                       : (algo == Algo::kNvls || algo == Algo::kDirect)    ? "IBCOMM_TWOSHOT_CHANNELS"
                                                                            : nullptr;
    const int forced = knob != nullptr ? Tunable(knob, 0) : 0;
    if (forced > 0) channels = std::min(forced, kMaxChannels);
  }
  channels = ClampChannels(algo, channels, bytes);
  OrderAfterPrevious(stream);
  switch (algo) {
    case Algo::kRing:
    case Algo::kRabenseifner:
      RunProgram(algo, dtype, wire, sendbuf, recvbuf, n, opts.scale, channels, stream);
      break;
    case Algo::kOneShot:
      RunOneShot(dtype, sendbuf, recvbuf, n, opts.scale, channels, stream);
      break;
    case Algo::kNvls:
      RunTwoShot(true, dtype, wire, sendbuf, recvbuf, n, opts.scale, channels, stream);
      break;
    case Algo::kDirect:
      RunTwoShot(false, dtype, wire, sendbuf, recvbuf, n, opts.scale, channels, stream);
      break;
    default:
      IBCOMM_FAIL(INVALID_ARGUMENT, "Unknown algorithm.\n");
  }
  MarkIssued(stream);
  last_algo_ = static_cast<int>(algo);
  last_channels_ = hybrid_channels_ > 0 ? hybrid_channels_ : (staged_channels_ > 0 ? staged_channels_ : channels);
  hybrid_channels_ = 0;
  staged_channels_ = 0;
  Finish(stream, opts.async);
}

// ------------------------------------------- reduce-scatter and all-gather
void DeviceContext::ReduceScatterOrAllGather(int mode, DType dtype, const void* sendbuf, void* recvbuf, size_t block_elems,
                                             const CudaAllreduceOptions& opts) {
  const bool rs = mode == kRsAgReduceScatter;
  NvtxRange nvtx(rs ? "ibcomm::ReduceScatterCuda" : "ibcomm::AllGatherCuda");
  if (sendbuf == nullptr || recvbuf == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "%s: null buffer.\n", rs ? "ReduceScatterCuda" : "AllGatherCuda");
  if (block_elems == 0) IBCOMM_FAIL(NOT_SUPPORTED, "%s: empty block.\n", rs ? "ReduceScatterCuda" : "AllGatherCuda");
  cudaStream_t stream = StreamFor(opts);
  const size_t esize = DTypeSize(dtype);
  const size_t block_bytes = block_elems * esize;
  if (ws_ == 1) {
    OrderAfterPrevious(stream);
    RunCopy(dtype, sendbuf, recvbuf, block_elems, rs ? opts.scale : 1.0, stream);
    MarkIssued(stream);
    last_algo_ = 0;
    last_channels_ = 0;
    Finish(stream, opts.async);
    return;
  }
  ConnectPeers();
  Algo algo = opts.algo;
  if (algo != Algo::kAuto && algo != Algo::kNvls && algo != Algo::kDirect)
    IBCOMM_FAIL(NOT_SUPPORTED, "Reduce-scatter and all-gather run the nvls or the direct algorithm.\n");
  if (algo == Algo::kAuto) {
    // IBCOMM_ALGO names an allreduce algorithm; it applies here when it names one of the two halves.
    const Algo from_env = AlgoFromName(env::ReadAlgo());
    if (from_env == Algo::kNvls || from_env == Algo::kDirect) algo = from_env;
  }

  RsAgParams p;
  memset(&p, 0, sizeof(p));
  p.rank = rank_;
  p.world_size = ws_;
  p.dtype = static_cast<int32_t>(dtype);
  p.mode = mode;
  p.peers = rr_.peers;
  p.sendbuf = sendbuf;
  p.recvbuf = recvbuf;
  p.block_elems = block_elems;
  p.scale = rs ? opts.scale : 1.0;
  p.timeout_ns = static_cast<uint64_t>(comm_->timeout_ms()) * 1000000ull;
  p.status = rr_.d_status;
  p.doorbell = rr_.d_doorbell;

  // The remote side: the input of a reduce-scatter, the output of an all-gather.
  const void* remote = rs ? sendbuf : recvbuf;
  const size_t remote_bytes = block_bytes * static_cast<size_t>(ws_);
  const bool vec = block_bytes % 16 == 0;
  unsigned char* mapped[kMaxRanks];
  bool zero_copy = vec && FindPeerMapped(remote, remote_bytes, mapped);
  for (int q = 0; q < ws_ && zero_copy; ++q)
    if ((reinterpret_cast<uintptr_t>(mapped[q]) & 15u) != 0) zero_copy = false;  // the same decision on every rank
  const SymmetricAlloc* sym = FindSymmetric(remote, remote_bytes);
  // The switch path asked for by name on a buffer that is mapped but not bound
  // to the multicast object (a registered one): through the pool.
  if (algo == Algo::kNvls && zero_copy && !(sym != nullptr && sym->mc)) zero_copy = false;
  const bool nvls_possible = mc_ != nullptr && NvlsSupportsDType(dtype) && vec && (!zero_copy || (sym != nullptr && sym->mc));
  if (algo == Algo::kNvls && !nvls_possible)
    IBCOMM_FAIL(NOT_SUPPORTED, "The NVLS algorithm needs NVSwitch multicast, a float32/float16/bfloat16 buffer and blocks of whole 16-byte vectors.\n");
  // Each half moves (ws-1)/ws of the message per direction whichever way it
  // runs, so the switch has no bandwidth edge here: mapped buffers go direct
  // (measured faster on 8 B200 at all sizes but 16 MiB); through the pool the
  // switch saves the reducing rank its peer loads.
  if (algo == Algo::kAuto) algo = (nvls_possible && ws_ > 2 && !zero_copy) ? Algo::kNvls : Algo::kDirect;
  p.use_multimem = algo == Algo::kNvls ? 1 : 0;

  if (zero_copy) {
    p.staged = 0;
    for (int q = 0; q < ws_; ++q) p.peer_buf[q] = mapped[q];
    if (p.use_multimem) p.mc_buf = sym->mc->ptr() + (static_cast<const unsigned char*>(remote) - sym->mine->ptr());
    p.window_elems = block_elems;
    p.sub_stride_bytes = block_bytes;
  } else {
    // The whole pool is one window of ws sub-blocks.
    const uint64_t sub = layout_.pool_bytes / static_cast<uint64_t>(ws_) / 4096 * 4096;
    if (sub < 4096) IBCOMM_FAIL(NOT_SUPPORTED, "Reduce-scatter / all-gather of ordinary buffers need a pool of at least %d KiB.\n", 4 * ws_);
    p.staged = 1;
    for (int q = 0; q < ws_; ++q) p.peer_buf[q] = rr_.peers.arena[q] + layout_.pool_offset;
    if (p.use_multimem) p.mc_buf = mc_->ptr() + layout_.pool_offset;
    p.sub_stride_bytes = sub;
    p.window_elems = std::min<uint64_t>(block_elems, sub / esize);
  }
  int channels = ClampChannels(Algo::kDirect, ChooseChannels(p.use_multimem && zero_copy ? Algo::kNvls : Algo::kDirect, remote_bytes, ws_, max_channels_));
  if (p.staged) {
    // Equal windows, each a whole number of units per channel.
    const uint64_t cap = p.sub_stride_bytes / esize;
    p.window_elems = TwoShotWindowElems(block_elems, cap, esize, 1, channels);
    if (!vec) p.window_elems = std::min<uint64_t>(std::max<uint64_t>(p.window_elems, 1), cap);
  }
  OrderAfterPrevious(stream);
  IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
  CUDACHECK(LaunchRsAgKernel(p, nullptr, 1, channels, stream));
  ++kernel_launches_;
  IBCOMM_TRACE(*tracer_, kTraceIssueReduKernel);
  MarkIssued(stream);
  last_algo_ = static_cast<int>(algo);
  last_channels_ = channels;
  Finish(stream, opts.async);
}

// ------------------------------------------------------------ point to point
void DeviceContext::Send(int dest, const void* buf, size_t len) {
  NvtxRange nvtx("ibcomm::Send(device)");
  P2pState& s = p2p_[static_cast<size_t>(dest)];
  if (s.send_done == nullptr) CUDACHECK(cudaEventCreateWithFlags(&s.send_done, cudaEventDisableTiming));
  if (IsLoopback(dest)) {
    // Both ends are this communicator on this device: the matching Recv does
    // one device-to-device copy.  (Two kernels that wait on each other must
    // never be separate launches on one GPU.)
    int owner = -1;
    for (size_t q = 0; q < comm_->eps_.size(); ++q)
      if (comm_->eps_[q].created && comm_->eps_[q].my_info.psn == comm_->eps_[static_cast<size_t>(dest)].peer_info.psn) owner = static_cast<int>(q);
    p2p_[static_cast<size_t>(owner)].loopback.push_back(LoopbackSend{buf, len});
    s.loopback_send_complete = false;
    return;
  }
  ConnectPeers();
  OrderAfterPrevious(send_stream_);
  P2pParams p;
  memset(&p, 0, sizeof(p));
  p.rank = rank_;
  p.peer = dest;
  p.is_send = 1;
  p.world_size = ws_;
  p.peers = rr_.peers;
  p.src = buf;
  p.bytes = len;
  p.mailbox_offset = layout_.mailbox_offset;
  p.slot_bytes = layout_.mailbox_slot_bytes;
  p.slots = layout_.mailbox_slots;
  p.first_piece = s.pieces_sent;
  p.seq = P2pSeq(rank_, dest, s.pieces_sent);
  p.timeout_ns = static_cast<uint64_t>(comm_->timeout_ms()) * 1000000ull;
  p.status = rr_.d_status;
  p.doorbell = rr_.d_doorbell;
  s.pieces_sent += len == 0 ? 1 : (len + p.slot_bytes - 1) / p.slot_bytes;
  IBCOMM_TRACE(*tracer_, kTraceIssueSend);
  CUDACHECK(LaunchP2pKernel(p, p2p_ctas_, send_stream_));
  ++kernel_launches_;
  IBCOMM_TRACE(*tracer_, kTraceIssueSend);
  CUDACHECK(cudaEventRecord(s.send_done, send_stream_));
}

void DeviceContext::Recv(int src, void* buf, size_t len) {
  NvtxRange nvtx("ibcomm::Recv(device)");
  P2pState& s = p2p_[static_cast<size_t>(src)];
  if (s.recv_done == nullptr) CUDACHECK(cudaEventCreateWithFlags(&s.recv_done, cudaEventDisableTiming));
  if (IsLoopback(src)) {
    if (s.loopback.empty())
      IBCOMM_FAIL(NOT_SUPPORTED, "Recv on a self-connected device endpoint needs the matching Send to be posted first.\n");
    LoopbackSend ls = s.loopback.front();
    s.loopback.pop_front();
    if (ls.len != len)
      IBCOMM_FAIL(TRANSPORT_ERROR, "Message length mismatch: %zu bytes posted for receive, %zu bytes incoming.\n", len, ls.len);
    CUDACHECK(cudaMemcpyAsync(buf, ls.buf, len, cudaMemcpyDeviceToDevice, stream_));
    CUDACHECK(cudaEventRecord(s.recv_done, stream_));
    for (P2pState& o : p2p_)
      if (o.send_done != nullptr && !o.loopback_send_complete) {
        CUDACHECK(cudaEventRecord(o.send_done, stream_));
        o.loopback_send_complete = true;
      }
    return;
  }
  ConnectPeers();
  OrderAfterPrevious(recv_stream_);
  P2pParams p;
  memset(&p, 0, sizeof(p));
  p.rank = rank_;
  p.peer = src;
  p.is_send = 0;
  p.world_size = ws_;
  p.peers = rr_.peers;
  p.dst = buf;
  p.bytes = len;
  p.mailbox_offset = layout_.mailbox_offset;
  p.slot_bytes = layout_.mailbox_slot_bytes;
  p.slots = layout_.mailbox_slots;
  p.first_piece = s.pieces_received;
  p.seq = P2pSeq(src, rank_, s.pieces_received);
  p.timeout_ns = static_cast<uint64_t>(comm_->timeout_ms()) * 1000000ull;
  p.status = rr_.d_status;
  p.doorbell = rr_.d_doorbell;
  s.pieces_received += len == 0 ? 1 : (len + p.slot_bytes - 1) / p.slot_bytes;
  IBCOMM_TRACE(*tracer_, kTraceIssueRecv);
  CUDACHECK(LaunchP2pKernel(p, p2p_ctas_, recv_stream_));
  ++kernel_launches_;
  IBCOMM_TRACE(*tracer_, kTraceIssueRecv);
  CUDACHECK(cudaEventRecord(s.recv_done, recv_stream_));
}

bool DeviceContext::Bcast(void* buf, size_t len, int root) {
  NvtxRange nvtx("ibcomm::Bcast(device)");
  ConnectPeers();
  if (mc_ == nullptr || len == 0 || len % 16 != 0) return false;  // the same on every rank
  if (Tunable("IBCOMM_BCAST_MULTICAST", 1) == 0) return false;
  OrderAfterPrevious(stream_);
  BcastParams p;
  memset(&p, 0, sizeof(p));
  p.rank = rank_;
  p.root = root;
  p.world_size = ws_;
  p.peers = rr_.peers;
  p.buf = buf;
  p.bytes = len;
  p.ring_offset = layout_.bcast_ring_offset;
  p.slot_bytes = layout_.mailbox_slot_bytes;
  p.slots = layout_.mailbox_slots;
  p.first_piece = bcast_pieces_;
  p.seq = 0xFE00000000000000ull | (bcast_pieces_ & 0xFFFFFFFFFFFFull);
  p.timeout_ns = static_cast<uint64_t>(comm_->timeout_ms()) * 1000000ull;
  p.status = rr_.d_status;
  p.doorbell = rr_.d_doorbell;
  bcast_pieces_ += (len + p.slot_bytes - 1) / p.slot_bytes;
  IBCOMM_TRACE(*tracer_, kTraceIssueSend);
  CUDACHECK(LaunchBcastKernel(p, p2p_ctas_, stream_));
  ++kernel_launches_;
  IBCOMM_TRACE(*tracer_, kTraceIssueSend);
  MarkIssued(stream_);
  CUDACHECK(cudaStreamSynchronize(stream_));
  Check();
  return true;
}

bool DeviceContext::SendPoll(int dest) {
  P2pState& s = p2p_[static_cast<size_t>(dest)];
  if (IsLoopback(dest) && !s.loopback_send_complete) return false;
  cudaError_t e = cudaEventQuery(s.send_done);
  if (e == cudaErrorNotReady) return false;
  CUDACHECK(e);
  Check();
  return true;
}

bool DeviceContext::RecvPoll(int src) {
  P2pState& s = p2p_[static_cast<size_t>(src)];
  cudaError_t e = cudaEventQuery(s.recv_done);
  if (e == cudaErrorNotReady) return false;
  CUDACHECK(e);
  Check();
  return true;
}

void DeviceContext::SendWait(int dest) {
  P2pState& s = p2p_[static_cast<size_t>(dest)];
  if (IsLoopback(dest) && !s.loopback_send_complete)
    IBCOMM_FAIL(NOT_SUPPORTED, "SendWait on a self-connected device endpoint needs the matching Recv to be posted first.\n");
  CUDACHECK(cudaEventSynchronize(s.send_done));
  Check();
}

void DeviceContext::RecvWait(int src) {
  P2pState& s = p2p_[static_cast<size_t>(src)];
  CUDACHECK(cudaEventSynchronize(s.recv_done));
  Check();
}

// ------------------------------------------------------- symmetric memory
void* DeviceContext::SymmetricAlloc_(size_t bytes) {
  ConnectPeers();
  std::unique_ptr<SymmetricAlloc> s(new SymmetricAlloc());
  s->mine.reset(new SharedAllocation());
  size_t align = 0;
  if (mc_ != nullptr) align = MulticastGroup::Granularity(ws_, bytes);
  s->mine->Create(bytes, device_, align);
  s->bytes = s->mine->bytes();
  if (ws_ > 1) ExchangeAllocation(s->mine.get(), &s->imported, s->peer_ptr, mc_ != nullptr, &s->mc);
  else s->peer_ptr[0] = s->mine->ptr();
  void* p = s->mine->ptr();
  symm_.push_back(std::move(s));
  return p;
}

void DeviceContext::SymmetricFree_(void* ptr) {
  CUDACHECK(cudaDeviceSynchronize());
  if (ws_ > 1) comm_->Barrier();
  for (auto& s : symm_)
    if (s && s->mine->ptr() == ptr) {
      s.reset();
      return;
    }
  IBCOMM_FAIL(INVALID_ARGUMENT, "SymmetricFree: %p is not a symmetric allocation of this communicator.\n", ptr);
}

// ------------------------------------------------------------------ trace
void DeviceContext::CollectTrace(Tracer* tracer) {
  if (d_trace_ == nullptr || tracer == nullptr || pending_trace_.empty()) return;
  CUDACHECK(cudaDeviceSynchronize());
  PendingTrace pt = pending_trace_.back();
  pending_trace_.clear();
  std::vector<DeviceTraceRec> recs(static_cast<size_t>(trace_capacity_) * static_cast<size_t>(pt.channels));
  CUDACHECK(cudaMemcpy(recs.data(), d_trace_, recs.size() * sizeof(DeviceTraceRec), cudaMemcpyDeviceToHost));
  // Device stamps are relative to the earliest one, which is pinned to the
  // host time of the launch.
  uint64_t t0 = ~0ull;
  for (int c = 0; c < pt.channels; ++c)
    for (int i = 0; i < pt.ops; ++i) {
      const DeviceTraceRec& r = recs[static_cast<size_t>(c) * trace_capacity_ + i];
      if (r.t_wait_done != 0) t0 = std::min(t0, r.t_wait_done);
    }
  if (t0 == ~0ull) return;
  const struct timespec& base = tracer->base();
  const double launch_ns = (static_cast<double>(pt.host_launch.tv_sec - base.tv_sec) * 1e9) +
                           static_cast<double>(pt.host_launch.tv_nsec - base.tv_nsec);
  if (pt.roles > 0) {
    staged_timeline_.assign(static_cast<size_t>(8 * pt.roles), 0);
    for (int i = 0; i < 4 * pt.roles; ++i) {
      const DeviceTraceRec& r = recs[static_cast<size_t>(i)];
      staged_timeline_[static_cast<size_t>(2 * i)] = r.t_wait_done >= t0 ? r.t_wait_done - t0 : 0;
      staged_timeline_[static_cast<size_t>(2 * i + 1)] = r.t_done >= t0 ? r.t_done - t0 : 0;
    }
  }
  // Channel 0 is representative; all channels run the same program.
  uint64_t prev = t0;
  for (int i = 0; i < pt.ops; ++i) {
    const DeviceTraceRec& r = recs[static_cast<size_t>(i)];
    if (r.t_wait_done == 0 || r.t_done == 0) continue;
    tracer->AddInterval(kTraceReceived, launch_ns + static_cast<double>(prev - t0), static_cast<double>(r.t_wait_done - prev));
    tracer->AddInterval(kTraceReduced, launch_ns + static_cast<double>(r.t_wait_done - t0), static_cast<double>(r.t_done - r.t_wait_done));
    prev = r.t_done;
  }
}

DeviceInfo DeviceContext::Info() const {
  DeviceInfo i;
  memset(&i, 0, sizeof(i));
  i.device = device_;
  i.nvls = mc_ != nullptr ? 1 : 0;
  i.share_mode = static_cast<int>(arena_.mode());
  i.arena_bytes = arena_.bytes();
  i.pool_bytes = layout_.pool_bytes;
  i.work_bytes = layout_.work_bytes;
  i.calls = calls_;
  i.kernel_launches = kernel_launches_;
  i.switch_registrations = 0;
  for (const RegisteredBuffer& r : registered_) i.switch_registrations += r.mc_ptr != nullptr ? 1 : 0;
  i.last_algo = last_algo_;
  i.last_channels = last_channels_;
  return i;
}

// ------------------------------------------------- free-function interface
bool DeviceContextIsDevicePointer(const void* p) {
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}
void DeviceContextSend(DeviceContext* d, int dest, const void* buf, size_t len) { d->Send(dest, buf, len); }
void DeviceContextRecv(DeviceContext* d, int src, void* buf, size_t len) { d->Recv(src, buf, len); }
bool DeviceContextSendPoll(DeviceContext* d, int dest) { return d->SendPoll(dest); }
bool DeviceContextRecvPoll(DeviceContext* d, int src) { return d->RecvPoll(src); }
void DeviceContextSendWait(DeviceContext* d, int dest) { d->SendWait(dest); }
void DeviceContextRecvWait(DeviceContext* d, int src) { d->RecvWait(src); }
bool DeviceContextBcast(DeviceContext* d, void* buf, size_t len, int root) { return d->Bcast(buf, len, root); }
void DeviceContextCollectTrace(DeviceContext* d, Tracer* tracer) { d->CollectTrace(tracer); }
size_t DeviceContextStagedTimeline(DeviceContext* d, uint64_t* out, size_t capacity_words) {
  const std::vector<uint64_t>& t = d->StagedTimeline();
  const size_t n = std::min(capacity_words, t.size());
  for (size_t i = 0; i < n; ++i) out[i] = t[i];
  return t.size();
}
DeviceInfo DeviceContextInfo(DeviceContext* d) { return d->Info(); }
void DeviceContextSetMaxChannels(DeviceContext* d, int channels) { d->SetMaxChannels(channels); }
void DeviceContextCheck(DeviceContext* d) { d->Check(); }
uint32_t DeviceContextPeekStatus(DeviceContext* d, DeviceStatus* out) { return d->Peek(out); }

void* DeviceContextSymmetricAlloc(Communicator* comm, size_t bytes) {
  comm->PrepareMemoryPool();
  return comm->device()->SymmetricAlloc_(bytes);
}
void DeviceContextSymmetricFree(Communicator* comm, void* ptr) {
  if (comm->device() == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "SymmetricFree: no device context.\n");
  comm->device()->SymmetricFree_(ptr);
}

int DeviceContextRegisterBuffer(Communicator* comm, void* ptr, size_t bytes) {
  comm->PrepareMemoryPool();
  return comm->device()->RegisterBuffer(ptr, bytes);
}
void DeviceContextDeregisterBuffer(Communicator* comm, int id) {
  if (comm->device() == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "DeregisterBuffer: no device context.\n");
  comm->device()->DeregisterBuffer(id);
}
int Communicator::RegisterCudaBuffer(void* ptr, size_t bytes) { return DeviceContextRegisterBuffer(this, ptr, bytes); }
void Communicator::DeregisterCudaBuffer(int id) { DeviceContextDeregisterBuffer(this, id); }

void DeviceContextDeleter::operator()(DeviceContext* d) const { delete d; }

// ---------------------------------------------------- Communicator methods
void Communicator::PrepareMemoryPool() {
  if (device_) return;
  if (!initialized_) IBCOMM_FAIL(INVALID_ARGUMENT, "PrepareMemoryPool: communicator is not initialized.\n");
  device_.reset(new DeviceContext(this));
}

void Communicator::AllreduceCuda(DType dtype, const void* sendbuf, void* recvbuf, size_t len_elements,
                                 const CudaAllreduceOptions& opts) {
  if (!initialized_) IBCOMM_FAIL(INVALID_ARGUMENT, "AllreduceCuda: communicator is not initialized.\n");
  if (sendbuf == nullptr || recvbuf == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "AllreduceCuda: null buffer.\n");
  if (world_size_ > 1 && my_rank_ < 0) IBCOMM_FAIL(INVALID_ARGUMENT, "AllreduceCuda: call RegisterMyself first.\n");
  CollectiveLease lease(this);
  PrepareMemoryPool();
  device_->Allreduce(dtype, sendbuf, recvbuf, len_elements, opts);
}

void Communicator::ReduceScatterCuda(DType dtype, const void* sendbuf, void* recvbuf, size_t block_elements,
                                     const CudaAllreduceOptions& opts) {
  if (!initialized_) IBCOMM_FAIL(INVALID_ARGUMENT, "ReduceScatterCuda: communicator is not initialized.\n");
  if (world_size_ > 1 && my_rank_ < 0) IBCOMM_FAIL(INVALID_ARGUMENT, "ReduceScatterCuda: call RegisterMyself first.\n");
  CollectiveLease lease(this);
  PrepareMemoryPool();
  device_->ReduceScatterOrAllGather(kRsAgReduceScatter, dtype, sendbuf, recvbuf, block_elements, opts);
}

void Communicator::AllGatherCuda(DType dtype, const void* sendbuf, void* recvbuf, size_t block_elements,
                                 const CudaAllreduceOptions& opts) {
  if (!initialized_) IBCOMM_FAIL(INVALID_ARGUMENT, "AllGatherCuda: communicator is not initialized.\n");
  if (world_size_ > 1 && my_rank_ < 0) IBCOMM_FAIL(INVALID_ARGUMENT, "AllGatherCuda: call RegisterMyself first.\n");
  CollectiveLease lease(this);
  PrepareMemoryPool();
  device_->ReduceScatterOrAllGather(kRsAgAllGather, dtype, sendbuf, recvbuf, block_elements, opts);
}

}  // namespace ibcomm
