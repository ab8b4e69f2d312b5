// ibcomm::Communicator — AllReduce(sum) over one NVLink/NVSwitch box.
//
// Same surface as the reference's IBVerbsCommunicator
// (ibcomm/ibverbs_communicator.h:59-123): connection management by an
// out-of-band exchange of ProcessInfo, two-sided Send/Recv with Poll/Wait,
// a naive Bcast, and four allreduce templates.  The substrate differs:
//
//   host buffers    shared-memory byte rings, one per ordered rank pair
//   device buffers  sm_100a kernels that store into / load from peer GPUs'
//                   memory over NVLink with peer-visible flags, or reduce in
//                   the NVSwitch with multimem instructions
//
// One communicator runs one collective at a time and is not thread-safe;
// several communicators (one per thread, one per GPU) may live in a process.
#pragma once

#include <cstddef>
#include <cstdint>
#include <deque>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "ibcomm/env.h"
#include "ibcomm/error.h"
#include "ibcomm/partition.h"
#include "ibcomm/process_info.h"
#include "ibcomm/shm_transport.h"
#include "ibcomm/trace.h"
#include "ibcomm/util.h"

namespace ibcomm {

// Element types understood by the device kernels and the C API.
enum class DType : int { kFloat32 = 0, kFloat64 = 1, kInt32 = 2, kInt64 = 3, kFloat16 = 4, kBFloat16 = 5 };
size_t DTypeSize(DType t);
const char* DTypeName(DType t);

// Device algorithms.  kAuto picks from the tuning table by message size.
enum class Algo : int { kAuto = 0, kRing = 1, kRabenseifner = 2, kNvls = 3, kOneShot = 4, kDirect = 5 };
const char* AlgoName(Algo a);
Algo AlgoFromName(const std::string& s);  // INVALID_ARGUMENT on unknown names

// What a bytes-in-flight reducer does with `bytes` of incoming data.
using ReduceFn = void (*)(void* dst, const void* src, size_t bytes);

template <typename T>
void SumBytes(void* dst, const void* src, size_t bytes) {
  T* d = static_cast<T*>(dst);
  const T* s = static_cast<const T*>(src);
  const size_t n = bytes / sizeof(T);
  for (size_t i = 0; i < n; ++i) d[i] += s[i];
}

class DeviceContext;  // device arena, peer mappings, kernels (src/cuda)
struct DeviceContextDeleter {
  void operator()(DeviceContext* d) const;
};

// Options of the device allreduce beyond the reference's plain sum.
struct CudaAllreduceOptions {
  Algo algo = Algo::kAuto;
  // Result is multiplied by `scale` exactly once (after the full sum).
  double scale = 1.0;
  // fp32 buffers may travel as bf16/fp16 on the wire (accumulation stays
  // fp32).  kFloat32 means "no compression".
  DType wire = DType::kFloat32;
  // The CUDA stream to run on.  With use_stream == false the communicator's
  // own stream is used (it synchronises with the legacy default stream).
  // use_stream == true takes `stream` literally, so the null stream can be
  // named too.
  void* stream = nullptr;
  bool use_stream = false;
  // false: the call returns when the result is in recvbuf (reference
  // behaviour).  true: the call only enqueues.
  bool async = false;
};

class Communicator {
 public:
  Communicator();
  explicit Communicator(int world_size);
  Communicator(const Communicator&) = delete;
  Communicator& operator=(const Communicator&) = delete;
  Communicator(Communicator&&) = delete;
  Communicator& operator=(Communicator&&) = delete;
  ~Communicator();

  // Idempotent; a second call only warns.
  void Init(int world_size);

  // ---- connection management (reference cpp:286-357) ----
  // Creates my receive endpoint for `dest_rank` and returns its descriptor.
  struct ProcessInfo CreateQueuePair(int dest_rank);
  // Attaches my send side to the peer's endpoint.
  void RegisterQueuePair(int dest_rank, struct ProcessInfo pinfo);
  // Both in one call; usable for a loop-back pair inside one process.
  struct ProcessInfo RegisterProcess(int dest_rank, struct ProcessInfo pinfo);
  void RegisterMyself(int my_rank);

  // ---- two-sided messaging ----
  // Host or device buffers.  One outstanding user-level non-blocking
  // operation per peer and direction; a second one is NOT_SUPPORTED.
  void Send(int dest_rank, const void* buf, size_t len, bool blocking = true);
  void Recv(int src_rank, void* buf, size_t len, bool blocking = true);
  bool SendPoll(int dest_rank);
  bool RecvPoll(int src_rank);
  void SendWait(int dest_rank);
  void RecvWait(int src_rank);
  void Bcast(void* buf, size_t len, int root);

  // ---- allreduce (sum), out-of-place; sendbuf == recvbuf is accepted ----
  template <typename T>
  void AllreduceRing(const T* sendbuf, T* recvbuf, size_t len_elements);
  template <typename T>
  void AllreduceRabenseifner(const T* sendbuf, T* recvbuf, size_t len_elements);
  // The halves of the ring allreduce on host buffers (no counterpart in the
  // reference): block r belongs to rank r.  ReduceScatter: sendbuf holds
  // world_size blocks of `block_elements`, recvbuf one; AllGather: the other
  // way round.
  template <typename T>
  void ReduceScatter(const T* sendbuf, T* recvbuf, size_t block_elements);
  template <typename T>
  void AllGather(const T* sendbuf, T* recvbuf, size_t block_elements);
#ifdef USE_CUDA
  template <typename T>
  void AllreduceRingCuda(const T* sendbuf, T* recvbuf, size_t len_elements);
  template <typename T>
  void AllreduceRabenseifnerCuda(const T* sendbuf, T* recvbuf, size_t len_elements);
  // The general entry: algorithm choice, fused scale, wire compression,
  // caller's stream.  Exposed for the C API and the PyTorch binding.
  void AllreduceCuda(DType dtype, const void* sendbuf, void* recvbuf, size_t len_elements,
                     const CudaAllreduceOptions& opts);
  // The halves of the allreduce as collectives (no counterpart in the
  // reference).  Block r of the message belongs to rank r.  ReduceScatterCuda:
  // sendbuf holds world_size blocks of `block_elements`, recvbuf receives the
  // sum of block `rank` over the ranks (times opts.scale).  AllGatherCuda:
  // sendbuf holds one block, recvbuf receives world_size blocks.  opts.algo:
  // kAuto, kNvls or kDirect; opts.wire is ignored.
  void ReduceScatterCuda(DType dtype, const void* sendbuf, void* recvbuf, size_t block_elements,
                         const CudaAllreduceOptions& opts);
  void AllGatherCuda(DType dtype, const void* sendbuf, void* recvbuf, size_t block_elements,
                     const CudaAllreduceOptions& opts);
  template <typename T>
  void ReduceScatterCuda(const T* sendbuf, T* recvbuf, size_t block_elements);
  template <typename T>
  void AllGatherCuda(const T* sendbuf, T* recvbuf, size_t block_elements);
  // Allocates the staging pool and the work region (lazily called by Init).
  void PrepareMemoryPool();
  // Collective: maps this rank's device buffer (cudaMalloc'ed memory, any
  // position inside its allocation) into every peer, the device analogue of
  // the reference's memory registration (ibv_reg_mr of a user region).
  // Allreduces on the buffer, or on the same sub-range of it on every rank,
  // then skip the staging copies (direct algorithm).  Every rank passes the
  // same size.  Returns a registration id, or -1 on every rank when some
  // rank's memory cannot be shared (the buffers then keep going through the
  // pool).  The caller keeps the memory allocated until DeregisterCudaBuffer.
  int RegisterCudaBuffer(void* ptr, size_t bytes);
  void DeregisterCudaBuffer(int id);
  DeviceContext* device() { return device_.get(); }
#endif

  void SetTimerBase();
  void DumpTrace() const;

  // ---- additions ----
  int rank() const { return my_rank_; }
  size_t world_size() const { return world_size_; }
  bool initialized() const { return initialized_; }
  // Dissemination barrier over the host transport.
  void Barrier();
  // Limit for host-side waits without progress; <= 0 restores the default.
  void SetTimeoutMs(int ms);
  int timeout_ms() const { return timeout_ms_; }
  Tracer& tracer() { return tracer_; }

  // Partition helpers, as members for source compatibility.
  std::vector<Range> SplitBuffer(size_t len_elements, size_t len_per_element) const {
    return ::ibcomm::SplitBufferEnv(len_elements, len_per_element, world_size_);
  }
  std::vector<std::vector<int>> GetRankToChunk(const std::vector<Range>& ranges) const {
    return ::ibcomm::GetRankToChunk(ranges.size(), world_size_);
  }

  // ---- internal queue interface used by the allreduce templates ----
  // Any number of operations may be outstanding per peer; they complete in
  // FIFO order and each completion is reaped by one successful *Poll call.
  void PostSend(int dest_rank, const void* buf, size_t len);
  void PostRecv(int src_rank, void* buf, size_t len);
  // Incoming payload is combined into `buf` by `fn` straight from the ring.
  void PostRecvReduce(int src_rank, void* buf, size_t len, ReduceFn fn);
  // Moves bytes on every endpoint of this communicator.
  void Progress();
  void ProgressPeer(int peer);

 private:
  struct Op {
    unsigned char* buf = nullptr;
    size_t len = 0;
    size_t done = 0;
    bool header_done = false;
    bool pad_done = false;
    ReduceFn reduce = nullptr;
  };
  struct Endpoint {
    std::unique_ptr<ShmInbox> inbox;    // messages from the peer to me
    std::unique_ptr<ShmOutbox> outbox;  // messages from me to the peer
    ProcessInfo my_info{};
    ProcessInfo peer_info{};
    bool created = false;
    bool connected = false;
    std::deque<Op> sendq, recvq;
    size_t send_completions = 0, recv_completions = 0;
    bool user_send_outstanding = false, user_recv_outstanding = false;
    // Device-buffer operations in flight (handled by DeviceContext).
    bool dev_send_outstanding = false, dev_recv_outstanding = false;
  };

  void CheckPeer(int peer, const char* what) const;
  bool ProgressSend(Endpoint& ep);
  bool ProgressRecv(Endpoint& ep);
  void WaitSendCompletion(int dest_rank);
  void WaitRecvCompletion(int src_rank);
  [[noreturn]] void TimeoutFailure(const char* what, int peer);

  bool initialized_ = false;
  int my_rank_ = -1;
  size_t world_size_ = 0;
  int timeout_ms_ = env::kDefaultTimeoutMs;
  std::vector<Endpoint> eps_;
  bool in_collective_ = false;
  Tracer tracer_;
#ifdef USE_CUDA
  std::unique_ptr<DeviceContext, DeviceContextDeleter> device_;
  friend class DeviceContext;
#endif

  template <typename T>
  friend struct CpuAllreduce;
  friend struct CollectiveLease;
};

// Exclusive use of a communicator by one collective (the reference's pool
// lease, memory_pool.h:111-121): a second concurrent collective is
// NOT_SUPPORTED.
struct CollectiveLease {
  explicit CollectiveLease(Communicator* c);
  ~CollectiveLease();
  Communicator* comm;
};

}  // namespace ibcomm

// Source compatibility with code written against the reference.
using IBVerbsCommunicator = ibcomm::Communicator;

#include "ibcomm/allreduce_cpu_impl.h"
#include "ibcomm/rsag_cpu_impl.h"
#ifdef USE_CUDA
#include "ibcomm/allreduce_cuda_impl.h"
#endif
