// Host side of ibcomm::Communicator: lifecycle, connection management,
// framed two-sided messaging over the shared-memory rings, Bcast, Barrier.
#include "ibcomm/communicator.h"

#include <sched.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <fstream>
#include <random>

#ifdef USE_CUDA
#include "ibcomm/device_context.h"
#endif

namespace ibcomm {

namespace {

struct FrameHeader {
  uint64_t len;
  uint64_t magic;
};
static_assert(sizeof(FrameHeader) == kFrameAlign, "frame header must be one alignment unit");
constexpr uint64_t kFrameMagic = 0x6962636f6d6d4652ull;  // "ibcommFR"

inline size_t RoundUp16(size_t n) { return (n + (kFrameAlign - 1)) & ~(kFrameAlign - 1); }
inline size_t RoundDown16(size_t n) { return n & ~(kFrameAlign - 1); }

uint16_t HostLid() {
  // 16-bit digest of the kernel's boot id: equal for every process on the
  // host, different (with high probability) across hosts.  Never 0.
  std::ifstream f("/proc/sys/kernel/random/boot_id");
  std::string s;
  if (f) std::getline(f, s);
  if (s.empty()) {
    char name[256] = {0};
    gethostname(name, sizeof(name) - 1);
    s = name;
  }
  uint32_t h = 2166136261u;
  for (unsigned char c : s) h = (h ^ c) * 16777619u;
  uint16_t lid = static_cast<uint16_t>(h ^ (h >> 16));
  return lid == 0 ? 1 : lid;
}

uint32_t RandomNonce() {
  static thread_local std::mt19937_64 gen([] {
    std::random_device rd;
    uint64_t seed = (static_cast<uint64_t>(rd()) << 32) ^ rd() ^
                    static_cast<uint64_t>(std::chrono::steady_clock::now().time_since_epoch().count());
    return seed;
  }());
  return static_cast<uint32_t>(gen());
}

using Clock = std::chrono::steady_clock;

}  // namespace

size_t DTypeSize(DType t) {
  switch (t) {
    case DType::kFloat32: return 4;
    case DType::kFloat64: return 8;
    case DType::kInt32: return 4;
    case DType::kInt64: return 8;
    case DType::kFloat16: return 2;
    case DType::kBFloat16: return 2;
  }
  return 0;
}

const char* DTypeName(DType t) {
  switch (t) {
    case DType::kFloat32: return "float32";
    case DType::kFloat64: return "float64";
    case DType::kInt32: return "int32";
    case DType::kInt64: return "int64";
    case DType::kFloat16: return "float16";
    case DType::kBFloat16: return "bfloat16";
  }
  return "?";
}

const char* AlgoName(Algo a) {
  switch (a) {
    case Algo::kAuto: return "auto";
    case Algo::kRing: return "ring";
    case Algo::kRabenseifner: return "rabenseifner";
    case Algo::kNvls: return "nvls";
    case Algo::kOneShot: return "oneshot";
    case Algo::kDirect: return "direct";
  }
  return "?";
}

Algo AlgoFromName(const std::string& s) {
  if (s == "auto" || s.empty()) return Algo::kAuto;
  if (s == "ring") return Algo::kRing;
  if (s == "rabenseifner" || s == "raben") return Algo::kRabenseifner;
  if (s == "nvls") return Algo::kNvls;
  if (s == "oneshot") return Algo::kOneShot;
  if (s == "direct" || s == "twoshot") return Algo::kDirect;
  IBCOMM_FAIL(INVALID_ARGUMENT, "Unknown allreduce algorithm '%s'.\n", s.c_str());
}

// ------------------------------------------------------------------ lifecycle
Communicator::Communicator() = default;

Communicator::Communicator(int world_size) { Init(world_size); }

Communicator::~Communicator() {
  if (initialized_ && tracer_.enabled()) DumpTrace();
#ifdef USE_CUDA
  device_.reset();
#endif
  eps_.clear();
}

void Communicator::Init(int world_size) {
  if (initialized_) {
    IBCOMM_WARN("Communicator is already initialized; Init(%d) ignored.\n", world_size);
    return;
  }
  if (world_size < 1) IBCOMM_FAIL(INVALID_ARGUMENT, "world_size must be >= 1 (got %d).\n", world_size);
  world_size_ = static_cast<size_t>(world_size);
  eps_.resize(world_size_);
  timeout_ms_ = env::ReadTimeoutMs();
#ifdef USE_CUDA
  // Knob validation happens here so that a bad value fails at start-up with
  // exit code 1 like the reference's pool constructor; the device memory
  // itself is allocated on first use, which keeps Init usable on hosts
  // without a GPU.
  (void)env::ReadNumCudaStream();
  (void)env::ReadPreAllocSize();
  (void)env::ReadWorkGpuMemorySize();
#endif
  initialized_ = true;
}

void Communicator::SetTimeoutMs(int ms) { timeout_ms_ = ms > 0 ? ms : env::ReadTimeoutMs(); }

void Communicator::SetTimerBase() { tracer_.SetTimerBase(); }

void Communicator::DumpTrace() const {
#ifdef USE_CUDA
  if (device_) DeviceContextCollectTrace(device_.get(), const_cast<Tracer*>(&tracer_));
#endif
  tracer_.Dump(my_rank_);
}

// ------------------------------------------------------- connection handling
void Communicator::CheckPeer(int peer, const char* what) const {
  if (!initialized_) IBCOMM_FAIL(INVALID_ARGUMENT, "%s: communicator is not initialized.\n", what);
  if (peer < 0 || static_cast<size_t>(peer) >= world_size_)
    IBCOMM_FAIL(INVALID_ARGUMENT, "%s: rank %d is outside 0..%zu.\n", what, peer, world_size_ - 1);
}

struct ProcessInfo Communicator::CreateQueuePair(int dest_rank) {
  CheckPeer(dest_rank, "CreateQueuePair");
  Endpoint& ep = eps_[static_cast<size_t>(dest_rank)];
  if (ep.created) {
    IBCOMM_WARN("CreateQueuePair(%d): endpoint already exists; returning it.\n", dest_rank);
    return ep.my_info;
  }
  const uint32_t pid = static_cast<uint32_t>(getpid());
  const size_t ring = ShmRingBytesFromEnv();
  ep.inbox.reset(new ShmInbox());
  uint32_t nonce = 0;
  for (int attempt = 0;; ++attempt) {
    nonce = RandomNonce();
    ErrorPolicy saved = GetErrorPolicy();
    if (attempt < 8) {
      // A name collision is retried with a new nonce.
      SetErrorPolicy(ErrorPolicy::kThrow);
      try {
        ep.inbox->Create(ShmName(pid, nonce), ring);
        SetErrorPolicy(saved);
        break;
      } catch (const Error&) {
        SetErrorPolicy(saved);
        continue;
      }
    }
    ep.inbox->Create(ShmName(pid, nonce), ring);
    break;
  }
  ep.my_info.lid = HostLid();
  ep.my_info.qp_n = pid;
  ep.my_info.psn = nonce;
  ep.created = true;
  return ep.my_info;
}

void Communicator::RegisterQueuePair(int dest_rank, struct ProcessInfo pinfo) {
  CheckPeer(dest_rank, "RegisterQueuePair");
  Endpoint& ep = eps_[static_cast<size_t>(dest_rank)];
  if (!ep.created)
    IBCOMM_FAIL(INVALID_ARGUMENT, "RegisterQueuePair(%d): call CreateQueuePair first.\n", dest_rank);
  if (pinfo.lid != HostLid())
    IBCOMM_FAIL(NOT_SUPPORTED,
                "RegisterQueuePair(%d): the peer lives on another host (lid %u, mine %u); this "
                "transport is intra-node.\n",
                dest_rank, pinfo.lid, HostLid());
  ep.outbox.reset(new ShmOutbox());
  if (!ep.outbox->Open(ShmName(pinfo.qp_n, pinfo.psn)))
    IBCOMM_FAIL(TRANSPORT_ERROR, "RegisterQueuePair(%d): cannot attach to endpoint %s.\n", dest_rank,
                ShmName(pinfo.qp_n, pinfo.psn).c_str());
  ep.peer_info = pinfo;
  ep.connected = true;
}

struct ProcessInfo Communicator::RegisterProcess(int dest_rank, struct ProcessInfo pinfo) {
  struct ProcessInfo mine = CreateQueuePair(dest_rank);
  RegisterQueuePair(dest_rank, pinfo);
  return mine;
}

void Communicator::RegisterMyself(int my_rank) {
  CheckPeer(my_rank, "RegisterMyself");
  my_rank_ = my_rank;
}

// ----------------------------------------------------------------- progress
bool Communicator::ProgressSend(Endpoint& ep) {
  bool moved = false;
  while (!ep.sendq.empty()) {
    Op& op = ep.sendq.front();
    ShmOutbox& out = *ep.outbox;
    if (!op.header_done) {
      if (out.Space() < sizeof(FrameHeader)) break;
      FrameHeader h{op.len, kFrameMagic};
      out.Write(&h, sizeof(h));
      op.header_done = true;
      moved = true;
      if (op.len == 0) out.Publish();
    }
    if (op.done < op.len) {
      const size_t rem = op.len - op.done;
      const size_t space = out.Space();
      if (space >= RoundUp16(rem)) {
        out.Write(op.buf + op.done, rem);
        out.Pad(RoundUp16(rem) - rem);
        op.done = op.len;
      } else {
        const size_t w = RoundDown16(space < rem ? space : rem);
        if (w == 0) {
          if (moved) out.Publish();
          break;
        }
        out.Write(op.buf + op.done, w);
        op.done += w;
      }
      out.Publish();
      moved = true;
    }
    if (op.done == op.len) {
      ep.sendq.pop_front();
      ++ep.send_completions;
    } else {
      break;
    }
  }
  return moved;
}

bool Communicator::ProgressRecv(Endpoint& ep) {
  bool moved = false;
  while (!ep.recvq.empty()) {
    Op& op = ep.recvq.front();
    ShmInbox& in = *ep.inbox;
    if (!op.header_done) {
      if (in.Available() < sizeof(FrameHeader)) break;
      size_t run = 0;
      const unsigned char* p = in.Peek(&run);
      FrameHeader h;
      memcpy(&h, p, sizeof(h));
      if (h.magic != kFrameMagic)
        IBCOMM_FAIL(TRANSPORT_ERROR, "Corrupt frame header on the host transport.\n");
      if (h.len != op.len)
        IBCOMM_FAIL(TRANSPORT_ERROR,
                    "Message length mismatch: %zu bytes posted for receive, %llu bytes incoming.\n",
                    op.len, static_cast<unsigned long long>(h.len));
      in.Release(sizeof(FrameHeader));
      op.header_done = true;
      moved = true;
    }
    while (op.done < op.len) {
      size_t run = 0;
      const unsigned char* p = in.Peek(&run);
      if (run == 0) break;
      const size_t rem = op.len - op.done;
      const size_t n = run < rem ? run : rem;
      if (op.reduce != nullptr) {
        op.reduce(op.buf + op.done, p, n);
      } else {
        memcpy(op.buf + op.done, p, n);
      }
      op.done += n;
      // The final piece was published together with its padding.
      in.Release(op.done == op.len ? n + (RoundUp16(op.len) - op.len) : n);
      moved = true;
    }
    if (op.done == op.len) {
      ep.recvq.pop_front();
      ++ep.recv_completions;
    } else {
      break;
    }
  }
  return moved;
}

void Communicator::ProgressPeer(int peer) {
  Endpoint& ep = eps_[static_cast<size_t>(peer)];
  if (!ep.sendq.empty()) ProgressSend(ep);
  if (!ep.recvq.empty()) ProgressRecv(ep);
}

void Communicator::Progress() {
  for (Endpoint& ep : eps_) {
    if (!ep.sendq.empty()) ProgressSend(ep);
    if (!ep.recvq.empty()) ProgressRecv(ep);
  }
}

void Communicator::TimeoutFailure(const char* what, int peer) {
  IBCOMM_FAIL(TRANSPORT_ERROR, "%s: no progress with rank %d for %d ms (rank %d).\n", what, peer,
              timeout_ms_, my_rank_);
}

// ---------------------------------------------------------------- messaging
void Communicator::PostSend(int dest_rank, const void* buf, size_t len) {
  Endpoint& ep = eps_[static_cast<size_t>(dest_rank)];
  if (!ep.connected)
    IBCOMM_FAIL(INVALID_ARGUMENT, "Send to rank %d: the queue pair is not registered.\n", dest_rank);
  Op op;
  op.buf = const_cast<unsigned char*>(static_cast<const unsigned char*>(buf));
  op.len = len;
  ep.sendq.push_back(op);
  ProgressSend(ep);
}

void Communicator::PostRecv(int src_rank, void* buf, size_t len) { PostRecvReduce(src_rank, buf, len, nullptr); }

void Communicator::PostRecvReduce(int src_rank, void* buf, size_t len, ReduceFn fn) {
  Endpoint& ep = eps_[static_cast<size_t>(src_rank)];
  if (!ep.created)
    IBCOMM_FAIL(INVALID_ARGUMENT, "Recv from rank %d: the queue pair is not created.\n", src_rank);
  Op op;
  op.buf = static_cast<unsigned char*>(buf);
  op.len = len;
  op.reduce = fn;
  ep.recvq.push_back(op);
  ProgressRecv(ep);
}

void Communicator::Send(int dest_rank, const void* buf, size_t len, bool blocking) {
  CheckPeer(dest_rank, "Send");
  if (buf == nullptr && len != 0) IBCOMM_FAIL(INVALID_ARGUMENT, "Send: buf is nullptr.\n");
  Endpoint& ep = eps_[static_cast<size_t>(dest_rank)];
  if (ep.user_send_outstanding || ep.dev_send_outstanding)
    IBCOMM_FAIL(NOT_SUPPORTED,
                "Send to rank %d: the previous non-blocking send has not been waited for.\n", dest_rank);
#ifdef USE_CUDA
  if (len != 0 && DeviceContextIsDevicePointer(buf)) {
    PrepareMemoryPool();
    DeviceContextSend(device_.get(), dest_rank, buf, len);
    ep.dev_send_outstanding = true;
    if (blocking) SendWait(dest_rank);
    return;
  }
#endif
  PostSend(dest_rank, buf, len);
  ep.user_send_outstanding = true;
  if (blocking) SendWait(dest_rank);
}

void Communicator::Recv(int src_rank, void* buf, size_t len, bool blocking) {
  CheckPeer(src_rank, "Recv");
  if (buf == nullptr && len != 0) IBCOMM_FAIL(INVALID_ARGUMENT, "Recv: buf is nullptr.\n");
  Endpoint& ep = eps_[static_cast<size_t>(src_rank)];
  if (ep.user_recv_outstanding || ep.dev_recv_outstanding)
    IBCOMM_FAIL(NOT_SUPPORTED,
                "Recv from rank %d: the previous non-blocking receive has not been waited for.\n",
                src_rank);
#ifdef USE_CUDA
  if (len != 0 && DeviceContextIsDevicePointer(buf)) {
    PrepareMemoryPool();
    DeviceContextRecv(device_.get(), src_rank, buf, len);
    ep.dev_recv_outstanding = true;
    if (blocking) RecvWait(src_rank);
    return;
  }
#endif
  PostRecv(src_rank, buf, len);
  ep.user_recv_outstanding = true;
  if (blocking) RecvWait(src_rank);
}

bool Communicator::SendPoll(int dest_rank) {
  CheckPeer(dest_rank, "SendPoll");
  Endpoint& ep = eps_[static_cast<size_t>(dest_rank)];
#ifdef USE_CUDA
  if (ep.dev_send_outstanding) {
    // A send whose kernel reported a failure is over all the same: the next
    // one must not be refused as "still outstanding".
    bool done;
    try {
      done = DeviceContextSendPoll(device_.get(), dest_rank);
    } catch (...) {
      ep.dev_send_outstanding = false;
      throw;
    }
    if (!done) return false;
    ep.dev_send_outstanding = false;
    return true;
  }
#endif
  if (!ep.sendq.empty()) ProgressSend(ep);
  if (ep.send_completions == 0) return false;
  --ep.send_completions;
  ep.user_send_outstanding = false;
  return true;
}

bool Communicator::RecvPoll(int src_rank) {
  CheckPeer(src_rank, "RecvPoll");
  Endpoint& ep = eps_[static_cast<size_t>(src_rank)];
#ifdef USE_CUDA
  if (ep.dev_recv_outstanding) {
    bool done;
    try {
      done = DeviceContextRecvPoll(device_.get(), src_rank);
    } catch (...) {
      ep.dev_recv_outstanding = false;
      throw;
    }
    if (!done) return false;
    ep.dev_recv_outstanding = false;
    return true;
  }
#endif
  if (!ep.recvq.empty()) ProgressRecv(ep);
  if (ep.recv_completions == 0) return false;
  --ep.recv_completions;
  ep.user_recv_outstanding = false;
  return true;
}

namespace {
// Spin helper: polls `done`, keeps the whole communicator moving, and fails
// when nothing moved for the limit or the peer vanished.
template <typename Done, typename Moved, typename Dead, typename Fail>
void BoundedSpin(int timeout_ms, Done done, Moved moved, Dead dead, Fail fail) {
  auto last = Clock::now();
  auto last_dead_check = last;
  unsigned spins = 0;
  while (!done()) {
    if (moved()) {
      last = Clock::now();
      spins = 0;
      continue;
    }
    if (++spins < 64) continue;
    sched_yield();
    if ((spins & 1023u) != 0) continue;
    auto now = Clock::now();
    if (now - last_dead_check > std::chrono::milliseconds(50)) {
      last_dead_check = now;
      if (dead() && !done()) fail(true);
    }
    if (now - last > std::chrono::milliseconds(timeout_ms)) fail(false);
  }
}
}  // namespace

void Communicator::WaitSendCompletion(int dest_rank) {
  Endpoint& ep = eps_[static_cast<size_t>(dest_rank)];
  if (ep.send_completions == 0 && ep.sendq.empty())
    IBCOMM_FAIL(INVALID_ARGUMENT, "SendWait(%d): nothing to wait for.\n", dest_rank);
  BoundedSpin(
      timeout_ms_, [&] { return ep.send_completions > 0; },
      [&] {
        bool m = ProgressSend(ep);
        for (Endpoint& o : eps_) {
          if (&o == &ep) continue;
          if (!o.sendq.empty()) m |= ProgressSend(o);
          if (!o.recvq.empty()) m |= ProgressRecv(o);
        }
        if (!ep.recvq.empty()) m |= ProgressRecv(ep);
        return m;
      },
      [&] { return ep.outbox->PeerDead(); },
      [&](bool dead) {
        if (dead)
          IBCOMM_FAIL(TRANSPORT_ERROR, "SendWait: rank %d is gone (rank %d).\n", dest_rank, my_rank_);
        TimeoutFailure("SendWait", dest_rank);
      });
}

void Communicator::WaitRecvCompletion(int src_rank) {
  Endpoint& ep = eps_[static_cast<size_t>(src_rank)];
  if (ep.recv_completions == 0 && ep.recvq.empty())
    IBCOMM_FAIL(INVALID_ARGUMENT, "RecvWait(%d): nothing to wait for.\n", src_rank);
  BoundedSpin(
      timeout_ms_, [&] { return ep.recv_completions > 0; },
      [&] {
        bool m = ProgressRecv(ep);
        for (Endpoint& o : eps_) {
          if (&o == &ep) continue;
          if (!o.sendq.empty()) m |= ProgressSend(o);
          if (!o.recvq.empty()) m |= ProgressRecv(o);
        }
        if (!ep.sendq.empty()) m |= ProgressSend(ep);
        return m;
      },
      [&] { return ep.inbox->PeerDead() && ep.inbox->Available() == 0; },
      [&](bool dead) {
        if (dead)
          IBCOMM_FAIL(TRANSPORT_ERROR, "RecvWait: rank %d is gone (rank %d).\n", src_rank, my_rank_);
        TimeoutFailure("RecvWait", src_rank);
      });
}

void Communicator::SendWait(int dest_rank) {
  CheckPeer(dest_rank, "SendWait");
  Endpoint& ep = eps_[static_cast<size_t>(dest_rank)];
#ifdef USE_CUDA
  if (ep.dev_send_outstanding) {
    ep.dev_send_outstanding = false;  // over when the wait returns, failed or not
    DeviceContextSendWait(device_.get(), dest_rank);
    return;
  }
#endif
  WaitSendCompletion(dest_rank);
  --ep.send_completions;
  ep.user_send_outstanding = false;
}

void Communicator::RecvWait(int src_rank) {
  CheckPeer(src_rank, "RecvWait");
  Endpoint& ep = eps_[static_cast<size_t>(src_rank)];
#ifdef USE_CUDA
  if (ep.dev_recv_outstanding) {
    ep.dev_recv_outstanding = false;  // over when the wait returns, failed or not
    DeviceContextRecvWait(device_.get(), src_rank);
    return;
  }
#endif
  WaitRecvCompletion(src_rank);
  --ep.recv_completions;
  ep.user_recv_outstanding = false;
}

void Communicator::Bcast(void* buf, size_t len, int root) {
  CheckPeer(root, "Bcast");
  if (my_rank_ < 0) IBCOMM_FAIL(INVALID_ARGUMENT, "Bcast: call RegisterMyself first.\n");
  if (world_size_ == 1) return;
#ifdef USE_CUDA
  // Device buffers on a box with NVSwitch multicast: the root writes every
  // piece once and the switch delivers it to all ranks.  (Every rank takes the
  // same decision: it depends on the box, the length and the alignment, and
  // the ranks pass buffers of the same kind.)
  if (len != 0 && DeviceContextIsDevicePointer(buf)) {
    PrepareMemoryPool();
    if (DeviceContextBcast(device_.get(), buf, len, root)) return;
  }
#endif
  if (my_rank_ == root) {
    for (size_t r = 0; r < world_size_; ++r)
      if (static_cast<int>(r) != root) Send(static_cast<int>(r), buf, len, false);
    for (size_t r = 0; r < world_size_; ++r)
      if (static_cast<int>(r) != root) SendWait(static_cast<int>(r));
  } else {
    Recv(root, buf, len, true);
  }
}

void Communicator::Barrier() {
  if (my_rank_ < 0) IBCOMM_FAIL(INVALID_ARGUMENT, "Barrier: call RegisterMyself first.\n");
  unsigned char token_out = 1, token_in = 0;
  const int ws = static_cast<int>(world_size_);
  for (int k = 1; k < ws; k <<= 1) {
    const int to = (my_rank_ + k) % ws;
    const int from = (my_rank_ - k + ws) % ws;
    PostSend(to, &token_out, 1);
    PostRecv(from, &token_in, 1);
    WaitRecvCompletion(from);
    --eps_[static_cast<size_t>(from)].recv_completions;
    WaitSendCompletion(to);
    --eps_[static_cast<size_t>(to)].send_completions;
  }
}

// -------------------------------------------------------------------- lease
CollectiveLease::CollectiveLease(Communicator* c) : comm(c) {
  if (c->in_collective_)
    IBCOMM_FAIL(NOT_SUPPORTED, "Another collective is already running on this communicator.\n");
  c->in_collective_ = true;
}

CollectiveLease::~CollectiveLease() { comm->in_collective_ = false; }

}  // namespace ibcomm
