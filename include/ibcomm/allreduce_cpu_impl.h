// Host-buffer allreduce schedules over the shared-memory transport.
//
// AllreduceRing        chunk-pipelined ring reduce-scatter + ring all-gather
//                      (reference ibcomm/allreduce_cpu_impl.h:23-244): own
//                      block goes first, chunk ids descend inside a block, and
//                      after the reduce-scatter rank r owns the reduced block
//                      of rank r+1.
// AllreduceRabenseifner recursive halving + recursive doubling
//                      (reference :246-372), one message per step, extended
//                      to any world size by folding the ranks above the
//                      largest power of two into their neighbours first.
//
// Incoming partial sums are added straight out of the transport ring
// (PostRecvReduce), so neither schedule needs a temporary buffer.
#pragma once

#include <chrono>
#include <cstring>
#include <vector>

#include "ibcomm/communicator.h"

namespace ibcomm {

// Fails the calling collective when nothing has moved for the communicator's
// limit.  Tick(true) re-arms it.
class StallWatch {
 public:
  explicit StallWatch(int timeout_ms)
      : limit_(std::chrono::milliseconds(timeout_ms)), last_(std::chrono::steady_clock::now()) {}
  // Returns false once the limit has passed without progress.
  bool Tick(bool moved) {
    if (moved) {
      idle_ = 0;
      last_ = std::chrono::steady_clock::now();
      return true;
    }
    if ((++idle_ & 0xfffu) != 0) return true;
    return std::chrono::steady_clock::now() - last_ <= limit_;
  }

 private:
  std::chrono::steady_clock::duration limit_;
  std::chrono::steady_clock::time_point last_;
  unsigned idle_ = 0;
};

template <typename T>
struct CpuAllreduce {
  static void Ring(Communicator* c, const T* sendbuf, T* recvbuf, size_t n);
  static void Rabenseifner(Communicator* c, const T* sendbuf, T* recvbuf, size_t n);

 private:
  static void WaitRecv(Communicator* c, int peer) {
    c->WaitRecvCompletion(peer);
    --c->eps_[static_cast<size_t>(peer)].recv_completions;
  }
  static void WaitSend(Communicator* c, int peer) {
    c->WaitSendCompletion(peer);
    --c->eps_[static_cast<size_t>(peer)].send_completions;
  }
};

template <typename T>
void CpuAllreduce<T>::Ring(Communicator* c, const T* sendbuf, T* recvbuf, size_t n) {
  if (sendbuf == nullptr || recvbuf == nullptr)
    IBCOMM_FAIL(INVALID_ARGUMENT, "AllreduceRing: null buffer.\n");
  const int ws = static_cast<int>(c->world_size());
  if (ws == 1) {
    if (sendbuf != recvbuf) memcpy(recvbuf, sendbuf, sizeof(T) * n);
    return;
  }
  if (c->rank() < 0) IBCOMM_FAIL(INVALID_ARGUMENT, "AllreduceRing: call RegisterMyself first.\n");
  CollectiveLease lease(c);
  const std::vector<Range> ranges = c->SplitBuffer(n, sizeof(T));
  const std::vector<std::vector<int>> blocks = c->GetRankToChunk(ranges);
  const int r = c->rank();
  const int from = (r - 1 + ws) % ws;
  const int to = (r + 1) % ws;
  auto mod = [ws](int x) { return ((x % ws) + ws) % ws; };
  const bool in_place = (sendbuf == recvbuf);

  // Everything I will receive, in wire order.
  struct In {
    int chunk;
    bool reduce;   // reduce-scatter phase
    bool forward;  // pass on to `to` once complete
  };
  std::vector<In> incoming;
  for (int k = 0; k <= ws - 2; ++k) {
    const std::vector<int>& blk = blocks[static_cast<size_t>(mod(r - 1 - k))];
    for (auto it = blk.rbegin(); it != blk.rend(); ++it) incoming.push_back({*it, true, true});
  }
  for (int k = 0; k <= ws - 2; ++k) {
    const std::vector<int>& blk = blocks[static_cast<size_t>(mod(r - k))];
    for (auto it = blk.rbegin(); it != blk.rend(); ++it) incoming.push_back({*it, false, k != ws - 2});
  }

  auto ptr = [&](T* base, int chunk) { return base + ranges[static_cast<size_t>(chunk)].first; };
  auto bytes = [&](int chunk) {
    const Range& g = ranges[static_cast<size_t>(chunk)];
    return (g.second - g.first) * sizeof(T);
  };

  // My own block leaves first, straight from sendbuf.
  size_t sends_posted = 0, sends_done = 0;
  {
    const std::vector<int>& mine = blocks[static_cast<size_t>(r)];
    for (auto it = mine.rbegin(); it != mine.rend(); ++it) {
      c->PostSend(to, sendbuf + ranges[static_cast<size_t>(*it)].first, bytes(*it));
      ++sends_posted;
    }
  }

  constexpr size_t kWindow = 3;  // receives kept posted, like the reference
  size_t next_post = 0, next_done = 0;
  StallWatch watch(c->timeout_ms());
  while (next_done < incoming.size() || sends_done < sends_posted) {
    bool moved = false;
    while (next_post < incoming.size() && next_post - next_done < kWindow) {
      const In& in = incoming[next_post];
      if (in.reduce) {
        if (!in_place) memcpy(ptr(recvbuf, in.chunk), sendbuf + ranges[static_cast<size_t>(in.chunk)].first, bytes(in.chunk));
        c->PostRecvReduce(from, ptr(recvbuf, in.chunk), bytes(in.chunk), &SumBytes<T>);
      } else {
        c->PostRecv(from, ptr(recvbuf, in.chunk), bytes(in.chunk));
      }
      ++next_post;
      moved = true;
    }
    while (next_done < next_post && c->RecvPoll(from)) {
      const In& in = incoming[next_done];
      if (in.forward) {
        c->PostSend(to, ptr(recvbuf, in.chunk), bytes(in.chunk));
        ++sends_posted;
      }
      ++next_done;
      moved = true;
    }
    while (sends_done < sends_posted && c->SendPoll(to)) {
      ++sends_done;
      moved = true;
    }
    if (!watch.Tick(moved))
      IBCOMM_FAIL(TRANSPORT_ERROR, "AllreduceRing: no progress for %d ms on rank %d.\n", c->timeout_ms(), r);
  }
}

template <typename T>
void CpuAllreduce<T>::Rabenseifner(Communicator* c, const T* sendbuf, T* recvbuf, size_t n) {
  if (sendbuf == nullptr || recvbuf == nullptr)
    IBCOMM_FAIL(INVALID_ARGUMENT, "AllreduceRabenseifner: null buffer.\n");
  const int ws = static_cast<int>(c->world_size());
  if (ws == 1) {
    if (sendbuf != recvbuf) memcpy(recvbuf, sendbuf, sizeof(T) * n);
    return;
  }
  if (c->rank() < 0)
    IBCOMM_FAIL(INVALID_ARGUMENT, "AllreduceRabenseifner: call RegisterMyself first.\n");
  if (n < static_cast<size_t>(ws))
    IBCOMM_FAIL(NOT_SUPPORTED,
                "Input vector is too short for Rabenseifner's algorithm: %zu elements for %d "
                "processes.\n",
                n, ws);
  CollectiveLease lease(c);
  const int r = c->rank();
  const int p = static_cast<int>(util::FloorPow2(static_cast<uint64_t>(ws)));
  const int extra = ws - p;  // ranks folded away before the power-of-two core
  const int exp = util::GetExpOfTwo(static_cast<uint64_t>(p));

  if (sendbuf != recvbuf) memcpy(recvbuf, sendbuf, sizeof(T) * n);
  unsigned char* base = reinterpret_cast<unsigned char*>(recvbuf);
  auto send = [&](int peer, size_t b, size_t e) { c->PostSend(peer, base + b * sizeof(T), (e - b) * sizeof(T)); };
  auto recv = [&](int peer, size_t b, size_t e) { c->PostRecv(peer, base + b * sizeof(T), (e - b) * sizeof(T)); };
  auto recv_sum = [&](int peer, size_t b, size_t e) {
    c->PostRecvReduce(peer, base + b * sizeof(T), (e - b) * sizeof(T), &SumBytes<T>);
  };

  // Fold: ranks below 2*extra work in pairs (even, odd).  The pair first
  // swaps halves and adds (both directions busy), then the even rank hands
  // its half to the odd one, which enters the core with the pair's sum.
  int vrank;  // rank inside the core, -1 for the ranks that sit out
  const size_t half = n / 2;
  if (r < 2 * extra) {
    if ((r & 1) == 0) {
      const int partner = r + 1;
      send(partner, half, n);
      recv_sum(partner, 0, half);
      WaitRecv(c, partner);
      WaitSend(c, partner);
      send(partner, 0, half);
      WaitSend(c, partner);
      vrank = -1;
    } else {
      const int partner = r - 1;
      send(partner, 0, half);
      recv_sum(partner, half, n);
      WaitRecv(c, partner);
      WaitSend(c, partner);
      recv(partner, 0, half);
      WaitRecv(c, partner);
      vrank = r / 2;
    }
  } else {
    vrank = r - extra;
  }
  auto real_rank = [extra](int v) { return v < extra ? 2 * v + 1 : v + extra; };

  if (vrank >= 0 && p > 1) {
    const std::vector<Range> blocks = SplitEven(n, static_cast<size_t>(p));
    auto lo = [&](int blk) { return blocks[static_cast<size_t>(blk)].first; };
    auto hi = [&](int blk) { return blocks[static_cast<size_t>(blk - 1)].second; };  // end of [.., blk)
    int b = 0, e = p;  // my current block range [b, e)
    // Reduce-scatter by recursive halving: nearest partner first; the lower
    // rank of a pair gives away the front part and keeps the back part.
    for (int s = 0; s < exp; ++s) {
      const int vpeer = vrank ^ (1 << s);
      const int peer = real_rank(vpeer);
      const int mid = e - (e - b) / 2;
      int sb, se, kb, ke;
      if (vrank < vpeer) {
        sb = b; se = mid; kb = mid; ke = e;
      } else {
        kb = b; ke = mid; sb = mid; se = e;
      }
      send(peer, lo(sb), hi(se));
      recv_sum(peer, lo(kb), hi(ke));
      WaitRecv(c, peer);
      WaitSend(c, peer);
      b = kb;
      e = ke;
    }
    // All-gather by recursive doubling: farthest partner first.
    for (int s = 0; s < exp; ++s) {
      const int vpeer = vrank ^ (1 << (exp - 1 - s));
      const int peer = real_rank(vpeer);
      const int w = e - b;
      int rb, re;
      if (vrank > vpeer) {
        rb = e; re = e + w;
      } else {
        rb = b - w; re = b;
      }
      send(peer, lo(b), hi(e));
      recv(peer, lo(rb), hi(re));
      WaitRecv(c, peer);
      WaitSend(c, peer);
      b = b < rb ? b : rb;
      e = e > re ? e : re;
    }
  }

  // Unfold: the odd rank of each pair returns the full result.
  if (r < 2 * extra) {
    if ((r & 1) == 0) {
      recv(r + 1, 0, n);
      WaitRecv(c, r + 1);
    } else {
      send(r - 1, 0, n);
      WaitSend(c, r - 1);
    }
  }
}

template <typename T>
void Communicator::AllreduceRing(const T* sendbuf, T* recvbuf, size_t len_elements) {
  CpuAllreduce<T>::Ring(this, sendbuf, recvbuf, len_elements);
}

template <typename T>
void Communicator::AllreduceRabenseifner(const T* sendbuf, T* recvbuf, size_t len_elements) {
  CpuAllreduce<T>::Rabenseifner(this, sendbuf, recvbuf, len_elements);
}

}  // namespace ibcomm
