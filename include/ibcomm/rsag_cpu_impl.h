// Host-buffer reduce-scatter and all-gather over the shared-memory transport:
// the two halves of the ring allreduce as collectives of their own, with the
// ownership a user of the halves expects (block r belongs to rank r; the
// reference's ring, allreduce_cpu_impl.h:23-244, leaves rank r with block
// r+1 after its reduce-scatter and has no entry point for either half).
//
//   ReduceScatter(sendbuf[ws*m], recvbuf[m], m)   recvbuf = sum over ranks of block `rank`
//   AllGather(sendbuf[m], recvbuf[ws*m], m)       block q of recvbuf = rank q's sendbuf
//
// Both run ws-1 ring steps of one block each; incoming partial sums are added
// straight out of the transport ring (PostRecvReduce).
#pragma once

#include <cstring>
#include <vector>

#include "ibcomm/allreduce_cpu_impl.h"
#include "ibcomm/communicator.h"

namespace ibcomm {

template <typename T>
struct CpuRsAg {
  // One ring step: `send` goes to the next rank while `recv` arrives from the
  // previous one (added into `recv` when `reduce`).
  static void Step(Communicator* c, const T* send, T* recv, size_t m, bool reduce, const char* what) {
    const int ws = static_cast<int>(c->world_size()), r = c->rank();
    const int from = (r - 1 + ws) % ws, to = (r + 1) % ws;
    c->PostSend(to, send, m * sizeof(T));
    if (reduce) {
      c->PostRecvReduce(from, recv, m * sizeof(T), &SumBytes<T>);
    } else {
      c->PostRecv(from, recv, m * sizeof(T));
    }
    bool sent = false, received = false;
    StallWatch watch(c->timeout_ms());
    while (!sent || !received) {
      bool moved = false;
      if (!received && c->RecvPoll(from)) received = moved = true;
      if (!sent && c->SendPoll(to)) sent = moved = true;
      if (!watch.Tick(moved)) IBCOMM_FAIL(TRANSPORT_ERROR, "%s: no progress for %d ms on rank %d.\n", what, c->timeout_ms(), r);
    }
  }

  static void Check(Communicator* c, const T* sendbuf, T* recvbuf, size_t m, const char* what) {
    if (sendbuf == nullptr || recvbuf == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "%s: null buffer.\n", what);
    if (m == 0) IBCOMM_FAIL(NOT_SUPPORTED, "%s: empty block.\n", what);
    if (c->world_size() > 1 && c->rank() < 0) IBCOMM_FAIL(INVALID_ARGUMENT, "%s: call RegisterMyself first.\n", what);
  }

  static void ReduceScatter(Communicator* c, const T* sendbuf, T* recvbuf, size_t m) {
    Check(c, sendbuf, recvbuf, m, "ReduceScatter");
    const int ws = static_cast<int>(c->world_size());
    const int r = ws > 1 ? c->rank() : 0;
    if (ws == 1) {
      if (sendbuf != recvbuf) memcpy(recvbuf, sendbuf, m * sizeof(T));
      return;
    }
    CollectiveLease lease(c);
    auto mod = [ws](int x) { return ((x % ws) + ws) % ws; };
    auto block = [&](int b) { return sendbuf + static_cast<size_t>(mod(b)) * m; };
    // Step k sends the partial sum of block r-1-k and receives that of block
    // r-2-k; the last one received is block r.  Two scratch blocks alternate,
    // since the one being sent must stay intact while the next one fills.
    std::vector<T> scratch[2];
    const T* outgoing = block(r - 1);
    for (int k = 0; k <= ws - 2; ++k) {
      const bool last = k == ws - 2;
      T* incoming;
      if (last) {
        incoming = recvbuf;
      } else {
        scratch[k & 1].resize(m);
        incoming = scratch[k & 1].data();
      }
      const T* mine = block(r - 2 - k);
      if (incoming != mine) memcpy(incoming, mine, m * sizeof(T));
      Step(c, outgoing, incoming, m, true, "ReduceScatter");
      outgoing = incoming;
    }
  }

  static void AllGather(Communicator* c, const T* sendbuf, T* recvbuf, size_t m) {
    Check(c, sendbuf, recvbuf, m, "AllGather");
    const int ws = static_cast<int>(c->world_size());
    const int r = ws > 1 ? c->rank() : 0;
    T* own = recvbuf + static_cast<size_t>(r) * m;
    if (own != sendbuf) memcpy(own, sendbuf, m * sizeof(T));
    if (ws == 1) return;
    CollectiveLease lease(c);
    auto mod = [ws](int x) { return ((x % ws) + ws) % ws; };
    // Step k passes block r-k on and receives block r-1-k.
    for (int k = 0; k <= ws - 2; ++k)
      Step(c, recvbuf + static_cast<size_t>(mod(r - k)) * m, recvbuf + static_cast<size_t>(mod(r - 1 - k)) * m, m, false, "AllGather");
  }
};

template <typename T>
void Communicator::ReduceScatter(const T* sendbuf, T* recvbuf, size_t block_elements) {
  CpuRsAg<T>::ReduceScatter(this, sendbuf, recvbuf, block_elements);
}

template <typename T>
void Communicator::AllGather(const T* sendbuf, T* recvbuf, size_t block_elements) {
  CpuRsAg<T>::AllGather(this, sendbuf, recvbuf, block_elements);
}

}  // namespace ibcomm
