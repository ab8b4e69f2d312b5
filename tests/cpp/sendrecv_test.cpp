// Transport smoke test in one process: a communicator connected to itself
// through two endpoints ("rank 0" and "rank 1"), the way the reference's
// tests/sendrecv_test.cpp:8-32 loops a queue pair back through the adapter.
// Covers connection set-up, non-blocking send + blocking receive in both
// directions, message sizes around the ring capacity, Poll semantics and the
// one-outstanding-operation rule.
#include <cstdio>
#include <cstring>
#include <numeric>
#include <vector>

#include "ibcomm/communicator.h"
#include "mini_test.h"

static void Connect(ibcomm::Communicator* comm) {
  comm->Init(2);
  ProcessInfo a = comm->CreateQueuePair(1);        // endpoint "towards rank 1"
  ProcessInfo b = comm->RegisterProcess(0, a);     // endpoint "towards rank 0", attached to a
  comm->RegisterQueuePair(1, b);                   // attach a's sender to b
}

MINI_TEST(LoopbackBothDirections) {
  ibcomm::Communicator comm;
  Connect(&comm);
  for (size_t n : {size_t(0), size_t(1), size_t(15), size_t(16), size_t(17), size_t(4096), size_t(1) << 20}) {
    std::vector<unsigned char> out(n), in(n, 0xee);
    std::iota(out.begin(), out.end(), static_cast<unsigned char>(n));
    comm.Send(0, out.data(), n, false);   // lands in the inbox read by Recv(1)
    comm.Recv(1, in.data(), n, true);
    comm.SendWait(0);
    CHECK_TRUE(out == in);
    std::fill(in.begin(), in.end(), 0x11);
    comm.Send(1, out.data(), n, false);
    comm.Recv(0, in.data(), n, true);
    comm.SendWait(1);
    CHECK_TRUE(out == in);
  }
}

MINI_TEST(LargerThanRing) {
  // 9 MiB through a 4 MiB ring: the non-blocking send can only finish while
  // the receive drains, which the blocking Recv does through Progress().
  ibcomm::Communicator comm;
  Connect(&comm);
  const size_t n = (9u << 20) + 5;
  std::vector<unsigned char> out(n), in(n, 0);
  for (size_t i = 0; i < n; ++i) out[i] = static_cast<unsigned char>(i * 2654435761u >> 24);
  comm.Send(0, out.data(), n, false);
  CHECK_TRUE(!comm.SendPoll(0));
  comm.Recv(1, in.data(), n, true);
  comm.SendWait(0);
  CHECK_TRUE(out == in);
}

MINI_TEST(PollAndFifo) {
  ibcomm::Communicator comm;
  Connect(&comm);
  int a = 41, b = 42, ra = 0, rb = 0;
  CHECK_TRUE(!comm.RecvPoll(1));
  comm.Recv(1, &ra, sizeof(ra), false);
  CHECK_TRUE(!comm.RecvPoll(1));
  comm.Send(0, &a, sizeof(a), true);
  while (!comm.RecvPoll(1)) {
  }
  CHECK_EQ(ra, 41);
  // queued internal operations complete in order
  comm.PostSend(0, &a, sizeof(a));
  comm.PostSend(0, &b, sizeof(b));
  comm.PostRecv(1, &rb, sizeof(rb));
  comm.PostRecv(1, &ra, sizeof(ra));
  int reaped = 0;
  while (reaped < 2) reaped += comm.RecvPoll(1) ? 1 : 0;
  CHECK_EQ(rb, 41);
  CHECK_EQ(ra, 42);
  reaped = 0;
  while (reaped < 2) reaped += comm.SendPoll(0) ? 1 : 0;
}

MINI_TEST(ReduceOnReceive) {
  ibcomm::Communicator comm;
  Connect(&comm);
  std::vector<float> out(1000), acc(1000);
  for (size_t i = 0; i < out.size(); ++i) {
    out[i] = static_cast<float>(i);
    acc[i] = 1.0f;
  }
  comm.PostSend(0, out.data(), out.size() * sizeof(float));
  comm.PostRecvReduce(1, acc.data(), acc.size() * sizeof(float), &ibcomm::SumBytes<float>);
  while (!comm.RecvPoll(1)) {
  }
  while (!comm.SendPoll(0)) {
  }
  for (size_t i = 0; i < out.size(); ++i) CHECK_EQ(acc[i], static_cast<float>(i) + 1.0f);
}

MINI_TEST(ErrorCodes) {
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kThrow);
  auto code = [](auto fn) {
    try {
      fn();
    } catch (const ibcomm::Error& e) {
      return e.code();
    }
    return 0;
  };
  ibcomm::Communicator comm;
  Connect(&comm);
  int v = 1, w = 0;
  comm.Send(0, &v, sizeof(v), false);
  CHECK_EQ(code([&] { comm.Send(0, &v, sizeof(v), false); }), 4);  // second outstanding send
  comm.Recv(1, &w, sizeof(w), false);
  CHECK_EQ(code([&] { comm.Recv(1, &w, sizeof(w), false); }), 4);  // second outstanding receive
  comm.RecvWait(1);
  comm.SendWait(0);
  CHECK_EQ(code([&] { comm.Send(5, &v, sizeof(v)); }), 1);          // rank out of range
  CHECK_EQ(code([&] { comm.Send(0, nullptr, 4); }), 1);             // null buffer
  // length mismatch between the two sides is a transport error
  comm.Send(0, &v, sizeof(v), false);
  char small[2];
  CHECK_EQ(code([&] { comm.Recv(1, small, sizeof(small), true); }), 2);
  // waiting for a message nobody sends runs into the limit
  ibcomm::Communicator lonely;
  Connect(&lonely);
  lonely.SetTimeoutMs(50);
  CHECK_EQ(code([&] { lonely.Recv(1, &w, sizeof(w), true); }), 2);
  // a second Init only warns
  lonely.Init(2);
  ibcomm::Communicator uninit;
  CHECK_EQ(code([&] { uninit.Send(0, &v, sizeof(v)); }), 1);
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kExit);
}

int main(int argc, char** argv) { return mini::RunAll(argc > 1 ? argv[1] : nullptr); }
