// CPU-thread model of the staged two-shot protocols (nvls_kernel.cu,
// rsag_kernel.cu): one thread per (rank, CTA), the pool windows as plain
// arrays, the per-CTA cross-rank barriers as release/acquire flags.  It uses
// the kernels' own split (`WindowPart`) and window sizing
// (`TwoShotWindowElems`), so a split that lets a CTA run ahead into bytes
// another CTA still needs shows up here: as a wrong sum, and as a data race
// when the test is built with -fsanitize=thread.
//
// The reference has no such protocol (its chunks are driven by the host,
// allreduce_cuda_impl.h:35-301), hence no counterpart of this test.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <thread>
#include <vector>

#include "ibcomm/device_types.h"
#include "ibcomm/schedule.h"
#include "mini_test.h"

using namespace ibcomm;

namespace {

constexpr int kVec = 4;  // elements per "16-byte vector" of the model

struct World {
  int ws, ncta;
  std::vector<std::vector<int64_t>> in, out;  // pool halves per rank
  std::vector<std::vector<int64_t>> tail;     // the ragged end's own slot per rank
  // bar[rank][cta][source]
  std::vector<std::atomic<uint64_t>> bar;
  World(int ws_, int ncta_, size_t half_elems)
      : ws(ws_), ncta(ncta_), in(ws_, std::vector<int64_t>(half_elems)), out(ws_, std::vector<int64_t>(half_elems)),
        tail(ws_, std::vector<int64_t>(kVec)), bar(static_cast<size_t>(ws_) * ncta_ * ws_) {
    for (auto& b : bar) b.store(0);
  }
  std::atomic<uint64_t>& Bar(int rank, int cta, int src) { return bar[(static_cast<size_t>(rank) * ncta + cta) * ws + src]; }
  // Barrier between CTA `cta` of every rank (CrossRankBarrier).
  void Barrier(int rank, int cta, uint64_t phase) {
    for (int q = 0; q < ws; ++q)
      if (q != rank) Bar(q, cta, rank).store(phase, std::memory_order_release);
    for (int q = 0; q < ws; ++q)
      if (q != rank)
        while (Bar(rank, cta, q).load(std::memory_order_acquire) < phase) std::this_thread::yield();
  }
};

int64_t Value(int rank, uint64_t i) { return static_cast<int64_t>((i * 7 + 3) % 1009) * (rank + 1); }
int64_t Sum(int ws, uint64_t i) {
  int64_t s = 0;
  for (int r = 0; r < ws; ++r) s += Value(r, i);
  return s;
}

// TwoShotBody, direct variant, both buffers staged.
void AllreduceCta(World* w, int rank, int cta, const std::vector<int64_t>& send, std::vector<int64_t>* recv, uint64_t n,
                  uint64_t window_elems) {
  const int ws = w->ws, ncta = w->ncta;
  uint64_t phase = 0;
  const uint64_t full_nvec = (window_elems + kVec - 1) / kVec;
  for (uint64_t w0 = 0; w0 < n; w0 += window_elems) {
    const uint64_t wn = std::min<uint64_t>(window_elems, n - w0);
    const uint64_t nvec = wn / kVec, tail0 = nvec * kVec;
    for (int s = 0; s < ws; ++s) {
      uint64_t b, e;
      WindowPart(full_nvec, nvec, s, ws, cta, ncta, &b, &e);
      for (uint64_t i = b * kVec; i < e * kVec; ++i) w->in[rank][i] = send[w0 + i];
    }
    if (cta == 0)
      for (uint64_t i = tail0; i < wn; ++i) w->tail[rank][i - tail0] = send[w0 + i];
    w->Barrier(rank, cta, ++phase);
    {
      uint64_t b, e;
      WindowPart(full_nvec, nvec, rank, ws, cta, ncta, &b, &e);
      for (uint64_t i = b * kVec; i < e * kVec; ++i) {
        int64_t acc = 0;
        for (int q = 0; q < ws; ++q) acc += w->in[q][i];
        for (int q = 0; q < ws; ++q) w->out[q][i] = acc;
      }
    }
    std::vector<int64_t> tail_acc;
    if (cta == 0)
      for (uint64_t i = tail0; i < wn; ++i) {
        int64_t acc = 0;
        for (int q = 0; q < ws; ++q) acc += w->tail[q][i - tail0];
        tail_acc.push_back(acc);
      }
    w->Barrier(rank, cta, ++phase);
    if (cta == 0)
      for (uint64_t i = tail0; i < wn; ++i) (*recv)[w0 + i] = tail_acc[i - tail0];
    for (int s = 0; s < ws; ++s) {
      uint64_t b, e;
      WindowPart(full_nvec, nvec, s, ws, cta, ncta, &b, &e);
      for (uint64_t i = b * kVec; i < e * kVec; ++i) (*recv)[w0 + i] = w->out[rank][i];
    }
  }
}

bool RunAllreduce(int ws, int ncta, uint64_t n, uint64_t cap_elems) {
  const uint64_t window = TwoShotWindowElems(n, cap_elems, 16 / kVec, ws, ncta);
  World w(ws, ncta, cap_elems + kVec);
  std::vector<std::vector<int64_t>> send(ws, std::vector<int64_t>(n)), recv(ws, std::vector<int64_t>(n, -1));
  for (int r = 0; r < ws; ++r)
    for (uint64_t i = 0; i < n; ++i) send[r][i] = Value(r, i);
  // Two calls back to back (the second reuses the windows the first one left).
  for (int call = 0; call < 2; ++call) {
    std::vector<std::thread> th;
    for (int r = 0; r < ws; ++r)
      for (int c = 0; c < ncta; ++c) th.emplace_back(AllreduceCta, &w, r, c, std::cref(send[r]), &recv[r], n, window);
    for (auto& t : th) t.join();
    for (auto& b : w.bar) b.store(0);
    for (int r = 0; r < ws; ++r)
      for (uint64_t i = 0; i < n; ++i)
        if (recv[r][i] != Sum(ws, i)) {
          fprintf(stderr, "allreduce ws=%d ncta=%d n=%llu window=%llu: rank %d element %llu wrong\n", ws, ncta,
                  static_cast<unsigned long long>(n), static_cast<unsigned long long>(window), r, static_cast<unsigned long long>(i));
          return false;
        }
  }
  return true;
}

// RsAgBody, direct variant, remote side staged; units of one vector.
void RsAgCta(World* w, bool all_gather, int rank, int cta, const std::vector<int64_t>& send, std::vector<int64_t>* recv,
             uint64_t block_units, uint64_t win_units, uint64_t sub_stride) {
  const int ws = w->ws, ncta = w->ncta;
  uint64_t phase = 0;
  w->Barrier(rank, cta, ++phase);
  for (uint64_t w0 = 0; w0 < block_units; w0 += win_units) {
    const uint64_t wn = std::min<uint64_t>(win_units, block_units - w0);
    const bool last = w0 + wn >= block_units;
    uint64_t b, e;
    WindowPart(win_units, wn, 0, 1, cta, ncta, &b, &e);
    if (!all_gather) {
      for (int s = 0; s < ws; ++s)
        for (uint64_t i = b * kVec; i < e * kVec; ++i) w->in[rank][s * sub_stride + i] = send[(s * block_units + w0) * kVec + i];
      w->Barrier(rank, cta, ++phase);
      for (uint64_t i = b * kVec; i < e * kVec; ++i) {
        int64_t acc = 0;
        for (int q = 0; q < ws; ++q) acc += w->in[q][rank * sub_stride + i];
        (*recv)[w0 * kVec + i] = acc;
      }
      w->Barrier(rank, cta, ++phase);
    } else {
      for (uint64_t i = b * kVec; i < e * kVec; ++i)
        for (int q = 0; q < ws; ++q) w->in[q][rank * sub_stride + i] = send[w0 * kVec + i];
      w->Barrier(rank, cta, ++phase);
      for (int s = 0; s < ws; ++s)
        for (uint64_t i = b * kVec; i < e * kVec; ++i) (*recv)[(s * block_units + w0) * kVec + i] = w->in[rank][s * sub_stride + i];
      if (!last) w->Barrier(rank, cta, ++phase);
    }
  }
}

bool RunRsAg(int ws, int ncta, uint64_t block_units, uint64_t cap_units) {
  const uint64_t m = block_units * kVec;
  const uint64_t window = TwoShotWindowElems(m, cap_units * kVec, 16 / kVec, 1, ncta) / kVec;
  const uint64_t sub_stride = cap_units * kVec;
  World w(ws, ncta, sub_stride * ws);
  std::vector<std::vector<int64_t>> full(ws, std::vector<int64_t>(m * ws)), shard(ws, std::vector<int64_t>(m, -1)),
      gathered(ws, std::vector<int64_t>(m * ws, -1));
  for (int r = 0; r < ws; ++r)
    for (uint64_t i = 0; i < m * ws; ++i) full[r][i] = Value(r, i);
  for (int pass = 0; pass < 2; ++pass) {
    const bool all_gather = pass == 1;
    std::vector<std::thread> th;
    for (int r = 0; r < ws; ++r)
      for (int c = 0; c < ncta; ++c)
        th.emplace_back(RsAgCta, &w, all_gather, r, c, std::cref(all_gather ? shard[r] : full[r]),
                        all_gather ? &gathered[r] : &shard[r], block_units, window, sub_stride);
    for (auto& t : th) t.join();
    for (auto& b : w.bar) b.store(0);
  }
  for (int r = 0; r < ws; ++r)
    for (uint64_t i = 0; i < m * ws; ++i)
      if (gathered[r][i] != Sum(ws, i)) {
        fprintf(stderr, "rs+ag ws=%d ncta=%d block=%llu window=%llu: rank %d element %llu wrong\n", ws, ncta,
                static_cast<unsigned long long>(m), static_cast<unsigned long long>(window * kVec), r, static_cast<unsigned long long>(i));
        return false;
      }
  return true;
}

}  // namespace

MINI_TEST(PartOfAShortWindowLiesInsideThePartOfAFullOne) {
  // What the per-CTA barriers rely on: in every window of a call, CTA b only
  // touches bytes that are CTA b's in a full window.
  for (int ws : {1, 2, 3, 8})
    for (int ncta : {1, 3, 16, 128})
      for (uint64_t full : {uint64_t(1), uint64_t(100), uint64_t(4096), uint64_t(2000128)})
        for (uint64_t nvec : {uint64_t(0), uint64_t(1), full / 3, full - 1, full})
          for (int s = 0; s < ws; ++s)
            for (int c = 0; c < ncta; ++c) {
              uint64_t fb, fe, b, e;
              WindowPart(full, full, s, ws, c, ncta, &fb, &fe);
              WindowPart(full, nvec, s, ws, c, ncta, &b, &e);
              CHECK_TRUE(b <= e && e <= nvec);
              CHECK_TRUE(b == e || (fb <= b && e <= fe));
            }
}

MINI_TEST(WindowsAreEqualAndFit) {
  for (uint64_t n : {uint64_t(1), uint64_t(5), uint64_t(4096), uint64_t(40000001), uint64_t(1) << 28})
    for (uint64_t cap : {uint64_t(1024), uint64_t(8387584)})
      for (int ws : {2, 8})
        for (int ch : {1, 128}) {
          const uint64_t w = TwoShotWindowElems(n, cap, 4, ws, ch);
          CHECK_TRUE(w >= 1 && w <= std::max<uint64_t>(cap, 1));
          const uint64_t windows = (n + w - 1) / w;
          CHECK_EQ(windows, (n + cap - 1) / cap);          // as few windows as the pool allows
          if (windows > 1) CHECK_TRUE(w % 4 == 0);        // later windows start on a vector boundary
        }
}

MINI_TEST(StagedAllreduceProtocol) {
  for (int ws : {2, 3, 4})
    for (int ncta : {1, 3, 4})
      for (uint64_t n : {uint64_t(ws), uint64_t(37), uint64_t(256), uint64_t(1000), uint64_t(1003), uint64_t(2049)})
        CHECK_TRUE(RunAllreduce(ws, ncta, n, 256));
}

MINI_TEST(StagedReduceScatterAllGatherProtocol) {
  for (int ws : {2, 3, 4})
    for (int ncta : {1, 3, 4})
      for (uint64_t block_units : {uint64_t(1), uint64_t(7), uint64_t(64), uint64_t(150), uint64_t(257)})
        CHECK_TRUE(RunRsAg(ws, ncta, block_units, 64));
}

int main(int argc, char** argv) { return mini::RunAll(argc > 1 ? argv[1] : nullptr); }
