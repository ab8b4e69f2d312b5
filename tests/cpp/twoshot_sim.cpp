// CPU-thread model of the staged two-shot protocols (nvls_kernel.cu,
// rsag_kernel.cu, and the pipelined staged_kernel.cu with its three roles per CTA), of the one-shot protocol (oneshot_kernel.cu) and of the
// mailbox protocol of device Send/Recv (p2p_sendrecv.cu): one thread per (rank,
// CTA), the pool windows, push slots and mailboxes as plain arrays, the per-CTA
// cross-rank barriers, flags and credits as release/acquire atomics.  It uses
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
void AllreduceCta(World* w, uint64_t seq, int rank, int cta, const std::vector<int64_t>& send, std::vector<int64_t>* recv,
                  uint64_t n, uint64_t window_elems) {
  const int ws = w->ws, ncta = w->ncta;
  uint64_t phase = seq << 32;  // flag values only grow, call after call
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
  // Every rank runs two calls back to back, like two kernels of one stream
  // (the second reuses the windows the first one left); the ranks are not
  // synchronised with each other between the calls.
  std::atomic<int> bad{0};
  auto rank_body = [&](int r) {
    for (uint64_t seq = 1; seq <= 2; ++seq) {
      std::fill(recv[r].begin(), recv[r].end(), -1);
      std::vector<std::thread> ctas;
      for (int c = 0; c < ncta; ++c) ctas.emplace_back(AllreduceCta, &w, seq, r, c, std::cref(send[r]), &recv[r], n, window);
      for (auto& t : ctas) t.join();
      for (uint64_t i = 0; i < n; ++i)
        if (recv[r][i] != Sum(ws, i)) ++bad;
    }
  };
  std::vector<std::thread> ranks;
  for (int r = 0; r < ws; ++r) ranks.emplace_back(rank_body, r);
  for (auto& t : ranks) t.join();
  if (bad.load() != 0)
    fprintf(stderr, "allreduce ws=%d ncta=%d n=%llu window=%llu: %d wrong elements\n", ws, ncta, static_cast<unsigned long long>(n),
            static_cast<unsigned long long>(window), bad.load());
  return bad.load() == 0;
}

// ---- pipelined staged two-shot (staged_kernel.cu) ----
// One thread per (rank, CTA, role, group): loaders, reducers, storers; a role's
// groups take the windows in turn.  `bufs` input and `bufs` output windows per
// rank; flag rows per (group, rank, CTA, source) of three kinds: in_ready,
// reduced, out_free.  The waits and posts are the kernel's: loader k waits
// reduced >= k-bufs+1 (the window that used the buffer before), reducer k
// waits in_ready >= k+1 and out_free >= k-bufs+1, storer k waits reduced >= k+1.
struct PipeWorld {
  int ws, ncta, bufs;
  bool posters = false;  // a poster thread behind every reducer group publishes its windows
  std::vector<std::atomic<uint32_t>> stored;  // [rank][cta][reducer group]: windows the group has handed to its poster
  int groups[3];  // per kind of row: 0 in_ready (loader groups), 1 reduced (reducer groups), 2 out_free (storer groups)
  std::vector<std::vector<std::vector<int64_t>>> in, out;  // [buffer][rank][element]
  std::vector<std::atomic<uint64_t>> row[3];               // [group][rank][cta][source rank]
  PipeWorld(int ws_, int ncta_, size_t window, int bufs_, int lg, int rg, int sg) : ws(ws_), ncta(ncta_), bufs(bufs_), groups{lg, rg, sg} {
    in.assign(bufs_, std::vector<std::vector<int64_t>>(ws_, std::vector<int64_t>(window, -7)));
    out = in;
    for (int k = 0; k < 3; ++k) {
      row[k] = std::vector<std::atomic<uint64_t>>(static_cast<size_t>(groups[k]) * ws_ * ncta_ * ws_);
      for (auto& f : row[k]) f.store(0);
    }
    stored = std::vector<std::atomic<uint32_t>>(static_cast<size_t>(ws_) * ncta_ * rg);
    for (auto& c : stored) c.store(0);
  }
  std::atomic<uint32_t>& Stored(int rank, int cta, int group) { return stored[(static_cast<size_t>(rank) * ncta + cta) * groups[1] + group]; }
  // Window k's words of one kind live in the rows of group k % groups: the
  // groups of a role finish their windows in any order, a row's values only grow.
  std::atomic<uint64_t>& Flag(int kind, uint64_t window, int rank, int cta, int src) {
    const size_t g = static_cast<size_t>(window % static_cast<uint64_t>(groups[kind]));
    return row[kind][((g * ws + rank) * ncta + cta) * ws + src];
  }
  void WaitAll(int kind, uint64_t window, int rank, int cta, uint64_t v) {
    for (int q = 0; q < ws; ++q)
      while (Flag(kind, window, rank, cta, q).load(std::memory_order_acquire) < v) std::this_thread::yield();
  }
  void PostAll(int kind, uint64_t window, int rank, int cta, uint64_t v) {
    for (int q = 0; q < ws; ++q) Flag(kind, window, q, cta, rank).store(v, std::memory_order_release);
  }
};

// role: 0 loader, 1 reducer, 2 storer, 3 poster of a reducer group; `group` of the role's groups takes windows
// group, group + groups, ...  (StagedKernel: the groups are warps of a block, or of two blocks in split mode).
void PipeRole(PipeWorld* w, int role, int group, uint64_t seq, int rank, int cta, const std::vector<int64_t>& send,
              std::vector<int64_t>* recv, uint64_t total_nv, uint64_t full_nv) {
  const int ws = w->ws, ncta = w->ncta;
  const uint64_t base = seq << 32, bufs = static_cast<uint64_t>(w->bufs);
  const uint64_t windows = (total_nv + full_nv - 1) / full_nv;
  const int role_groups = w->groups[role == 3 ? 1 : role];
  if (role == 3) {
    // The poster: waits until its group has issued the stores of window k (a counter in the block's shared
    // memory, release / acquire), then publishes the window.  The calls of one rank follow each other in
    // one thread per role, so the counter restarts with every call.
    uint32_t seen = 0;
    for (uint64_t k = static_cast<uint64_t>(group); k < windows; k += static_cast<uint64_t>(role_groups)) {
      ++seen;
      while (w->Stored(rank, cta, group).load(std::memory_order_acquire) < seen) std::this_thread::yield();
      w->PostAll(1, k, rank, cta, base | (k + 1));
    }
    return;
  }
  uint32_t handed = 0;
  for (uint64_t k = static_cast<uint64_t>(group); k < windows; k += static_cast<uint64_t>(role_groups)) {
    const int j = static_cast<int>(k % bufs);
    const uint64_t v0 = k * full_nv, nv = std::min(full_nv, total_nv - v0);
    if (role == 0) {
      if (k >= bufs) w->WaitAll(1, k - bufs, rank, cta, base | (k - bufs + 1));
      for (int s = 0; s < ws; ++s) {
        uint64_t b, e;
        WindowPart(full_nv, nv, s, ws, cta, ncta, &b, &e);
        for (uint64_t i = b * kVec; i < e * kVec; ++i) w->in[j][rank][i] = send[v0 * kVec + i];
      }
      w->PostAll(0, k, rank, cta, base | (k + 1));
    } else if (role == 1) {
      w->WaitAll(0, k, rank, cta, base | (k + 1));
      if (k >= bufs) w->WaitAll(2, k - bufs, rank, cta, base | (k - bufs + 1));
      uint64_t b, e;
      WindowPart(full_nv, nv, rank, ws, cta, ncta, &b, &e);
      for (uint64_t i = b * kVec; i < e * kVec; ++i) {
        int64_t acc = 0;
        for (int q = 0; q < ws; ++q) acc += w->in[j][q][i];
        for (int q = 0; q < ws; ++q) w->out[j][q][i] = acc;
      }
      if (w->posters) w->Stored(rank, cta, group).store(++handed, std::memory_order_release);
      else w->PostAll(1, k, rank, cta, base | (k + 1));
    } else {
      w->WaitAll(1, k, rank, cta, base | (k + 1));
      for (int s = 0; s < ws; ++s) {
        uint64_t b, e;
        WindowPart(full_nv, nv, s, ws, cta, ncta, &b, &e);
        for (uint64_t i = b * kVec; i < e * kVec; ++i) (*recv)[v0 * kVec + i] = w->out[j][rank][i];
      }
      w->PostAll(2, k, rank, cta, base | (k + 1));
    }
  }
}

bool RunPipelined(int ws, int ncta, uint64_t n_vec, uint64_t cap_elems, int bufs = 3, int lg = 1, int rg = 2, int sg = 1, bool posters = false) {
  const uint64_t n = n_vec * kVec;
  const uint64_t window = TwoShotWindowElems(n, cap_elems, 16 / kVec, ws, ncta);
  const uint64_t full_nv = window / kVec;
  if (full_nv == 0) return true;
  PipeWorld w(ws, ncta, window, bufs, lg, rg, sg);
  w.posters = posters;
  std::vector<std::vector<int64_t>> send(ws, std::vector<int64_t>(n)), recv(ws, std::vector<int64_t>(n, -1));
  for (int r = 0; r < ws; ++r)
    for (uint64_t i = 0; i < n; ++i) send[r][i] = Value(r, i);
  std::atomic<int> bad{0};
  auto rank_body = [&](int r) {
    // Three calls back to back; the ranks are not synchronised in between.
    for (uint64_t seq = 1; seq <= 3; ++seq) {
      std::fill(recv[r].begin(), recv[r].end(), -1);
      for (int c = 0; c < ncta; ++c)
        for (int g = 0; g < rg; ++g) w.Stored(r, c, g).store(0);
      std::vector<std::thread> t;
      for (int c = 0; c < ncta; ++c)
        for (int role = 0; role < (posters ? 4 : 3); ++role)
          for (int g = 0; g < w.groups[role == 3 ? 1 : role]; ++g)
            t.emplace_back(PipeRole, &w, role, g, seq, r, c, std::cref(send[r]), &recv[r], n_vec, full_nv);
      for (auto& x : t) x.join();
      for (uint64_t i = 0; i < n; ++i)
        if (recv[r][i] != Sum(ws, i)) ++bad;
    }
  };
  std::vector<std::thread> ranks;
  for (int r = 0; r < ws; ++r) ranks.emplace_back(rank_body, r);
  for (auto& t : ranks) t.join();
  if (bad.load() != 0)
    fprintf(stderr, "pipelined ws=%d ncta=%d nvec=%llu window=%llu bufs=%d groups=%d/%d/%d: %d wrong elements\n", ws, ncta,
            static_cast<unsigned long long>(n_vec), static_cast<unsigned long long>(window), bufs, lg, rg, sg, bad.load());
  return bad.load() == 0;
}

// HybridKernel (hybrid_kernel.cu): zero-copy buffers; CTAs [0, na) own vectors [0, split), the other CTAs
// [split, nvec); rank r reduces shard r of its role's part and writes it to every rank.  (The switch
// role is modelled as the same sum; what is checked is the split and the barrier placement.)
void HybridCta(World* w, uint64_t seq, int rank, int block, int na, std::vector<std::vector<int64_t>>* bufs_in,
               std::vector<std::vector<int64_t>>* bufs_out, uint64_t n, uint64_t split_vec) {
  const int ws = w->ws, grid = w->ncta;
  const bool switch_role = block < na;
  const int cta = switch_role ? block : block - na, ncta = switch_role ? na : grid - na;
  const uint64_t nvec = n / kVec, tail0 = nvec * kVec, split = std::min(split_vec, nvec);
  uint64_t sb, se, b, e;
  SubRange(switch_role ? 0 : split, switch_role ? split : nvec, rank, ws, &sb, &se);
  SubRange(sb, se, cta, ncta, &b, &e);
  w->Barrier(rank, block, (seq << 32) | 1);
  for (uint64_t i = b * kVec; i < e * kVec; ++i) {
    int64_t acc = 0;
    for (int q = 0; q < ws; ++q) acc += (*bufs_in)[q][i];
    for (int q = 0; q < ws; ++q) (*bufs_out)[q][i] = acc;
  }
  std::vector<int64_t> tail_acc;
  const bool has_tail = !switch_role && cta == 0;
  if (has_tail)
    for (uint64_t i = tail0; i < n; ++i) {
      int64_t acc = 0;
      for (int q = 0; q < ws; ++q) acc += (*bufs_in)[q][i];
      tail_acc.push_back(acc);
    }
  w->Barrier(rank, block, (seq << 32) | 2);
  if (has_tail)
    for (uint64_t i = tail0; i < n; ++i) (*bufs_out)[rank][i] = tail_acc[i - tail0];
}

bool RunHybrid(int ws, int na, int nb, uint64_t n, uint64_t split_vec) {
  World w(ws, na + nb, kVec);
  std::vector<std::vector<int64_t>> in(ws, std::vector<int64_t>(n)), out(ws, std::vector<int64_t>(n, -1));
  for (int r = 0; r < ws; ++r)
    for (uint64_t i = 0; i < n; ++i) in[r][i] = Value(r, i);
  std::atomic<int> bad{0};
  auto rank_body = [&](int r) {
    for (uint64_t seq = 1; seq <= 2; ++seq) {
      std::vector<std::thread> ctas;
      for (int c = 0; c < na + nb; ++c) ctas.emplace_back(HybridCta, &w, seq, r, c, na, &in, &out, n, split_vec);
      for (auto& t : ctas) t.join();
      for (uint64_t i = 0; i < n; ++i)
        if (out[r][i] != Sum(ws, i)) ++bad;
    }
  };
  std::vector<std::thread> ranks;
  for (int r = 0; r < ws; ++r) ranks.emplace_back(rank_body, r);
  for (auto& t : ranks) t.join();
  if (bad.load() != 0)
    fprintf(stderr, "hybrid ws=%d ctas=%d+%d n=%llu split=%llu: %d wrong elements\n", ws, na, nb, static_cast<unsigned long long>(n),
            static_cast<unsigned long long>(split_vec), bad.load());
  return bad.load() == 0;
}

// RsAgBody, direct variant, remote side staged; units of one vector.
void RsAgCta(World* w, uint64_t seq, bool all_gather, int rank, int cta, const std::vector<int64_t>& send,
             std::vector<int64_t>* recv, uint64_t block_units, uint64_t win_units, uint64_t sub_stride) {
  const int ws = w->ws, ncta = w->ncta;
  uint64_t phase = seq << 32;
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
  // Every rank runs the reduce-scatter and then the all-gather of its shard,
  // as two kernels of one stream, twice; nothing else synchronises the ranks.
  std::atomic<int> bad{0};
  auto rank_body = [&](int r) {
    uint64_t seq = 0;
    for (int rep = 0; rep < 2; ++rep)
      for (int pass = 0; pass < 2; ++pass) {
        const bool all_gather = pass == 1;
        ++seq;
        std::vector<std::thread> ctas;
        for (int c = 0; c < ncta; ++c)
          ctas.emplace_back(RsAgCta, &w, seq, all_gather, r, c, std::cref(all_gather ? shard[r] : full[r]),
                            all_gather ? &gathered[r] : &shard[r], block_units, window, sub_stride);
        for (auto& t : ctas) t.join();
        if (all_gather)
          for (uint64_t i = 0; i < m * ws; ++i)
            if (gathered[r][i] != Sum(ws, i)) ++bad;
      }
  };
  std::vector<std::thread> ranks;
  for (int r = 0; r < ws; ++r) ranks.emplace_back(rank_body, r);
  for (auto& t : ranks) t.join();
  if (bad.load() != 0)
    fprintf(stderr, "rs+ag ws=%d ncta=%d block=%llu window=%llu: %d wrong elements\n", ws, ncta, static_cast<unsigned long long>(m),
            static_cast<unsigned long long>(window * kVec), bad.load());
  return bad.load() == 0;
}

// ---- one-shot: push to every peer's slot, flag, sum locally; slots are
// double-buffered by the parity of the call number and there is no barrier at
// the end of a call.  A rank runs its calls one after the other (kernels of
// one stream), every call with its own number of CTAs.
struct OneShotWorld {
  int ws;
  size_t cap;
  static constexpr int kMaxCta = 8;
  std::vector<std::vector<int64_t>> slots;  // [rank][(parity * ws + src) * cap + i]
  std::vector<std::atomic<uint64_t>> flag;  // [rank][parity][cta][src]
  OneShotWorld(int ws_, size_t cap_) : ws(ws_), cap(cap_), slots(ws_, std::vector<int64_t>(2 * ws_ * cap_)), flag(static_cast<size_t>(ws_) * 2 * kMaxCta * ws_) {
    for (auto& f : flag) f.store(0);
  }
  int64_t* Slot(int owner, unsigned parity, int src) { return slots[owner].data() + (static_cast<size_t>(parity) * ws + src) * cap; }
  std::atomic<uint64_t>& Flag(int owner, unsigned parity, int cta, int src) {
    return flag[((static_cast<size_t>(owner) * 2 + parity) * kMaxCta + cta) * ws + src];
  }
};

void OneShotCta(OneShotWorld* w, int me, int cta, int ncta, uint64_t seq, const std::vector<int64_t>& send, std::vector<int64_t>* recv) {
  const int ws = w->ws;
  const uint64_t n = send.size();
  const unsigned parity = static_cast<unsigned>(seq & 1u);
  const uint64_t nvec = (n + kVec - 1) / kVec, per = (nvec + ncta - 1) / ncta;
  const uint64_t lo = std::min<uint64_t>(per * cta * kVec, n), hi = std::min<uint64_t>(lo + per * kVec, n);
  for (int k = 1; k < ws; ++k) {
    const int q = (me + k) % ws;
    int64_t* dst = w->Slot(q, parity, me);
    for (uint64_t i = lo; i < hi; ++i) dst[i] = send[i];
  }
  for (int q = 0; q < ws; ++q)
    if (q != me) w->Flag(q, parity, cta, me).store(seq, std::memory_order_release);
  for (int q = 0; q < ws; ++q)
    if (q != me)
      while (w->Flag(me, parity, cta, q).load(std::memory_order_acquire) < seq) std::this_thread::yield();
  for (uint64_t i = lo; i < hi; ++i) {
    int64_t acc = 0;
    for (int q = 0; q < ws; ++q) acc += (q == me) ? send[i] : w->Slot(me, parity, q)[i];
    (*recv)[i] = acc;
  }
}

bool RunOneShot(int ws, const std::vector<std::pair<uint64_t, int>>& calls) {
  OneShotWorld w(ws, 1024);
  std::atomic<int> bad{0};
  auto rank_body = [&](int me) {
    uint64_t seq = 0;
    for (size_t c = 0; c < calls.size(); ++c) {
      const uint64_t n = calls[c].first;
      const int ncta = calls[c].second;
      ++seq;
      std::vector<int64_t> send(n), recv(n, -1);
      for (uint64_t i = 0; i < n; ++i) send[i] = Value(me, i + 31 * c);
      std::vector<std::thread> ctas;
      for (int b = 0; b < ncta; ++b) ctas.emplace_back(OneShotCta, &w, me, b, ncta, seq, std::cref(send), &recv);
      for (auto& t : ctas) t.join();  // the kernel is over before the next one starts
      for (uint64_t i = 0; i < n; ++i)
        if (recv[i] != Sum(ws, i + 31 * c)) ++bad;
    }
  };
  std::vector<std::thread> ranks;
  for (int r = 0; r < ws; ++r) ranks.emplace_back(rank_body, r);
  for (auto& t : ranks) t.join();
  if (bad.load() != 0) fprintf(stderr, "one-shot ws=%d: %d wrong elements\n", ws, bad.load());
  return bad.load() == 0;
}

// ---- device Send/Recv: the sender stores piece k of the pair into slot
// k % slots of its mailbox at the receiver and publishes the cumulative piece
// count; the receiver copies the piece out and returns a credit; a slot is
// reused once the piece that held it before has been consumed.
struct Mailbox {
  size_t slots, slot_elems;
  std::vector<int64_t> data;
  std::atomic<uint64_t> flag{0}, credit{0};
  Mailbox(size_t s, size_t e) : slots(s), slot_elems(e), data(s * e) {}
};

void MailboxSend(Mailbox* mb, const std::vector<int64_t>& msg, uint64_t first_piece) {
  const uint64_t pieces = (msg.size() + mb->slot_elems - 1) / mb->slot_elems;
  for (uint64_t j = 0; j < pieces; ++j) {
    const uint64_t k = first_piece + j, off = j * mb->slot_elems;
    const uint64_t len = std::min<uint64_t>(mb->slot_elems, msg.size() - off);
    if (k >= mb->slots)
      while (mb->credit.load(std::memory_order_acquire) < k - mb->slots + 1) std::this_thread::yield();
    int64_t* dst = mb->data.data() + (k % mb->slots) * mb->slot_elems;
    for (uint64_t i = 0; i < len; ++i) dst[i] = msg[off + i];
    mb->flag.store(k + 1, std::memory_order_release);
  }
}

void MailboxRecv(Mailbox* mb, std::vector<int64_t>* msg, uint64_t first_piece) {
  const uint64_t pieces = (msg->size() + mb->slot_elems - 1) / mb->slot_elems;
  for (uint64_t j = 0; j < pieces; ++j) {
    const uint64_t k = first_piece + j, off = j * mb->slot_elems;
    const uint64_t len = std::min<uint64_t>(mb->slot_elems, msg->size() - off);
    while (mb->flag.load(std::memory_order_acquire) < k + 1) std::this_thread::yield();
    const int64_t* src = mb->data.data() + (k % mb->slots) * mb->slot_elems;
    for (uint64_t i = 0; i < len; ++i) (*msg)[off + i] = src[i];
    mb->credit.store(k + 1, std::memory_order_release);
  }
}

}  // namespace

MINI_TEST(MailboxProtocol) {
  // Messages of many lengths, one after the other, through a mailbox of two slots.
  Mailbox mb(2, 64);
  const std::vector<size_t> lengths = {1, 63, 64, 65, 128, 1000, 5, 4096, 129};
  std::vector<std::vector<int64_t>> got;
  for (size_t n : lengths) got.emplace_back(n, -1);
  std::thread sender([&] {
    uint64_t piece = 0;
    for (size_t m = 0; m < lengths.size(); ++m) {
      std::vector<int64_t> msg(lengths[m]);
      for (size_t i = 0; i < msg.size(); ++i) msg[i] = Value(static_cast<int>(m), i);
      MailboxSend(&mb, msg, piece);
      piece += (lengths[m] + mb.slot_elems - 1) / mb.slot_elems;
    }
  });
  std::thread receiver([&] {
    uint64_t piece = 0;
    for (size_t m = 0; m < lengths.size(); ++m) {
      MailboxRecv(&mb, &got[m], piece);
      piece += (lengths[m] + mb.slot_elems - 1) / mb.slot_elems;
    }
  });
  sender.join();
  receiver.join();
  for (size_t m = 0; m < lengths.size(); ++m)
    for (size_t i = 0; i < got[m].size(); ++i) CHECK_EQ(got[m][i], Value(static_cast<int>(m), i));
}

MINI_TEST(OneShotParityProtocol) {
  // Calls of changing length and CTA count back to back, no barrier between them.
  std::vector<std::pair<uint64_t, int>> calls;
  const std::pair<uint64_t, int> pattern[] = {{100, 1}, {1000, 4}, {37, 1}, {1000, 3}, {1024, 8}, {64, 2}, {5, 1}, {999, 5}};
  for (int rep = 0; rep < 6; ++rep)
    for (const auto& c : pattern) calls.push_back(c);
  for (int ws : {2, 3, 4}) CHECK_TRUE(RunOneShot(ws, calls));
}

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

MINI_TEST(PipelinedStagedProtocol) {
  // Windows of 256 elements (64 vectors): messages of one to nine windows, the last one short.
  for (int ws : {2, 3, 4})
    for (int ncta : {1, 2, 3})
      for (uint64_t nvec : {uint64_t(1), uint64_t(9), uint64_t(64), uint64_t(65), uint64_t(200), uint64_t(513)})
        CHECK_TRUE(RunPipelined(ws, ncta, nvec, 256));
  // Split mode: several groups per role, up to six windows of each kind.
  for (int ws : {2, 3})
    for (int bufs : {3, 4, 6})
      for (int lg : {1, 3, 4})
        for (int rg : {1, 2, 3})
          for (uint64_t nvec : {uint64_t(9), uint64_t(200), uint64_t(1100)})
            CHECK_TRUE(RunPipelined(ws, 2, nvec, 256, bufs, lg, rg, lg == 4 ? 2 : 3, (bufs + lg + rg) % 2 == 0));
}

MINI_TEST(HybridSplitProtocol) {
  for (int ws : {2, 3, 4})
    for (int na : {1, 2})
      for (int nb : {1, 3})
        for (uint64_t n : {uint64_t(8), uint64_t(403), uint64_t(1024), uint64_t(2051)})
          for (uint64_t split : {uint64_t(0), uint64_t(1), n / kVec / 2, n / kVec, n})
            CHECK_TRUE(RunHybrid(ws, na, nb, n, split));
}

MINI_TEST(RandomStagedConfigurations) {
  // Seeded fuzz over world size, CTAs, message length and window capacity.
  uint64_t state = 88172645463325252ull;
  auto next = [&] {
    state ^= state << 13;
    state ^= state >> 7;
    state ^= state << 17;
    return state;
  };
  auto pick = [&](uint64_t lo, uint64_t hi) { return lo + next() % (hi - lo + 1); };
  for (int it = 0; it < 200; ++it) {
    const int ws = static_cast<int>(pick(2, 5)), ncta = static_cast<int>(pick(1, 5));
    const uint64_t cap = pick(4, 40) * 16;  // a whole number of vectors
    CHECK_TRUE(RunAllreduce(ws, ncta, pick(static_cast<uint64_t>(ws), 6 * cap), cap));
    CHECK_TRUE(RunRsAg(ws, ncta, pick(1, 6 * cap / kVec), cap / kVec));
    if (it % 4 == 0) CHECK_TRUE(RunPipelined(std::min(ws, 4), std::min(ncta, 3), pick(1, 6 * cap / kVec), cap));
  }
}

int main(int argc, char** argv) { return mini::RunAll(argc > 1 ? argv[1] : nullptr); }
