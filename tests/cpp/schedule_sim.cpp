// Schedule simulator tests: every rank's op program is interpreted on CPU
// threads (program_interp.h) for world sizes 1..8, message lengths around
// chunk boundaries, few and many staging slots, one and several channels, in
// place and out of place.  Results are compared with the exact integer sum;
// the per-pair transfer counts of sender and receiver must agree.
#include <cstdio>
#include <random>

#include "ibcomm/program_interp.h"
#include "mini_test.h"

using namespace ibcomm;

template <typename T>
static bool RunCase(Algo algo, int ws, size_t n, int64_t env_chunk, size_t stage_bytes, int nch, bool in_place,
                    double scale, size_t max_chunk_bytes = 0, size_t piece_elems = 0) {
  std::vector<Range> ranges = SplitForDevice(n, sizeof(T), static_cast<size_t>(ws), env_chunk, max_chunk_bytes);
  std::vector<std::vector<T>> in(static_cast<size_t>(ws), std::vector<T>(n)), out;
  std::mt19937 gen(static_cast<unsigned>(n * 31 + static_cast<size_t>(ws)));
  for (int r = 0; r < ws; ++r)
    for (size_t i = 0; i < n; ++i) in[static_cast<size_t>(r)][i] = static_cast<T>(static_cast<int>(gen() % 2001) - 1000);
  ProgramSimulator<T> sim(algo, ws, stage_bytes, nch, piece_elems);
  SimResult res = sim.Run(ranges, in, &out, scale, in_place);
  if (!res.ok) {
    fprintf(stderr, "%s ws=%d n=%zu: %s", AlgoName(algo), ws, n, res.error.c_str());
    return false;
  }
  // transfer-count audit
  const auto& progs = sim.programs();
  for (int a = 0; a < ws; ++a)
    for (int b = 0; b < ws; ++b)
      if (progs[static_cast<size_t>(a)].sent_to[b] != progs[static_cast<size_t>(b)].received_from[a]) {
        fprintf(stderr, "%s ws=%d: %d->%d sends %u, receiver expects %u\n", AlgoName(algo), ws, a, b,
                progs[static_cast<size_t>(a)].sent_to[b], progs[static_cast<size_t>(b)].received_from[a]);
        return false;
      }
  for (size_t i = 0; i < n; ++i) {
    double want = 0;
    for (int r = 0; r < ws; ++r) want += static_cast<double>(in[static_cast<size_t>(r)][i]);
    want *= scale;
    for (int r = 0; r < ws; ++r) {
      if (static_cast<double>(out[static_cast<size_t>(r)][i]) != static_cast<double>(static_cast<T>(want))) {
        fprintf(stderr, "%s ws=%d n=%zu nch=%d rank %d elem %zu: got %g want %g\n", AlgoName(algo), ws, n, nch, r, i,
                static_cast<double>(out[static_cast<size_t>(r)][i]), want);
        return false;
      }
    }
  }
  return true;
}

MINI_TEST(RingAllWorldSizes) {
  for (int ws = 2; ws <= 8; ++ws)
    for (size_t n : {size_t(ws), size_t(2 * ws), size_t(2521), size_t(4096), size_t(100003)})
      for (size_t stage : {size_t(1) << 22, size_t(1) << 16})
        CHECK_TRUE(RunCase<int>(Algo::kRing, ws, n, 0, stage, 1, false, 1.0, stage / 4));
}

MINI_TEST(RabenseifnerAllWorldSizes) {
  for (int ws = 2; ws <= 8; ++ws)
    for (size_t n : {size_t(ws), size_t(2 * ws), size_t(2521), size_t(4096), size_t(100003)})
      for (size_t stage : {size_t(1) << 22, size_t(1) << 17})
        CHECK_TRUE(RunCase<int>(Algo::kRabenseifner, ws, n, 0, stage, 1, false, 1.0, stage / 16));
}

MINI_TEST(TwoSlotsOnly) {
  // Exactly two slots per region: the tightest legal staging area.
  for (int ws = 2; ws <= 8; ++ws) {
    const size_t n = 64 * 4 * static_cast<size_t>(ws) * 3;  // chunks of 192 ints = 768 bytes
    std::vector<Range> rg = SplitForDevice(n, 4, static_cast<size_t>(ws), 0, 0);
    const size_t slot = (MaxChunkElems(rg) * 4 + 127) / 128 * 128;
    CHECK_TRUE(RunCase<int>(Algo::kRing, ws, n, 0, 2 * slot * static_cast<size_t>(NumRegions(Algo::kRing, ws)), 1, false, 1.0));
    CHECK_TRUE(RunCase<int>(Algo::kRabenseifner, ws, n, 0,
                            2 * slot * static_cast<size_t>(NumRegions(Algo::kRabenseifner, ws)), 1, false, 1.0));
  }
}

MINI_TEST(ChannelsInPlaceScale) {
  for (Algo a : {Algo::kRing, Algo::kRabenseifner})
    for (int ws : {2, 3, 4, 5, 6, 7, 8}) {
      CHECK_TRUE(RunCase<int>(a, ws, 70001, 0, size_t(1) << 20, 3, true, 1.0));
      CHECK_TRUE(RunCase<double>(a, ws, 33333, 0, size_t(1) << 20, 2, false, 0.25));
      CHECK_TRUE(RunCase<double>(a, ws, 4096, 0, size_t(1) << 20, 4, true, 0.5));
    }
}

MINI_TEST(SlotReuseWithSeveralChannels) {
  // Small staging areas (every slot is reused many times), lengths that make
  // the last chunk shorter than the others, several channels: the byte range
  // a channel owns inside a slot must not depend on the chunk in it.
  for (Algo a : {Algo::kRing, Algo::kRabenseifner})
    for (int ws : {2, 3, 4, 5, 7, 8})
      for (int nch : {2, 4, 5}) {
        const size_t stage = 400000;
        const size_t maxc = stage / (static_cast<size_t>(NumRegions(a, ws)) * 4) / 128 * 128;
        CHECK_TRUE(RunCase<int>(a, ws, 100000, 0, stage, nch, false, 1.0, maxc));
        CHECK_TRUE(RunCase<int>(a, ws, 10007, 0, 40000, nch, true, 1.0, 40000 / (static_cast<size_t>(NumRegions(a, ws)) * 4) / 128 * 128));
      }
}

MINI_TEST(RabenseifnerMergedPieces) {
  // Transfer pieces that ignore chunk boundaries: larger than a chunk, smaller
  // than a chunk, and not a divisor of anything; tight staging and several channels.
  for (int ws = 2; ws <= 8; ++ws)
    for (size_t piece : {size_t(32), size_t(1000), size_t(4096), size_t(100000)})
      for (int nch : {1, 3}) {
        CHECK_TRUE(RunCase<int>(Algo::kRabenseifner, ws, 100003, 0, size_t(1) << 22, nch, false, 1.0, 0, piece));
        const size_t regions = static_cast<size_t>(NumRegions(Algo::kRabenseifner, ws));
        CHECK_TRUE(RunCase<int>(Algo::kRabenseifner, ws, 50000, 0, 2 * regions * ((piece * 4 + 127) / 128 * 128), nch, true, 1.0, 0, piece));
      }
}

MINI_TEST(EnvChunkSizes) {
  for (int64_t chunk : {4, 8, 16, 32, 64, 128})
    CHECK_TRUE(RunCase<int>(Algo::kRing, 4, 256, chunk, size_t(1) << 16, 1, false, 1.0));
  CHECK_TRUE(RunCase<int>(Algo::kRabenseifner, 4, 256, 32, size_t(1) << 16, 1, false, 1.0));
}

MINI_TEST(RingOwnershipAfterReduceScatter) {
  // The op that stores locally with the scale flag marks the block a rank owns
  // after the reduce-scatter: it must be the block of rank r+1.
  const int ws = 4;
  std::vector<Range> rg = SplitForDevice(1600, 4, ws, 0, 0);
  auto blocks = GetRankToChunk(rg.size(), ws);
  for (int r = 0; r < ws; ++r) {
    ProgramRequest q;
    q.algo = Algo::kRing; q.rank = r; q.world_size = ws; q.ranges = rg; q.stage_bytes = 1 << 20; q.apply_scale = true;
    Program p = BuildProgram(q);
    std::vector<uint64_t> owned;
    for (const Op& op : p.ops)
      if (op.flags & kOpScale) owned.push_back(op.elem_begin);
    std::vector<uint64_t> want;
    for (auto it = blocks[(r + 1) % ws].rbegin(); it != blocks[(r + 1) % ws].rend(); ++it) want.push_back(rg[*it].first);
    CHECK_TRUE(owned == want);
    // first op: own block's highest chunk, straight from the send buffer
    CHECK_EQ(p.ops[0].src_a, uint8_t(kSrcSend));
    CHECK_EQ(p.ops[0].elem_begin, uint64_t(rg[blocks[r].back()].first));
  }
}

MINI_TEST(RandomConfigurations) {
  // Seeded fuzz over world size, length, channels, staging size, in-place and scale: the directed cases
  // above came from bugs that only some combinations showed.
  std::mt19937 gen(20240607u);
  auto pick = [&](size_t lo, size_t hi) { return lo + static_cast<size_t>(gen() % (hi - lo + 1)); };
  for (int it = 0; it < 250; ++it) {
    const Algo a = (gen() & 1u) ? Algo::kRing : Algo::kRabenseifner;
    const int ws = static_cast<int>(pick(2, 8));
    const size_t n = (gen() % 4 == 0) ? pick(static_cast<size_t>(ws), 64) : pick(static_cast<size_t>(ws), 150000);
    const int nch = static_cast<int>(pick(1, 6));
    const size_t stage = pick(40000, size_t(1) << 20);
    const size_t maxc = std::max<size_t>(128, stage / (static_cast<size_t>(NumRegions(a, ws)) * 4) / 128 * 128);
    const bool in_place = (gen() & 1u) != 0;
    bool ok;
    if (gen() % 3 == 0) ok = RunCase<double>(a, ws, n, 0, stage, nch, in_place, 0.5, maxc);
    else ok = RunCase<int>(a, ws, n, 0, stage, nch, in_place, 1.0, maxc);
    if (!ok) fprintf(stderr, "failing configuration: %s ws=%d n=%zu nch=%d stage=%zu in_place=%d\n", AlgoName(a), ws, n, nch, stage, in_place ? 1 : 0);
    CHECK_TRUE(ok);
  }
}

MINI_TEST(ValidateProgramFindsOutOfBoundsOps) {
  // Every program the builders cut passes; an op pushed out of the message,
  // out of its slot or out of the staging area is named.
  for (Algo algo : {Algo::kRing, Algo::kRabenseifner})
    for (int ws : {2, 3, 5, 8}) {
      const size_t n = 100003;
      std::vector<Range> rg = SplitForDevice(n, 4, ws, 0, 0);
      for (int r = 0; r < ws; ++r) {
        ProgramRequest q;
        q.algo = algo; q.rank = r; q.world_size = ws; q.ranges = rg; q.stage_bytes = 1 << 20;
        Program p = BuildProgram(q);
        CHECK_TRUE(ValidateProgram(p, n, 4, ws).empty());
        CHECK_TRUE(!ValidateProgram(p, n / 2, 4, ws).empty());  // the same ops against a shorter message
        Program bad = p;
        for (Op& op : bad.ops)
          if (op.flags & kOpStoreRemote) { op.slot_out = bad.stage.slots; break; }
        CHECK_TRUE(ValidateProgram(bad, n, 4, ws).find("output slot") != std::string::npos);
        bad = p;
        bad.stage.slot_bytes = 64;
        CHECK_TRUE(ValidateProgram(bad, n, 4, ws).find("does not fit") != std::string::npos);
      }
    }
}

int main(int argc, char** argv) { return mini::RunAll(argc > 1 ? argv[1] : nullptr); }
