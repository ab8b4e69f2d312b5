// Algorithm and channel selection by message size.
//
// The defaults below come from bus-bandwidth sweeps on an 8 x B200 NVSwitch
// box (bench.py --sweep); IBCOMM_TUNING_FILE replaces them with a table of
// lines "world_size max_bytes algorithm channels" (first matching line wins,
// max_bytes 0 = no limit), which bench.py --sweep --write-tuning produces.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <string>
#include <vector>

#include "ibcomm/device_context.h"
#include "ibcomm/tunables.h"

namespace ibcomm {

namespace {

struct Rule {
  int world_size;  // 0 = any
  size_t max_bytes;  // 0 = unlimited
  Algo algo;
  int channels;  // 0 = derive from the size
};

std::vector<Rule> g_rules;
std::once_flag g_once;

void LoadRules() {
  std::string path = env::ReadTuningFile();
  if (path.empty()) return;
  FILE* f = fopen(path.c_str(), "r");
  if (f == nullptr) {
    IBCOMM_WARN("cannot open IBCOMM_TUNING_FILE '%s'; using built-in tuning.\n", path.c_str());
    return;
  }
  char line[256];
  while (fgets(line, sizeof(line), f) != nullptr) {
    if (line[0] == '#' || line[0] == '\n') continue;
    int ws = 0, ch = 0;
    unsigned long long mb = 0;
    char name[64] = {0};
    if (sscanf(line, "%d %llu %63s %d", &ws, &mb, name, &ch) != 4) continue;
    std::string n = name;
    Algo a;
    if (n == "ring") a = Algo::kRing;
    else if (n == "rabenseifner") a = Algo::kRabenseifner;
    else if (n == "nvls") a = Algo::kNvls;
    else if (n == "oneshot") a = Algo::kOneShot;
    else if (n == "direct") a = Algo::kDirect;
    else continue;
    g_rules.push_back(Rule{ws, static_cast<size_t>(mb), a, ch});
  }
  fclose(f);
}

}  // namespace

int ChooseChannels(Algo algo, size_t bytes, int world_size, int max_channels) {
  max_channels = std::max(1, std::min(max_channels, kMaxChannels));
  int ch;
  switch (algo) {
    case Algo::kOneShot:
      // One CTA per 32 KiB keeps the flag fan-out small at the latency end; a
      // CTA sustains about 10 GB/s of peer stores, so megabyte messages get
      // up to 96 of them.
      ch = static_cast<int>(std::min<size_t>(96, (bytes + (32u << 10) - 1) / (32u << 10)));
      break;
    case Algo::kNvls:
      // The switch does the math; 32-64 CTAs saturate it (more only add
      // barrier traffic).
      ch = static_cast<int>(std::min<size_t>(64, std::max<size_t>(1, bytes / (128u << 10))));
      break;
    case Algo::kDirect:
      // Peer loads are latency-bound: as many CTAs as there are SMs to spare.
      ch = static_cast<int>(std::min<size_t>(128, std::max<size_t>(1, bytes / (128u << 10))));
      break;
    default: {
      // Ring / Rabenseifner: a chunk is bytes / (4 * ws); give every channel
      // at least 16 KiB of it per step.  More channels than needed to fill the
      // links hide the flag round trips of the others.
      size_t chunk = bytes / static_cast<size_t>(4 * std::max(1, world_size));
      ch = static_cast<int>(std::min<size_t>(kMaxChannels, std::max<size_t>(1, chunk / (16u << 10))));
      break;
    }
  }
  return std::max(1, std::min(ch, max_channels));
}

// Largest message of ordinary buffers that goes one-shot.  A one-shot call
// moves (ws - 1) S per direction against the two-shot's 2 S (ws - 1) / ws but
// needs one synchronisation instead of three; with two ranks the byte counts
// are equal and only the slot size limits it.
static size_t OneShotLimit(int world_size) {
  const int knob = Tunable("IBCOMM_ONESHOT_MAX_KIB", 0);
  if (knob > 0) return static_cast<size_t>(knob) << 10;
  if (world_size <= 2) return 16u << 20;
  if (world_size <= 4) return 2u << 20;
  return 1u << 20;
}

TunerChoice ChooseAlgorithm(size_t bytes, int world_size, bool nvls_available, bool zero_copy, int max_channels) {
  std::call_once(g_once, LoadRules);
  for (const Rule& r : g_rules) {
    if (r.world_size != 0 && r.world_size != world_size) continue;
    if (r.max_bytes != 0 && bytes > r.max_bytes) continue;
    if (r.algo == Algo::kNvls && !nvls_available) continue;
    int ch = r.channels > 0 ? std::min(r.channels, max_channels) : ChooseChannels(r.algo, bytes, world_size, max_channels);
    return TunerChoice{r.algo, ch};
  }
  // Built-in table, from bus-bandwidth sweeps on 2 and 8 B200 (profiles/).
  Algo a;
  if (zero_copy) {
    // Buffers every peer maps (symmetric memory): nothing is staged.
    if (world_size <= 2) {
      // Two ranks: one push each is all the traffic an allreduce needs, and it
      // takes one synchronisation instead of three (12-23 us up to 4 MiB
      // against 13-25 us for the two-shot kernels); above, peer loads in
      // place.  The switch path moves 1.5 S per direction against 1.0 S and
      // loses at every size.
      a = bytes <= (4u << 20) ? Algo::kOneShot : Algo::kDirect;
    } else if (bytes <= (16u << 10)) {
      a = Algo::kOneShot;
    } else if (nvls_available) {
      a = Algo::kNvls;  // in-switch reduction: 1 + 1/ws of the message per direction
    } else {
      // Peer-mapped without the switch (registered buffers, no multicast):
      // one push per peer wins while the fan-out is small.
      a = bytes <= (world_size > 4 ? (16u << 10) : (512u << 10)) ? Algo::kOneShot : Algo::kDirect;
    }
  } else if (bytes <= OneShotLimit(world_size)) {
    a = Algo::kOneShot;  // ordinary buffers: one push per peer beats three staged phases
  } else if (nvls_available && world_size > 2) {
    a = Algo::kNvls;  // through the pool, pipelined inside the kernel (staged_kernel.cu)
  } else if (world_size > 2 && bytes <= (32u << 20)) {
    a = Algo::kDirect;  // staged direct two-shot, pipelined inside the kernel
  } else {
    // Large messages in ordinary memory without the switch, and two ranks: the
    // chunk-pipelined programs keep their staging inside the transfer (two
    // ranks, one 512-thread block per SM: 89 / 137 / 238 / 440 us at 32 / 64 /
    // 128 / 256 MiB against the staged direct kernel's 98 / 154 / 264 / 462).
    // Halving/doubling needs fewer steps.
    a = (world_size > 2 && util::GetExpOfTwo(static_cast<uint64_t>(world_size)) != 0) ? Algo::kRabenseifner : Algo::kRing;
  }
  int ch = ChooseChannels(a, bytes, world_size, max_channels);
  // Staged switch path: the copies in and out of the pool run on the same
  // CTAs, and 64 of them cannot pull full HBM bandwidth.
  if (a == Algo::kNvls && !zero_copy) ch = std::max(ch, ChooseChannels(Algo::kDirect, bytes, world_size, max_channels));
  return TunerChoice{a, ch};
}

}  // namespace ibcomm
