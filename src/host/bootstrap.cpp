#include "ibcomm/bootstrap.h"

#include <errno.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <thread>

namespace ibcomm {

static int EnvInt(const char* a, const char* b, int dflt) {
  const char* s = getenv(a);
  if (s == nullptr && b != nullptr) s = getenv(b);
  return s ? atoi(s) : dflt;
}

BootstrapEnv ReadBootstrapEnv() {
  BootstrapEnv e;
  e.rank = EnvInt("IBCOMM_RANK", "RANK", 0);
  e.world_size = EnvInt("IBCOMM_WORLD_SIZE", "WORLD_SIZE", 1);
  e.local_rank = EnvInt("IBCOMM_LOCAL_RANK", "LOCAL_RANK", e.rank);
  const char* d = getenv("IBCOMM_BOOTSTRAP_DIR");
  if (d != nullptr) e.dir = d;
  if (e.world_size < 1 || e.rank < 0 || e.rank >= e.world_size)
    IBCOMM_FAIL(INVALID_ARGUMENT, "Bad bootstrap environment: rank %d of %d.\n", e.rank, e.world_size);
  return e;
}

static std::string InfoPath(const BootstrapEnv& env, const std::string& tag, int src, int dst) {
  return env.dir + "/" + tag + ".qp." + std::to_string(src) + "." + std::to_string(dst);
}

void ConnectAll(Communicator* comm, const BootstrapEnv& env, const std::string& tag, int timeout_ms) {
  if (!comm->initialized()) comm->Init(env.world_size);
  comm->RegisterMyself(env.rank);
  if (env.world_size == 1) return;
  if (env.dir.empty())
    IBCOMM_FAIL(INVALID_ARGUMENT,
                "IBCOMM_BOOTSTRAP_DIR is not set; start the ranks with ibcomm_run.\n");
  for (int d = 0; d < env.world_size; ++d) {
    if (d == env.rank) continue;
    ProcessInfo mine = comm->CreateQueuePair(d);
    std::string path = InfoPath(env, tag, env.rank, d);
    std::string tmp = path + ".tmp";
    FILE* f = fopen(tmp.c_str(), "w");
    if (f == nullptr) IBCOMM_FAIL(TRANSPORT_ERROR, "cannot write %s: %s\n", tmp.c_str(), strerror(errno));
    fprintf(f, "%u %u %u\n", static_cast<unsigned>(mine.lid), mine.qp_n, mine.psn);
    fclose(f);
    if (rename(tmp.c_str(), path.c_str()) != 0)
      IBCOMM_FAIL(TRANSPORT_ERROR, "cannot publish %s: %s\n", path.c_str(), strerror(errno));
  }
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (int d = 0; d < env.world_size; ++d) {
    if (d == env.rank) continue;
    std::string path = InfoPath(env, tag, d, env.rank);
    for (;;) {
      FILE* f = fopen(path.c_str(), "r");
      if (f != nullptr) {
        unsigned lid = 0, qpn = 0, psn = 0;
        int got = fscanf(f, "%u %u %u", &lid, &qpn, &psn);
        fclose(f);
        if (got == 3) {
          ProcessInfo pi;
          pi.lid = static_cast<uint16_t>(lid);
          pi.qp_n = qpn;
          pi.psn = psn;
          comm->RegisterQueuePair(d, pi);
          break;
        }
      }
      if (std::chrono::steady_clock::now() > deadline)
        IBCOMM_FAIL(TRANSPORT_ERROR, "Bootstrap: rank %d never published its endpoint for rank %d.\n", d,
                    env.rank);
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
  }
  // Nobody may leave (and take its endpoints away) before everybody attached.
  comm->Barrier();
}

BootstrapEnv SubsetEnv(const BootstrapEnv& env, const std::vector<int>& ranks, std::string* tag) {
  BootstrapEnv sub = env;
  sub.rank = -1;
  std::string suffix = ".sub";
  for (size_t i = 0; i < ranks.size(); ++i) {
    const int r = ranks[i];
    if (r < 0 || r >= env.world_size) IBCOMM_FAIL(INVALID_ARGUMENT, "SubsetEnv: rank %d is not a rank of this job (%d ranks).\n", r, env.world_size);
    for (size_t j = 0; j < i; ++j)
      if (ranks[j] == r) IBCOMM_FAIL(INVALID_ARGUMENT, "SubsetEnv: rank %d is listed twice.\n", r);
    if (r == env.rank) sub.rank = static_cast<int>(i);
    suffix += (i == 0 ? "" : "_") + std::to_string(r);
  }
  if (sub.rank < 0) IBCOMM_FAIL(INVALID_ARGUMENT, "SubsetEnv: rank %d is not in the list.\n", env.rank);
  sub.world_size = static_cast<int>(ranks.size());
  if (tag != nullptr) *tag += suffix;
  return sub;
}

long long SumOverRanks(Communicator* comm, long long value) {
  const int ws = static_cast<int>(comm->world_size());
  if (ws == 1) return value;
  long long total = value;
  if (comm->rank() == 0) {
    for (int r = 1; r < ws; ++r) {
      long long v = 0;
      comm->Recv(r, &v, sizeof(v), true);
      total += v;
    }
  } else {
    comm->Send(0, &value, sizeof(value), true);
  }
  comm->Bcast(&total, sizeof(total), 0);
  return total;
}

}  // namespace ibcomm
