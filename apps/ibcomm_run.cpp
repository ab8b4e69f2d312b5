// ibcomm_run — minimal process launcher for one host (stands in for mpiexec,
// which the reference's harness relies on: tests/allreduce_test.py:89).
//
//   ibcomm_run -np N [-x NAME=VALUE]... [--] program [args...]
//
// Starts N copies of `program` with IBCOMM_RANK / IBCOMM_LOCAL_RANK /
// IBCOMM_WORLD_SIZE / IBCOMM_BOOTSTRAP_DIR set (RANK, LOCAL_RANK, WORLD_SIZE
// as well), waits for them and returns the first non-zero exit status in rank
// order (128 + signal for a killed rank).  When one rank fails, the others get
// a grace period (IBCOMM_RUN_GRACE_MS, default 5000) and are then killed, so a
// failed job cannot hang the caller.
#include <errno.h>
#include <signal.h>
#include <sys/stat.h>
#include <sys/types.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

static void Usage() {
  fprintf(stderr, "usage: ibcomm_run -np N [-x NAME=VALUE]... [--] program [args...]\n");
  exit(1);
}

static void RemoveDir(const std::string& dir) {
  std::string cmd = "rm -rf '" + dir + "'";
  if (system(cmd.c_str()) != 0) {
  }
}

int main(int argc, char** argv) {
  int np = 1;
  std::vector<std::string> envs;
  int i = 1;
  for (; i < argc; ++i) {
    std::string a = argv[i];
    if ((a == "-np" || a == "-n") && i + 1 < argc) {
      np = atoi(argv[++i]);
    } else if (a == "-x" && i + 1 < argc) {
      envs.push_back(argv[++i]);
    } else if (a == "--") {
      ++i;
      break;
    } else {
      break;
    }
  }
  if (i >= argc || np < 1) Usage();

  char tmpl[] = "/tmp/ibcomm_run.XXXXXX";
  if (mkdtemp(tmpl) == nullptr) {
    perror("mkdtemp");
    return 1;
  }
  const std::string dir = tmpl;

  std::vector<pid_t> pids(static_cast<size_t>(np), -1);
  for (int r = 0; r < np; ++r) {
    pid_t pid = fork();
    if (pid < 0) {
      perror("fork");
      for (int k = 0; k < r; ++k) kill(pids[static_cast<size_t>(k)], SIGKILL);
      RemoveDir(dir);
      return 1;
    }
    if (pid == 0) {
      std::string rs = std::to_string(r), ws = std::to_string(np);
      setenv("IBCOMM_RANK", rs.c_str(), 1);
      setenv("IBCOMM_LOCAL_RANK", rs.c_str(), 1);
      setenv("IBCOMM_WORLD_SIZE", ws.c_str(), 1);
      setenv("IBCOMM_BOOTSTRAP_DIR", dir.c_str(), 1);
      setenv("RANK", rs.c_str(), 1);
      setenv("LOCAL_RANK", rs.c_str(), 1);
      setenv("WORLD_SIZE", ws.c_str(), 1);
      for (const std::string& kv : envs) {
        size_t eq = kv.find('=');
        if (eq == std::string::npos) continue;
        setenv(kv.substr(0, eq).c_str(), kv.substr(eq + 1).c_str(), 1);
      }
      execvp(argv[i], argv + i);
      fprintf(stderr, "ibcomm_run: cannot execute %s: %s\n", argv[i], strerror(errno));
      _exit(127);
    }
    pids[static_cast<size_t>(r)] = pid;
  }

  const char* g = getenv("IBCOMM_RUN_GRACE_MS");
  const int grace_ms = g ? atoi(g) : 5000;
  std::vector<int> status(static_cast<size_t>(np), -1);
  int remaining = np;
  bool failed = false;
  auto fail_time = std::chrono::steady_clock::now();
  while (remaining > 0) {
    int st = 0;
    pid_t done = waitpid(-1, &st, failed ? WNOHANG : 0);
    if (done > 0) {
      for (int r = 0; r < np; ++r) {
        if (pids[static_cast<size_t>(r)] != done) continue;
        int code = WIFEXITED(st) ? WEXITSTATUS(st) : 128 + (WIFSIGNALED(st) ? WTERMSIG(st) : 0);
        status[static_cast<size_t>(r)] = code;
        --remaining;
        if (code != 0 && !failed) {
          failed = true;
          fail_time = std::chrono::steady_clock::now();
        }
      }
      continue;
    }
    if (done < 0 && errno != EINTR) break;
    if (failed) {
      if (std::chrono::steady_clock::now() - fail_time > std::chrono::milliseconds(grace_ms)) {
        for (int r = 0; r < np; ++r)
          if (status[static_cast<size_t>(r)] < 0) kill(pids[static_cast<size_t>(r)], SIGKILL);
        failed = false;  // block in waitpid for the killed ones
        fail_time = std::chrono::steady_clock::now();
      } else {
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
      }
    }
  }
  RemoveDir(dir);
  // A rank that failed on its own wins over ranks this launcher had to kill.
  for (int r = 0; r < np; ++r) {
    int c = status[static_cast<size_t>(r)];
    if (c > 0 && c < 128) return c;
  }
  for (int r = 0; r < np; ++r)
    if (status[static_cast<size_t>(r)] != 0) return status[static_cast<size_t>(r)] < 0 ? 1 : status[static_cast<size_t>(r)];
  return 0;
}
