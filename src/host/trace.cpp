#include "ibcomm/trace.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "ibcomm/env.h"
#include "ibcomm/error.h"

namespace ibcomm {

static const char* const kNames[kTraceNumCategories] = {
    "received", "reduced", "issue_send", "issue_copy_kernel", "issue_redu_kernel", "issue_recv", "other"};

const char* TraceCategoryName(int c) {
  return (c >= 0 && c < kTraceNumCategories) ? kNames[c] : "?";
}

Tracer::Tracer() {
#ifdef USE_TRACE
  enabled_ = true;
#else
  const char* s = getenv("IBCOMM_TRACE");
  enabled_ = (s != nullptr && s[0] != '\0' && strcmp(s, "0") != 0);
#endif
  clock_gettime(CLOCK_MONOTONIC_RAW, &base_);
}

void Tracer::SetTimerBase() { clock_gettime(CLOCK_MONOTONIC_RAW, &base_); }

void Tracer::StampAlways(TraceCategory c) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC_RAW, &ts);
  stamps_[c].push_back(ts);
}

void Tracer::AddInterval(TraceCategory c, double start_ns, double dur_ns) {
  if (!enabled_) return;
  auto mk = [this](double ns) {
    struct timespec t = base_;
    long long add = static_cast<long long>(ns);
    t.tv_sec += add / 1000000000ll;
    t.tv_nsec += add % 1000000000ll;
    if (t.tv_nsec >= 1000000000l) {
      t.tv_nsec -= 1000000000l;
      t.tv_sec += 1;
    }
    return t;
  };
  stamps_[c].push_back(mk(start_ns));
  stamps_[c].push_back(mk(start_ns + dur_ns));
}

static double MsSince(const struct timespec& base, const struct timespec& t) {
  return (static_cast<double>(t.tv_sec - base.tv_sec) * 1e3) +
         (static_cast<double>(t.tv_nsec - base.tv_nsec) * 1e-6);
}

std::string Tracer::Dump(int rank) const {
  if (!enabled_) return std::string();
  std::string path = env::ReadTraceFile() + "_" + std::to_string(rank) + ".dat";
  FILE* f = fopen(path.c_str(), "w");
  if (f == nullptr) {
    IBCOMM_WARN("cannot open trace file %s\n", path.c_str());
    return std::string();
  }
  for (int c = 0; c < kTraceNumCategories; ++c) {
    fprintf(f, "%s,", kNames[c]);
    const auto& v = stamps_[c];
    for (size_t i = 0; i + 1 < v.size(); i += 2) {
      double start = MsSince(base_, v[i]);
      double dur = MsSince(v[i], v[i + 1]);
      fprintf(f, "%e,%e,", start, dur);
    }
    fputc('\n', f);
  }
  fclose(f);
  return path;
}

}  // namespace ibcomm
