// Host-side trace of the communicator, in the reference's seven categories
// and file format (ibverbs_communicator.h:168-189, ibverbs_communicator.cpp:157-216):
// one line per category, "name," followed by "start_ms,duration_ms," pairs in
// scientific notation, written to "<IBCOMM_TRACE_FILE or ibcomm_trace>_<rank>.dat".
// Stamps come in begin/end pairs.  Tracing is active when the library is built
// with -DUSE_TRACE or when IBCOMM_TRACE=1 is set at run time.  Device kernels
// add per-step %globaltimer stamps that DumpTrace converts into the same pairs
// (category "received" = wait satisfied, "reduced" = step finished).
#pragma once

#include <time.h>

#include <string>
#include <vector>

namespace ibcomm {

enum TraceCategory : int {
  kTraceReceived = 0,
  kTraceReduced,
  kTraceIssueSend,
  kTraceIssueCopyKernel,
  kTraceIssueReduKernel,
  kTraceIssueRecv,
  kTraceOther,
  kTraceNumCategories
};

class Tracer {
 public:
  Tracer();
  bool enabled() const { return enabled_; }
  void set_enabled(bool e) { enabled_ = e; }
  void SetTimerBase();
  void Stamp(TraceCategory c) {
    if (enabled_) StampAlways(c);
  }
  // Adds a finished interval given in nanoseconds relative to the timer base.
  void AddInterval(TraceCategory c, double start_ns, double dur_ns);
  // Writes <prefix>_<rank>.dat; returns the path ("" when disabled or empty).
  std::string Dump(int rank) const;
  size_t Count(TraceCategory c) const { return stamps_[c].size(); }
  const struct timespec& base() const { return base_; }

 private:
  void StampAlways(TraceCategory c);
  bool enabled_;
  struct timespec base_;
  std::vector<struct timespec> stamps_[kTraceNumCategories];
};

const char* TraceCategoryName(int c);

}  // namespace ibcomm

#define IBCOMM_TRACE(tracer, cat) (tracer).Stamp(::ibcomm::cat)
