// Host-side plumbing shared by the multi-GPU DeviceContext and the one-GPU
// EmuWorld: arena layout, per-rank resources, the program cache and the
// parameter blocks of the kernels.
#pragma once

#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <tuple>
#include <vector>

#include "ibcomm/device_context.h"
#include "ibcomm/schedule.h"
#include "kernels.h"

namespace ibcomm {

// What a launch needs to know about one rank.
struct RankResources {
  int rank = 0;
  int world_size = 1;
  PeerTable peers{};
  ArenaLayout layout{};
  DeviceStatus* d_status = nullptr;   // device memory
  uint32_t* h_doorbell = nullptr;     // pinned host word (host view)
  uint32_t* d_doorbell = nullptr;     // the same word as the device sees it
};

// Status block + doorbell of one rank.
struct StatusBlock {
  DeviceStatus* d_status = nullptr;
  uint32_t* h_doorbell = nullptr;
  uint32_t* d_doorbell = nullptr;
  void Create();
  void Destroy();
  // 0 when nothing failed.  On failure copies the report, clears both.
  uint32_t Consume(DeviceStatus* out, cudaStream_t stream);
};

struct CachedProgram {
  Program prog;
  Op* d_ops = nullptr;
  int slab = -1;        // slab that holds d_ops
  bool pinned = false;  // recorded into a CUDA graph: kept for the cache's lifetime
};

// Op programs by (algorithm, rank, length, types, knobs), resident on the
// device.  A new program costs no allocation and no host synchronisation on
// the call path: its ops are written into a slab of pinned host memory and
// copied with cudaMemcpyAsync, on the stream of the call that needs them, into
// the twin slab of device memory (slabs are allocated a megabyte at a time).
// Programs are dropped only at a point where the caller has just synchronised
// its stream, and never one that was used while a stream capture was active
// (a captured graph keeps the program's device address).
class ProgramCache {
 public:
  ~ProgramCache();
  // Cuts the message and compiles (or finds) the program of `rank`; a new one
  // is uploaded on `stream`.  `capturing`: the call is being recorded into a graph.
  const CachedProgram& Get(Algo algo, int rank, int world_size, size_t len_elements, DType dtype, DType wire,
                           const ArenaLayout& layout, bool apply_scale, cudaStream_t stream, bool capturing);
  // Everything issued with programs of this cache has finished (the caller
  // synchronised): the moment at which an over-full cache lets go of the
  // programs no graph refers to.
  void NoteSynchronized();
  void Clear();
  size_t size() const { return cache_.size(); }
  // Entries above which NoteSynchronized() evicts (test hook; default 4096).
  void SetBound(size_t entries) { bound_ = entries; }

 private:
  using Key = std::tuple<int, int, int, size_t, int, int, long long, bool, uint64_t, uint64_t, int>;
  struct Slab {
    Op* d = nullptr;  // device memory
    Op* h = nullptr;  // pinned host memory, the upload's source
    size_t cap = 0, used = 0;
    int pinned = 0;   // programs in this slab that a graph may refer to
  };
  Op* Place(const std::vector<Op>& ops, cudaStream_t stream, int* slab_index);
  std::map<Key, std::unique_ptr<CachedProgram>> cache_;
  std::vector<Slab> slabs_;
  size_t bound_ = 4096;
};

ExecParams MakeExecParams(const RankResources& rr, const CachedProgram& cp, DType dtype, DType wire, const void* sendbuf,
                          void* recvbuf, size_t len_elements, double scale, uint64_t timeout_ns,
                          DeviceTraceRec* trace, int trace_capacity);

OneShotParams MakeOneShotParams(const RankResources& rr, DType dtype, const void* sendbuf, void* recvbuf,
                                size_t len_elements, double scale, uint64_t timeout_ns);

// Formats a failure report.
std::string DescribeStatus(const DeviceStatus& st);

// True when NVLS kernels exist for the type.
inline bool NvlsSupportsDType(DType t) { return t == DType::kFloat32 || t == DType::kFloat16 || t == DType::kBFloat16; }

}  // namespace ibcomm
