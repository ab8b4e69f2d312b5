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
};

class ProgramCache {
 public:
  ~ProgramCache();
  // Cuts the message and compiles (or finds) the program of `rank`.
  const CachedProgram& Get(Algo algo, int rank, int world_size, size_t len_elements, DType dtype, DType wire,
                           const ArenaLayout& layout, bool apply_scale);
  void Clear();

 private:
  using Key = std::tuple<int, int, int, size_t, int, int, long long, bool, uint64_t, uint64_t>;
  std::map<Key, std::unique_ptr<CachedProgram>> cache_;
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
