// Several ranks on ONE GPU, for tests and for machines with fewer GPUs than
// ranks.  Kernels of different ranks wait on each other, and nothing
// guarantees that separate launches on one GPU run at the same time, so here
// every collective is a single cooperative launch whose grid covers all
// ranks (blockIdx.y = rank).  The kernels, programs, flag protocol and
// staging layout are exactly the ones the multi-GPU path uses; only the
// "peer" pointers are local.
#pragma once

#include <memory>
#include <vector>

#include "ibcomm/communicator.h"
#include "ibcomm/device_types.h"

namespace ibcomm {

class EmuWorld {
 public:
  explicit EmuWorld(int num_ranks, size_t pool_bytes = 0, size_t work_bytes = 0);
  ~EmuWorld();
  EmuWorld(const EmuWorld&) = delete;
  EmuWorld& operator=(const EmuWorld&) = delete;

  int num_ranks() const { return ws_; }

  // Device pointers, one per rank.  Runs on `stream` (0 = default stream) and
  // returns after synchronising unless `async`.
  void Allreduce(Algo algo, DType dtype, const std::vector<const void*>& sendbufs,
                 const std::vector<void*>& recvbufs, size_t len_elements, double scale = 1.0,
                 DType wire = DType::kFloat32, int channels = 0, void* stream = nullptr, bool async = false);
  // Reduce-scatter (`all_gather` false: sendbufs hold num_ranks blocks,
  // recvbufs one) or all-gather (the other way round) with the direct
  // algorithm; the remote side is used in place or, with SetDirectStaging(1),
  // goes through the pool.
  void ReduceScatterOrAllGather(bool all_gather, DType dtype, const std::vector<const void*>& sendbufs,
                                const std::vector<void*>& recvbufs, size_t block_elements, double scale = 1.0,
                                int channels = 0, void* stream = nullptr, bool async = false);
  // Convenience for the tester: host buffers in, host buffers out.
  void AllreduceHostBuffers(Algo algo, DType dtype, const std::vector<const void*>& in,
                            const std::vector<void*>& out, size_t len_elements);
  // Status of the last collective (kStatusOk when nothing failed) and the
  // first failure report among the ranks.
  uint32_t LastStatus(DeviceStatus* report) const;
  void SetTimeoutMs(int ms);
  // Test hook: rank `r` takes no part in the following collectives (its CTAs
  // return at once), so its peers' bounded waits run out and they report a
  // timeout; nothing faults or hangs.  -1 restores normal operation.
  void SetSilentRank(int r);
  // Test hook for the executor's self-check: rank `r` is told a message length
  // of one element for programs cut for the real length, so its first op fails
  // the bounds check before any memory is touched; the rank reports "bad
  // program", the others are told to stop.  -1 restores normal operation.
  void SetBadProgramRank(int r);
  // How the direct algorithm treats the buffers: 0 in place, 1 staged through
  // the pool window by window (as for buffers the peers cannot map).
  void SetDirectStaging(int mode);
  int last_channels() const;

  struct Impl;

 private:
  int ws_;
  std::unique_ptr<Impl> impl_;
};

}  // namespace ibcomm
