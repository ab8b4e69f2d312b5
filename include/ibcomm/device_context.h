// Device side of a communicator: the peer-mapped arena (staging pool, work
// region, mailboxes, control page), the peer and multicast mappings, the
// program cache and the kernel launches.  Counterpart of the reference's
// memory pool + work buffer (ibcomm/ibverbs_communicator_cuda.cpp:11-37,
// ibcomm/memory_pool.h) — but resident on the device and mapped by the peers
// instead of pinned on the host and registered with an adapter.
#pragma once

#include <cstddef>
#include <cstdint>

#include "ibcomm/communicator.h"
#include "ibcomm/device_types.h"

namespace ibcomm {

// Byte layout of one rank's arena.  Every rank uses the same layout.
struct ArenaLayout {
  uint64_t control_offset = 0;   // ControlPage
  uint64_t oneshot_offset = 0;   // [2 parities][world_size sources] slots of oneshot_slot_bytes
  uint64_t oneshot_slot_bytes = 0;  // the one-shot area (kOneShotAreaBytes) divided by 2 * world_size
  uint64_t mailbox_offset = 0;   // [kMaxRanks sources][mailbox_slots] of mailbox_slot_bytes
  uint64_t mailbox_slot_bytes = 0;
  uint32_t mailbox_slots = 0;
  uint64_t bcast_ring_offset = 0;  // one more ring of mailbox_slots slots: device broadcasts through the switch
  uint64_t pool_offset = 0;      // IBCOMM_MEMORY_POOL_PRE_ALLOC bytes
  uint64_t pool_bytes = 0;
  uint64_t work_offset = 0;      // IBCOMM_WORK_GPU_MEMORY_SIZE bytes
  uint64_t work_bytes = 0;
  uint64_t total_bytes = 0;
};
// Bytes of the one-shot area: 16 MiB slots for two ranks, 4 MiB for eight.
constexpr uint64_t kOneShotAreaBytes = 64ull << 20;
ArenaLayout MakeArenaLayout(size_t pool_bytes, size_t work_bytes, int world_size);

// Algorithm and channel choice for a message (src/host/tuner.cpp).
struct TunerChoice {
  Algo algo;
  int channels;
};
TunerChoice ChooseAlgorithm(size_t bytes, int world_size, bool nvls_available, bool zero_copy, int max_channels);
// Channels for a forced algorithm.
int ChooseChannels(Algo algo, size_t bytes, int world_size, int max_channels);

// Functions the host half of the communicator calls (defined in src/cuda).
bool DeviceContextIsDevicePointer(const void* p);
void DeviceContextSend(DeviceContext* d, int dest, const void* buf, size_t len);
void DeviceContextRecv(DeviceContext* d, int src, void* buf, size_t len);
bool DeviceContextSendPoll(DeviceContext* d, int dest);
bool DeviceContextRecvPoll(DeviceContext* d, int src);
void DeviceContextSendWait(DeviceContext* d, int dest);
void DeviceContextRecvWait(DeviceContext* d, int src);
// Broadcast of a device buffer through NVSwitch multicast; false (nothing done)
// when the box has no multicast or the length is not a multiple of 16 (the
// same on every rank): the caller then falls back to sends.
bool DeviceContextBcast(DeviceContext* d, void* buf, size_t len, int root);
void DeviceContextCollectTrace(DeviceContext* d, Tracer* tracer);
// Per-role stamps of the last traced call of the pipelined staged kernel (CTA
// 0), in nanoseconds from the call's first stamp: for W windows, 4 W pairs -
// reducers (waits satisfied, window published), loader (input buffer free,
// input window published), storer (window reduced everywhere, output buffer
// released), reducers again (last store issued, 0).  Copies at most
// `capacity_words` words and returns the number available (8 W, or 0).
size_t DeviceContextStagedTimeline(DeviceContext* d, uint64_t* out, size_t capacity_words);

// Introspection for bindings and tests.
struct DeviceInfo {
  int device;
  int nvls;            // multicast alias of the arena is mapped
  int share_mode;      // 0 = virtual-memory descriptors, 1 = CUDA IPC
  uint64_t arena_bytes;
  uint64_t pool_bytes;
  uint64_t work_bytes;
  uint64_t calls;      // collectives issued so far
  int last_algo;       // Algo of the most recent allreduce
  int last_channels;
  uint64_t kernel_launches;  // kernels of this library launched so far
  uint64_t switch_registrations;  // registered user buffers that are bound to the NVSwitch multicast
};
DeviceInfo DeviceContextInfo(DeviceContext* d);
// Caps the channels a collective may use (0 = back to IBCOMM_NUM_CUDA_STREAM).
void DeviceContextSetMaxChannels(DeviceContext* d, int channels);

// Symmetric (peer-mapped, multicast-bound when possible) user memory.  Every
// rank must call with the same size in the same order.  Buffers inside such
// an allocation are reduced in place by the switch without staging copies.
void* DeviceContextSymmetricAlloc(Communicator* comm, size_t bytes);
void DeviceContextSymmetricFree(Communicator* comm, void* ptr);

// Buffer registration (see Communicator::RegisterCudaBuffer).
int DeviceContextRegisterBuffer(Communicator* comm, void* ptr, size_t bytes);
void DeviceContextDeregisterBuffer(Communicator* comm, int id);

// Reads the failure doorbell; on failure fetches the report, resets it and
// raises TRANSPORT_ERROR.  Called after every synchronous collective; callers
// of asynchronous collectives call it after they synchronised their stream.
void DeviceContextCheck(DeviceContext* d);
// Non-raising variant: returns the status code and copies the report.
uint32_t DeviceContextPeekStatus(DeviceContext* d, DeviceStatus* out);

}  // namespace ibcomm
