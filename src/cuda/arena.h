// Device memory that peers can map: the replacement of the reference's pinned,
// adapter-registered staging blocks (ibcomm/memory_pool.h:28-54).
//
// A SharedAllocation is created with the virtual-memory API so that it can be
// (a) exported to other processes as a POSIX file descriptor and (b) bound to
// an NVSwitch multicast object.  When that API is unavailable the allocation
// falls back to cudaMalloc + a CUDA IPC handle (no multicast then).
#pragma once

#include <string>

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <vector>

namespace ibcomm {

enum class ShareMode : int { kVmm = 0, kIpc = 1 };

// What one rank tells another about an allocation (travels over the host
// transport; the descriptor itself travels over the FdChannel).
struct ShareTicket {
  int32_t mode;     // ShareMode
  int32_t device;   // CUDA ordinal in the owner's process
  int32_t pid;      // owner process
  int32_t has_fd;   // a descriptor follows on the fd channel
  uint64_t bytes;   // mapped size
  uint64_t owner_ptr;  // address in the owner's process (same-process shortcut)
  cudaIpcMemHandle_t ipc;
};

class SharedAllocation {
 public:
  SharedAllocation() = default;
  ~SharedAllocation();
  SharedAllocation(const SharedAllocation&) = delete;
  SharedAllocation& operator=(const SharedAllocation&) = delete;

  // Allocates at least `bytes` on `device` (current device must be `device`).
  // `align_to` > 0 rounds the size up to that multiple as well (multicast
  // granularity).  Memory is zeroed.
  void Create(size_t bytes, int device, size_t align_to);
  // Descriptor for export; -1 in IPC mode.  The caller owns (closes) it.
  int ExportFd() const;
  ShareTicket Ticket() const;

  // Maps a peer's allocation into this process for `my_device`.
  void Import(const ShareTicket& ticket, int fd, int my_device);

  unsigned char* ptr() const { return ptr_; }
  size_t bytes() const { return bytes_; }
  ShareMode mode() const { return mode_; }
  bool imported() const { return imported_; }
  CUmemGenericAllocationHandle handle() const { return handle_; }
  void Release();

 private:
  unsigned char* ptr_ = nullptr;
  size_t bytes_ = 0;
  int device_ = -1;
  ShareMode mode_ = ShareMode::kVmm;
  bool imported_ = false;
  bool same_process_alias_ = false;
  CUmemGenericAllocationHandle handle_ = 0;
};

// NVSwitch multicast object covering one SharedAllocation per rank.
class MulticastGroup {
 public:
  MulticastGroup() = default;
  ~MulticastGroup();
  MulticastGroup(const MulticastGroup&) = delete;
  MulticastGroup& operator=(const MulticastGroup&) = delete;

  // True when the device and the driver offer multicast.
  static bool Supported(int device);
  // Size granularity for allocations that will be bound (0 if unsupported).
  static size_t Granularity(int num_devices, size_t bytes);

  // Root: creates the object; returns the descriptor to hand to the peers.
  int CreateRoot(size_t bytes, int num_devices);
  // Others: adopt the root's object.
  void Import(int fd, size_t bytes, int num_devices);
  void AddDevice(int device);
  // After EVERY rank has added its device: bind my memory, map the alias.
  void BindAndMap(const SharedAllocation& mem, int device);
  // The same for `bytes()` bytes of existing device memory at `ptr` (any
  // allocation of this device; address and size multiples of the
  // granularity).  Not fatal: false, with a reason in `why`, when the driver
  // refuses; the group is then unusable and must be released by every rank.
  bool BindAddrAndMap(void* ptr, int device, std::string* why);
  size_t bytes() const { return bytes_; }
  unsigned char* ptr() const { return ptr_; }
  bool valid() const { return ptr_ != nullptr; }
  void Release();

 private:
  CUmemGenericAllocationHandle mc_ = 0;
  bool have_handle_ = false;
  bool bound_ = false;
  int device_ = -1;
  int num_devices_ = 1;
  size_t bytes_ = 0;
  unsigned char* ptr_ = nullptr;
};

}  // namespace ibcomm
