#include "arena.h"

#include <unistd.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>

#include "driver_api.h"
#include "ibcomm/error.h"

namespace ibcomm {

static size_t RoundUp(size_t v, size_t a) { return a == 0 ? v : (v + a - 1) / a * a; }

static bool ForceIpc() {
  const char* s = getenv("IBCOMM_ARENA_MODE");
  return s != nullptr && strcmp(s, "ipc") == 0;
}

static CUmemAllocationProp DeviceProp(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

static void GrantAccess(const drv::Api* api, CUdeviceptr va, size_t bytes, int device) {
  CUmemAccessDesc desc;
  memset(&desc, 0, sizeof(desc));
  desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  desc.location.id = device;
  desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUCHECK(api->MemSetAccess(va, bytes, &desc, 1));
}

// ------------------------------------------------------------ allocation
SharedAllocation::~SharedAllocation() { Release(); }

void SharedAllocation::Release() {
  if (ptr_ == nullptr) return;
  const drv::Api* api = drv::Get();
  if (same_process_alias_) {
    // nothing owned
  } else if (mode_ == ShareMode::kVmm && api != nullptr) {
    api->MemUnmap(reinterpret_cast<CUdeviceptr>(ptr_), bytes_);
    api->MemAddressFree(reinterpret_cast<CUdeviceptr>(ptr_), bytes_);
    api->MemRelease(handle_);
  } else if (imported_) {
    cudaIpcCloseMemHandle(ptr_);
  } else {
    cudaFree(ptr_);
  }
  (void)cudaGetLastError();
  ptr_ = nullptr;
  bytes_ = 0;
}

void SharedAllocation::Create(size_t bytes, int device, size_t align_to) {
  device_ = device;
  imported_ = false;
  const drv::Api* api = ForceIpc() ? nullptr : drv::Get();
  if (api != nullptr) {
    CUmemAllocationProp prop = DeviceProp(device);
    size_t gran = 0;
    CUresult r = api->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (r == CUDA_SUCCESS && gran != 0) {
      size_t size = RoundUp(RoundUp(bytes, gran), align_to);
      CUmemGenericAllocationHandle h = 0;
      r = api->MemCreate(&h, size, &prop, 0);
      if (r == CUDA_SUCCESS) {
        CUdeviceptr va = 0;
        CUCHECK(api->MemAddressReserve(&va, size, align_to > gran ? align_to : gran, 0, 0));
        CUCHECK(api->MemMap(va, size, 0, h, 0));
        GrantAccess(api, va, size, device);
        handle_ = h;
        ptr_ = reinterpret_cast<unsigned char*>(va);
        bytes_ = size;
        mode_ = ShareMode::kVmm;
        if (cudaMemset(ptr_, 0, bytes_) != cudaSuccess) IBCOMM_FAIL(CUDA_ERROR, "cudaMemset of a new arena failed.\n");
        if (cudaDeviceSynchronize() != cudaSuccess) IBCOMM_FAIL(CUDA_ERROR, "cudaDeviceSynchronize failed.\n");
        return;
      }
    }
    IBCOMM_WARN("Shareable device memory is not available (%s); falling back to CUDA IPC, without multicast.\n",
                drv::ErrorString(r));
  }
  size_t size = RoundUp(bytes, 2u << 20);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, size);
  if (e != cudaSuccess) IBCOMM_FAIL(CUDA_ERROR, "cudaMalloc(%zu) failed: %s\n", size, cudaGetErrorString(e));
  e = cudaMemset(p, 0, size);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) IBCOMM_FAIL(CUDA_ERROR, "clearing a new arena failed: %s\n", cudaGetErrorString(e));
  ptr_ = static_cast<unsigned char*>(p);
  bytes_ = size;
  mode_ = ShareMode::kIpc;
}

int SharedAllocation::ExportFd() const {
  if (mode_ != ShareMode::kVmm) return -1;
  const drv::Api* api = drv::Get();
  int fd = -1;
  CUCHECK(api->MemExportToShareableHandle(&fd, handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  return fd;
}

ShareTicket SharedAllocation::Ticket() const {
  ShareTicket t;
  memset(&t, 0, sizeof(t));
  t.mode = static_cast<int32_t>(mode_);
  t.device = device_;
  t.pid = static_cast<int32_t>(getpid());
  t.has_fd = mode_ == ShareMode::kVmm ? 1 : 0;
  t.bytes = bytes_;
  t.owner_ptr = reinterpret_cast<uint64_t>(ptr_);
  if (mode_ == ShareMode::kIpc) {
    cudaError_t e = cudaIpcGetMemHandle(&t.ipc, ptr_);
    if (e != cudaSuccess) IBCOMM_FAIL(CUDA_ERROR, "cudaIpcGetMemHandle failed: %s\n", cudaGetErrorString(e));
  }
  return t;
}

void SharedAllocation::Import(const ShareTicket& ticket, int fd, int my_device) {
  device_ = my_device;
  imported_ = true;
  bytes_ = ticket.bytes;
  mode_ = static_cast<ShareMode>(ticket.mode);
  if (mode_ == ShareMode::kVmm) {
    const drv::Api* api = drv::Get();
    if (api == nullptr) IBCOMM_FAIL(CUDA_ERROR, "The peer shares virtual-memory allocations but this process cannot load the driver API.\n");
    if (fd < 0) IBCOMM_FAIL(TRANSPORT_ERROR, "No descriptor arrived for a peer allocation.\n");
    CUmemGenericAllocationHandle h = 0;
    CUCHECK(api->MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    close(fd);
    CUdeviceptr va = 0;
    CUCHECK(api->MemAddressReserve(&va, bytes_, 2u << 20, 0, 0));
    CUCHECK(api->MemMap(va, bytes_, 0, h, 0));
    GrantAccess(api, va, bytes_, my_device);
    handle_ = h;
    ptr_ = reinterpret_cast<unsigned char*>(va);
    return;
  }
  if (ticket.pid == static_cast<int32_t>(getpid())) {
    // Same process: IPC handles cannot be opened by their creator; use the
    // owner's pointer and enable peer access between the two devices.
    if (ticket.device != my_device) {
      cudaError_t e = cudaDeviceEnablePeerAccess(ticket.device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
        IBCOMM_FAIL(CUDA_ERROR, "cudaDeviceEnablePeerAccess(%d) failed: %s\n", ticket.device, cudaGetErrorString(e));
      (void)cudaGetLastError();
    }
    ptr_ = reinterpret_cast<unsigned char*>(ticket.owner_ptr);
    same_process_alias_ = true;
    return;
  }
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, ticket.ipc, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) IBCOMM_FAIL(CUDA_ERROR, "cudaIpcOpenMemHandle failed: %s\n", cudaGetErrorString(e));
  ptr_ = static_cast<unsigned char*>(p);
}

// -------------------------------------------------------------- multicast
MulticastGroup::~MulticastGroup() { Release(); }

void MulticastGroup::Release() {
  const drv::Api* api = drv::Get();
  if (api == nullptr) return;
  if (ptr_ != nullptr) {
    api->MemUnmap(reinterpret_cast<CUdeviceptr>(ptr_), bytes_);
    api->MemAddressFree(reinterpret_cast<CUdeviceptr>(ptr_), bytes_);
    ptr_ = nullptr;
  }
  if (bound_) {
    CUdevice dev;
    if (api->DeviceGet(&dev, device_) == CUDA_SUCCESS) api->MulticastUnbind(mc_, dev, 0, bytes_);
    bound_ = false;
  }
  if (have_handle_) {
    api->MemRelease(mc_);
    have_handle_ = false;
  }
}

bool MulticastGroup::Supported(int device) {
  if (!drv::HasMulticastApi()) return false;
  const drv::Api* api = drv::Get();
  CUdevice dev;
  if (api->DeviceGet(&dev, device) != CUDA_SUCCESS) return false;
  int v = 0;
  if (api->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return false;
  return v != 0;
}

static CUmulticastObjectProp McProp(int num_devices, size_t bytes) {
  CUmulticastObjectProp p;
  memset(&p, 0, sizeof(p));
  p.numDevices = static_cast<unsigned>(num_devices);
  p.size = bytes;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

size_t MulticastGroup::Granularity(int num_devices, size_t bytes) {
  if (!drv::HasMulticastApi()) return 0;
  CUmulticastObjectProp p = McProp(num_devices, bytes);
  size_t g = 0;
  if (drv::Get()->MulticastGetGranularity(&g, &p, CU_MULTICAST_GRANULARITY_MINIMUM) != CUDA_SUCCESS) return 0;
  return g;
}

int MulticastGroup::CreateRoot(size_t bytes, int num_devices) {
  const drv::Api* api = drv::Get();
  CUmulticastObjectProp p = McProp(num_devices, bytes);
  CUresult r = api->MulticastCreate(&mc_, &p);
  if (r != CUDA_SUCCESS) {
    IBCOMM_WARN("cuMulticastCreate(%zu bytes, %d devices) failed: %s; multicast paths are disabled.\n", bytes,
                num_devices, drv::ErrorString(r));
    return -1;
  }
  have_handle_ = true;
  bytes_ = bytes;
  num_devices_ = num_devices;
  int fd = -1;
  r = api->MemExportToShareableHandle(&fd, mc_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    IBCOMM_WARN("exporting the multicast object failed: %s; multicast paths are disabled.\n", drv::ErrorString(r));
    Release();
    return -1;
  }
  return fd;
}

void MulticastGroup::Import(int fd, size_t bytes, int num_devices) {
  num_devices_ = num_devices;
  const drv::Api* api = drv::Get();
  CUCHECK(api->MemImportFromShareableHandle(&mc_, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                            CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  close(fd);
  have_handle_ = true;
  bytes_ = bytes;
}

void MulticastGroup::AddDevice(int device) {
  const drv::Api* api = drv::Get();
  CUdevice dev;
  CUCHECK(api->DeviceGet(&dev, device));
  CUCHECK(api->MulticastAddDevice(mc_, dev));
  device_ = device;
}

void MulticastGroup::BindAndMap(const SharedAllocation& mem, int device) {
  const drv::Api* api = drv::Get();
  CUCHECK(api->MulticastBindMem(mc_, 0, mem.handle(), 0, bytes_, 0));
  bound_ = true;
  CUdeviceptr va = 0;
  size_t gran = Granularity(num_devices_, bytes_);
  if (gran < (2u << 20)) gran = 2u << 20;
  CUCHECK(api->MemAddressReserve(&va, bytes_, gran, 0, 0));
  CUCHECK(api->MemMap(va, bytes_, 0, mc_, 0));
  CUmemAccessDesc desc;
  memset(&desc, 0, sizeof(desc));
  desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  desc.location.id = device;
  desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUCHECK(api->MemSetAccess(va, bytes_, &desc, 1));
  ptr_ = reinterpret_cast<unsigned char*>(va);
}

bool MulticastGroup::BindAddrAndMap(void* ptr, int device, std::string* why) {
  const drv::Api* api = drv::Get();
  if (api == nullptr || api->MulticastBindAddr == nullptr) {
    *why = "the driver has no cuMulticastBindAddr";
    return false;
  }
  CUresult r = api->MulticastBindAddr(mc_, 0, reinterpret_cast<CUdeviceptr>(ptr), bytes_, 0);
  if (r != CUDA_SUCCESS) {
    *why = std::string("cuMulticastBindAddr: ") + drv::ErrorString(r);
    return false;
  }
  bound_ = true;
  CUdeviceptr va = 0;
  size_t gran = Granularity(num_devices_, bytes_);
  if (gran < (2u << 20)) gran = 2u << 20;
  r = api->MemAddressReserve(&va, bytes_, gran, 0, 0);
  if (r != CUDA_SUCCESS) {
    *why = std::string("cuMemAddressReserve: ") + drv::ErrorString(r);
    return false;
  }
  r = api->MemMap(va, bytes_, 0, mc_, 0);
  if (r != CUDA_SUCCESS) {
    api->MemAddressFree(va, bytes_);
    *why = std::string("cuMemMap: ") + drv::ErrorString(r);
    return false;
  }
  ptr_ = reinterpret_cast<unsigned char*>(va);  // from here on Release() unmaps and frees
  CUmemAccessDesc desc;
  memset(&desc, 0, sizeof(desc));
  desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  desc.location.id = device;
  desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = api->MemSetAccess(va, bytes_, &desc, 1);
  if (r != CUDA_SUCCESS) {
    *why = std::string("cuMemSetAccess: ") + drv::ErrorString(r);
    return false;
  }
  return true;
}

}  // namespace ibcomm
