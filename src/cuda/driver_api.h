// CUDA driver entry points used for virtual-memory and multicast management,
// resolved at run time through the runtime (cudaGetDriverEntryPoint) so that
// the library has no link-time dependency on libcuda and still loads on hosts
// without a driver.
#pragma once

#include <cuda.h>

namespace ibcomm {
namespace drv {

struct Api {
  bool loaded = false;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr) = nullptr;
  CUresult (*PointerGetAttribute)(void*, CUpointer_attribute, CUdeviceptr) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  // Optional on its own (registration of user buffers with the switch): may be null.
  CUresult (*MulticastBindAddr)(CUmemGenericAllocationHandle, size_t, CUdeviceptr, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
};

// Loads the table once per process.  Returns nullptr (after a warning) when a
// required symbol is missing; multicast symbols are optional.
const Api* Get();
bool HasMulticastApi();
const char* ErrorString(CUresult r);

}  // namespace drv
}  // namespace ibcomm

// Fails the process (or throws, by policy) with CUDA_ERROR on a driver error.
#define CUCHECK(call)                                                                     \
  do {                                                                                    \
    CUresult r__ = (call);                                                                \
    if (r__ != CUDA_SUCCESS)                                                              \
      IBCOMM_FAIL(CUDA_ERROR, "%s failed: %s\n", #call, ::ibcomm::drv::ErrorString(r__)); \
  } while (0)
