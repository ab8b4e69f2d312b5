#include "driver_api.h"

#include <cuda_runtime.h>

#include <mutex>

#include "ibcomm/error.h"

namespace ibcomm {
namespace drv {

static Api g_api;
static bool g_multicast = false;
static std::once_flag g_once;

template <typename Fn>
static bool Load(const char* name, Fn* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    (void)cudaGetLastError();
    return false;
  }
  *out = reinterpret_cast<Fn>(p);
  return true;
}

static void LoadAll() {
  bool ok = true;
  ok &= Load("cuGetErrorString", &g_api.GetErrorString);
  ok &= Load("cuDeviceGet", &g_api.DeviceGet);
  ok &= Load("cuDeviceGetAttribute", &g_api.DeviceGetAttribute);
  ok &= Load("cuMemGetAllocationGranularity", &g_api.MemGetAllocationGranularity);
  ok &= Load("cuMemCreate", &g_api.MemCreate);
  ok &= Load("cuMemRelease", &g_api.MemRelease);
  ok &= Load("cuMemAddressReserve", &g_api.MemAddressReserve);
  ok &= Load("cuMemAddressFree", &g_api.MemAddressFree);
  ok &= Load("cuMemMap", &g_api.MemMap);
  ok &= Load("cuMemUnmap", &g_api.MemUnmap);
  ok &= Load("cuMemSetAccess", &g_api.MemSetAccess);
  ok &= Load("cuMemExportToShareableHandle", &g_api.MemExportToShareableHandle);
  ok &= Load("cuMemImportFromShareableHandle", &g_api.MemImportFromShareableHandle);
  ok &= Load("cuMemGetAddressRange", &g_api.MemGetAddressRange);
  ok &= Load("cuPointerGetAttribute", &g_api.PointerGetAttribute);
  bool mc = true;
  mc &= Load("cuMulticastCreate", &g_api.MulticastCreate);
  mc &= Load("cuMulticastAddDevice", &g_api.MulticastAddDevice);
  mc &= Load("cuMulticastBindMem", &g_api.MulticastBindMem);
  mc &= Load("cuMulticastUnbind", &g_api.MulticastUnbind);
  mc &= Load("cuMulticastGetGranularity", &g_api.MulticastGetGranularity);
  (void)Load("cuMulticastBindAddr", &g_api.MulticastBindAddr);
  g_multicast = ok && mc;
  g_api.loaded = ok;
}

const Api* Get() {
  std::call_once(g_once, LoadAll);
  return g_api.loaded ? &g_api : nullptr;
}

bool HasMulticastApi() {
  Get();
  return g_multicast;
}

const char* ErrorString(CUresult r) {
  const Api* a = Get();
  const char* s = nullptr;
  if (a != nullptr && a->GetErrorString(r, &s) == CUDA_SUCCESS && s != nullptr) return s;
  return "unknown driver error";
}

}  // namespace drv
}  // namespace ibcomm
