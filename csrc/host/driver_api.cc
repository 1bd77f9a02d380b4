#include "driver_api.h"
#include "launch.h"
#include <mutex>

namespace mep {

static DriverApi g_api;
static bool g_ok = false;
static std::once_flag g_once;
static std::string g_why;

template <class F>
static bool load(F& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    g_why = std::string("driver entry point ") + name + " unavailable: " + cudaGetErrorString(e);
    (void)cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

static void init() {
  g_ok = load(g_api.GetErrorString, "cuGetErrorString") && load(g_api.DeviceGet, "cuDeviceGet") &&
         load(g_api.DeviceGetAttribute, "cuDeviceGetAttribute") &&
         load(g_api.MemGetAllocationGranularity, "cuMemGetAllocationGranularity") &&
         load(g_api.MemCreate, "cuMemCreate") && load(g_api.MemRelease, "cuMemRelease") &&
         load(g_api.MemAddressReserve, "cuMemAddressReserve") && load(g_api.MemAddressFree, "cuMemAddressFree") &&
         load(g_api.MemMap, "cuMemMap") && load(g_api.MemUnmap, "cuMemUnmap") &&
         load(g_api.MemSetAccess, "cuMemSetAccess") &&
         load(g_api.MemExportToShareableHandle, "cuMemExportToShareableHandle") &&
         load(g_api.MemImportFromShareableHandle, "cuMemImportFromShareableHandle") &&
         load(g_api.MulticastCreate, "cuMulticastCreate") && load(g_api.MulticastAddDevice, "cuMulticastAddDevice") &&
         load(g_api.MulticastBindMem, "cuMulticastBindMem") && load(g_api.MulticastUnbind, "cuMulticastUnbind") &&
         load(g_api.MulticastGetGranularity, "cuMulticastGetGranularity") &&
         load(g_api.TensorMapEncodeTiled, "cuTensorMapEncodeTiled");
}

const DriverApi* driver() {
  std::call_once(g_once, init);
  if (!g_ok) { set_error("CUDA driver API unavailable: %s", g_why.c_str()); return nullptr; }
  return &g_api;
}

}  // namespace mep
