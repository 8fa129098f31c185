// CUDA driver entry points of the VMM backend, resolved at run time so that libcoccl.so has no
// link-time dependency on libcuda (it must load on machines without a driver).
#include "memory/buffer_manager.h"

namespace coccl {
namespace {

template <typename Fn>
Fn resolve(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return reinterpret_cast<Fn>(p);
}

int peerDevicesOf(int device, int* out, int capacity) {
  int n = 0, count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) count = 0;
  if (n < capacity) out[n++] = device;
  for (int d = 0; d < count && n < capacity; ++d) {
    if (d == device) continue;
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, d, device) == cudaSuccess && can) out[n++] = d;
  }
  return n;
}

bool vmmSupported(int device) {
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryPoolsSupported, device) != cudaSuccess) return false;
  // virtual memory management itself is reported through the driver attribute
  typedef CUresult (*GetAttr)(int*, CUdevice_attribute, CUdevice);
  static GetAttr getAttr = resolve<GetAttr>("cuDeviceGetAttribute");
  if (!getAttr) return false;
  int vmm = 0;
  if (getAttr(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, device) != CUDA_SUCCESS) return false;
  return vmm != 0;
}

}  // namespace

const VmmDriverApi* cudaVmmDriverApi() {
  static VmmDriverApi api;
  static bool tried = false, ok = false;
  if (!tried) {
    tried = true;
    api.getGranularity = resolve<decltype(api.getGranularity)>("cuMemGetAllocationGranularity");
    api.addressReserve = resolve<decltype(api.addressReserve)>("cuMemAddressReserve");
    api.addressFree = resolve<decltype(api.addressFree)>("cuMemAddressFree");
    api.create = resolve<decltype(api.create)>("cuMemCreate");
    api.release = resolve<decltype(api.release)>("cuMemRelease");
    api.map = resolve<decltype(api.map)>("cuMemMap");
    api.unmap = resolve<decltype(api.unmap)>("cuMemUnmap");
    api.setAccess = resolve<decltype(api.setAccess)>("cuMemSetAccess");
    api.peerDevices = &peerDevicesOf;
    api.supported = &vmmSupported;
    ok = api.getGranularity && api.addressReserve && api.addressFree && api.create && api.release && api.map &&
         api.unmap && api.setAccess;
  }
  return ok ? &api : nullptr;
}

}  // namespace coccl
