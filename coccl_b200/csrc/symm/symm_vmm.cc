// cuMem VMM backend of the symmetric memory (symm.h) and the NVSwitch multicast binding.
//
// A buffer is a virtual range reserved well beyond its size with physical chunks mapped into its front. Every chunk is
// exported as a POSIX file descriptor; descriptors reach other processes through fd_channel.h, and the export handle
// (plain bytes, exchanged by the caller) only names them: {pid, device, reserve size, chunk sizes, key of chunk 0}.
// An importer reserves the same amount of address space for the peer and maps the chunks in order, so growing a buffer
// is "create one more chunk, map it behind the others, export again": no pointer on any rank changes. This is the
// growth-in-place scheme of the reference's workspace (src/coccl-extend/core/memory/coccl_buffer_vmm.cc:152-240,
// which maps within one process) carried across processes the way NCCL carries its cuMem allocations
// (src/transport/p2p.cc:199-284, src/misc/ipcsocket.cc). The multicast part follows NCCL's NVLS set-up
// (src/transport/nvls.cc:72-203): one object created by a root, imported by the others, every device added, every
// rank's memory bound, the object mapped next to the unicast mapping.
//
// libcoccl.so does not link libcuda: the driver entry points are looked up at run time.
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <new>

#include "symm/fd_channel.h"
#include "symm/symm_internal.h"

namespace coccl {
namespace {

constexpr uint32_t kVmmMagic = 0x484d4d56u;  // "VMMH"
constexpr int kMaxChunks = 8;
constexpr size_t kGranule = 2u << 20;        // chunk sizes travel in units of 2 MiB
constexpr int kFetchTimeoutMs = 10000;

// Export handle of a VMM buffer: the first 64 bytes of the COCCL_SYMM_HANDLE_BYTES blob (the tail keeps the layout of
// the IPC backend's same-process record, which this backend fills too).
struct VmmHandle {
  uint32_t magic;
  int32_t pid;
  int32_t device;
  int32_t nChunks;
  uint64_t reserveBytes;
  uint64_t serial;                  // key of chunk i = serial << 8 | i; of the multicast object serial << 8 | 0xff
  uint32_t chunkGranules[kMaxChunks];
};
static_assert(sizeof(VmmHandle) <= 64, "VMM handle must fit in front of the same-process record");
struct SameProcess {
  unsigned long long pid;
  void* address;
  int device;
};
static_assert(64 + sizeof(SameProcess) <= COCCL_SYMM_HANDLE_BYTES, "export handle too small");

struct McHandle {
  uint32_t magic;
  int32_t pid;
  uint64_t key;
  uint64_t bytes;
  int32_t nRanks;
};

struct Driver {
  CUresult (*getGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*addressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*setAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*exportHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*importHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*deviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  // multicast (optional)
  CUresult (*mcCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*mcGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*mcAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*mcBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*mcUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  bool ok = false, mcOk = false;
};

template <typename Fn>
void resolve(Fn* out, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
    *out = reinterpret_cast<Fn>(p);
  else
    cudaGetLastError();
}

const Driver& driver() {
  static Driver d;
  static bool tried = false;
  if (!tried) {
    tried = true;
    resolve(&d.getGranularity, "cuMemGetAllocationGranularity");
    resolve(&d.create, "cuMemCreate");
    resolve(&d.release, "cuMemRelease");
    resolve(&d.addressReserve, "cuMemAddressReserve");
    resolve(&d.addressFree, "cuMemAddressFree");
    resolve(&d.map, "cuMemMap");
    resolve(&d.unmap, "cuMemUnmap");
    resolve(&d.setAccess, "cuMemSetAccess");
    resolve(&d.exportHandle, "cuMemExportToShareableHandle");
    resolve(&d.importHandle, "cuMemImportFromShareableHandle");
    resolve(&d.deviceGetAttribute, "cuDeviceGetAttribute");
    resolve(&d.mcCreate, "cuMulticastCreate");
    resolve(&d.mcGranularity, "cuMulticastGetGranularity");
    resolve(&d.mcAddDevice, "cuMulticastAddDevice");
    resolve(&d.mcBindMem, "cuMulticastBindMem");
    resolve(&d.mcUnbind, "cuMulticastUnbind");
    d.ok = d.getGranularity && d.create && d.release && d.addressReserve && d.addressFree && d.map && d.unmap && d.setAccess &&
           d.exportHandle && d.importHandle && d.deviceGetAttribute;
    d.mcOk = d.ok && d.mcCreate && d.mcGranularity && d.mcAddDevice && d.mcBindMem && d.mcUnbind;
  }
  return d;
}

int deviceAttr(CUdevice_attribute a, int device) {
  int v = 0;
  if (!driver().deviceGetAttribute || driver().deviceGetAttribute(&v, a, device) != CUDA_SUCCESS) return 0;
  return v;
}

CUmemAllocationProp propFor(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

size_t roundUp(size_t v, size_t g) { return (v + g - 1) / g * g; }

// Granularity of a chunk: what the allocator recommends, what a multicast binding needs where the device has one, and
// the 2 MiB unit the handle counts in.
size_t chunkGranularity(int device) {
  const Driver& d = driver();
  size_t g = kGranule;
  const CUmemAllocationProp p = propFor(device);
  size_t v = 0;
  if (d.getGranularity(&v, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && v > g) g = roundUp(v, kGranule);
  if (d.mcOk && deviceAttr(CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device)) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = 2;
    mp.size = g;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d.mcGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS && mg > g) g = roundUp(mg, kGranule);
  }
  return g;
}

int grantAccess(CUdeviceptr base, size_t bytes, int device) {
  CUmemAccessDesc a;
  memset(&a, 0, sizeof(a));
  a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  a.location.id = device;
  a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  return driver().setAccess(base, bytes, &a, 1) == CUDA_SUCCESS ? 0 : (int)cudaErrorUnknown;
}

std::atomic<uint64_t> gSerial{1};
uint64_t serialOf(const cocclSymmBuffer* b) { return b->own.chunks.empty() ? 0 : b->own.chunks[0].key >> 8; }

// Create one chunk on `device`, map it at the end of `m`, publish its descriptor under `key`.
int addOwnChunk(VmmMapping& m, size_t bytes, int device, uint64_t key) {
  const Driver& d = driver();
  if (m.mapped + bytes > m.reserved || (int)m.chunks.size() >= kMaxChunks) return (int)cudaErrorMemoryAllocation;
  const CUmemAllocationProp p = propFor(device);
  VmmChunk c;
  c.bytes = bytes;
  c.key = key;
  if (d.create(&c.handle, bytes, &p, 0) != CUDA_SUCCESS) return (int)cudaErrorMemoryAllocation;
  int fd = -1;
  bool ok = d.exportHandle(&fd, c.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS && fd >= 0;
  if (ok) {
    ok = fdChannelPublish(key, fd) == 0;
    close(fd);
  }
  if (ok) ok = d.map(m.base + m.mapped, bytes, 0, c.handle, 0) == CUDA_SUCCESS;
  if (ok && grantAccess(m.base + m.mapped, bytes, device) != 0) {
    d.unmap(m.base + m.mapped, bytes);
    ok = false;
  }
  if (!ok) {
    fdChannelWithdraw(key);
    d.release(c.handle);
    return (int)cudaErrorMemoryAllocation;
  }
  m.chunks.push_back(c);
  m.mapped += bytes;
  return 0;
}

void unmapAll(VmmMapping& m, bool withdraw) {
  const Driver& d = driver();
  size_t off = 0;
  for (VmmChunk& c : m.chunks) {
    d.unmap(m.base + off, c.bytes);
    d.release(c.handle);
    if (withdraw && c.key) fdChannelWithdraw(c.key);
    off += c.bytes;
  }
  m.chunks.clear();
  if (m.base) d.addressFree(m.base, m.reserved);
  m.base = 0;
  m.reserved = m.mapped = 0;
}

}  // namespace

bool vmmAvailable() {
  if (cudaFree(nullptr) != cudaSuccess) { cudaGetLastError(); return false; }
  if (!driver().ok) return false;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return false; }
  return deviceAttr(CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev) != 0 &&
         deviceAttr(CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev) != 0;
}

int vmmAlloc(size_t bytes, cocclSymmBuffer** out) {
  if (!vmmAvailable()) return (int)cudaErrorNotSupported;
  cocclSymmBuffer* b = new (std::nothrow) cocclSymmBuffer();
  if (!b) return (int)cudaErrorMemoryAllocation;
  b->vmm = true;
  if (cudaGetDevice(&b->device) != cudaSuccess) { delete b; return (int)cudaErrorInvalidDevice; }
  const size_t g = chunkGranularity(b->device);
  const size_t first = roundUp(bytes, g);
  // room to grow: eight times the first size, at least 1 GiB, at most 64 GiB of ADDRESS SPACE (no memory behind it)
  size_t reserve = first * 8;
  if (reserve < (1ull << 30)) reserve = 1ull << 30;
  if (reserve > (64ull << 30)) reserve = roundUp(first, g) > (64ull << 30) ? first : (64ull << 30);
  if (driver().addressReserve(&b->own.base, reserve, g, 0, 0) != CUDA_SUCCESS) { delete b; return (int)cudaErrorMemoryAllocation; }
  b->own.reserved = reserve;
  const uint64_t serial = gSerial.fetch_add(1);
  int rc = addOwnChunk(b->own, first, b->device, serial << 8);
  if (rc == 0 && (cudaMemset(reinterpret_cast<void*>(b->own.base), 0, first) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess)) {
    cudaGetLastError();
    rc = (int)cudaErrorUnknown;
  }
  if (rc != 0) {
    unmapAll(b->own, true);
    delete b;
    return rc;
  }
  b->local = reinterpret_cast<void*>(b->own.base);
  b->bytes = first;
  *out = b;
  return 0;
}

int vmmGrow(cocclSymmBuffer* b, size_t bytes) {
  if (bytes <= b->bytes) return 0;
  const size_t g = chunkGranularity(b->device);
  const size_t add = roundUp(bytes - b->bytes, g);
  const size_t at = b->own.mapped;
  const int rc = addOwnChunk(b->own, add, b->device, (serialOf(b) << 8) | (uint64_t)b->own.chunks.size());
  if (rc != 0) return rc;
  if (cudaMemset(reinterpret_cast<void*>(b->own.base + at), 0, add) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    return (int)cudaErrorUnknown;
  }
  b->bytes = b->own.mapped;
  return 0;
}

int vmmExport(const cocclSymmBuffer* b, void* handle) {
  memset(handle, 0, COCCL_SYMM_HANDLE_BYTES);
  VmmHandle h;
  memset(&h, 0, sizeof(h));
  h.magic = kVmmMagic;
  h.pid = (int32_t)getpid();
  h.device = b->device;
  h.nChunks = (int32_t)b->own.chunks.size();
  h.reserveBytes = b->own.reserved;
  h.serial = serialOf(b);
  for (int i = 0; i < h.nChunks; ++i) h.chunkGranules[i] = (uint32_t)(b->own.chunks[(size_t)i].bytes / kGranule);
  memcpy(handle, &h, sizeof(h));
  const SameProcess sp{(unsigned long long)getpid(), b->local, b->device};
  memcpy(static_cast<char*>(handle) + 64, &sp, sizeof(sp));
  return 0;
}

int vmmImport(cocclSymmBuffer* owner, int peer, const void* handle, void** mapped) {
  const Driver& d = driver();
  VmmHandle h;
  memcpy(&h, handle, sizeof(h));
  if (h.magic != kVmmMagic || h.nChunks < 1 || h.nChunks > kMaxChunks) return (int)cudaErrorInvalidValue;
  if ((size_t)peer >= owner->peers.size()) {
    owner->peers.resize((size_t)peer + 1);
    owner->imported.resize((size_t)peer + 1, nullptr);
    owner->direct.resize((size_t)peer + 1, 0);
  }
  int mine = -1;
  if (cudaGetDevice(&mine) != cudaSuccess) return (int)cudaErrorInvalidDevice;
  size_t total = 0;
  for (int i = 0; i < h.nChunks; ++i) total += (size_t)h.chunkGranules[i] * kGranule;
  if (h.pid == (int32_t)getpid()) {
    // ranks of one process: the exporter's range is this process's range; this device only needs access to it
    SameProcess sp;
    memcpy(&sp, static_cast<const char*>(handle) + 64, sizeof(sp));
    if (mine != h.device && grantAccess(reinterpret_cast<CUdeviceptr>(sp.address), total, mine) != 0) return (int)cudaErrorPeerAccessUnsupported;
    owner->imported[(size_t)peer] = sp.address;
    owner->direct[(size_t)peer] = 1;
    *mapped = sp.address;
    return 0;
  }
  VmmMapping& m = owner->peers[(size_t)peer];
  if (m.base == 0) {
    const size_t g = chunkGranularity(mine);
    if (d.addressReserve(&m.base, (size_t)h.reserveBytes, g, 0, 0) != CUDA_SUCCESS) return (int)cudaErrorMemoryAllocation;
    m.reserved = (size_t)h.reserveBytes;
  }
  for (int i = (int)m.chunks.size(); i < h.nChunks; ++i) {
    const size_t bytes = (size_t)h.chunkGranules[i] * kGranule;
    if (m.mapped + bytes > m.reserved) return (int)cudaErrorMemoryAllocation;
    const int fd = fdChannelFetch(h.pid, (h.serial << 8) | (uint64_t)i, kFetchTimeoutMs);
    if (fd < 0) return (int)cudaErrorUnknown;
    VmmChunk c;
    c.bytes = bytes;
    const CUresult r = d.importHandle(&c.handle, reinterpret_cast<void*>((uintptr_t)fd), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    if (r != CUDA_SUCCESS) return (int)cudaErrorUnknown;
    if (d.map(m.base + m.mapped, bytes, 0, c.handle, 0) != CUDA_SUCCESS) { d.release(c.handle); return (int)cudaErrorUnknown; }
    if (grantAccess(m.base + m.mapped, bytes, mine) != 0) {
      d.unmap(m.base + m.mapped, bytes);
      d.release(c.handle);
      return (int)cudaErrorPeerAccessUnsupported;
    }
    m.chunks.push_back(c);
    m.mapped += bytes;
  }
  owner->imported[(size_t)peer] = reinterpret_cast<void*>(m.base);
  owner->direct[(size_t)peer] = 0;
  *mapped = reinterpret_cast<void*>(m.base);
  return 0;
}

int vmmCloseImports(cocclSymmBuffer* b) {
  for (size_t p = 0; p < b->peers.size(); ++p) {
    unmapAll(b->peers[p], false);
    b->imported[p] = nullptr;
  }
  for (size_t p = 0; p < b->imported.size(); ++p) b->imported[p] = nullptr;
  return 0;
}

int vmmFree(cocclSymmBuffer* b) {
  cocclSymmMulticastUnbind(b);
  vmmCloseImports(b);
  unmapAll(b->own, true);
  delete b;
  return 0;
}

}  // namespace coccl

using namespace coccl;

// ------------------------------------------------------------------------------------------------- multicast
extern "C" int cocclSymmMulticastSupported(void) {
  if (!vmmAvailable() || !driver().mcOk) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  return deviceAttr(CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != 0 ? 1 : 0;
}

extern "C" int cocclSymmMulticastCreate(cocclSymmBuffer* b, int nRanks, void* handle) {
  if (!b || !b->vmm || !handle || nRanks < 2 || b->own.chunks.empty() || b->mc.handle != 0) return (int)cudaErrorInvalidValue;
  if (!cocclSymmMulticastSupported()) return (int)cudaErrorNotSupported;
  const Driver& d = driver();
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = (unsigned)nRanks;
  mp.size = b->own.chunks[0].bytes;   // the first chunk: its size is already a multiple of the multicast granularity
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  if (d.mcCreate(&b->mc.handle, &mp) != CUDA_SUCCESS) { b->mc.handle = 0; return (int)cudaErrorNotSupported; }
  int fd = -1;
  const uint64_t key = (serialOf(b) << 8) | 0xffu;
  bool ok = d.exportHandle(&fd, b->mc.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS && fd >= 0;
  if (ok) {
    ok = fdChannelPublish(key, fd) == 0;
    close(fd);
  }
  if (!ok) {
    d.release(b->mc.handle);
    b->mc.handle = 0;
    return (int)cudaErrorUnknown;
  }
  b->mc.key = key;
  b->mc.bytes = mp.size;
  McHandle h;
  memset(&h, 0, sizeof(h));
  h.magic = kVmmMagic;
  h.pid = (int32_t)getpid();
  h.key = key;
  h.bytes = mp.size;
  h.nRanks = nRanks;
  memset(handle, 0, COCCL_SYMM_HANDLE_BYTES);
  memcpy(handle, &h, sizeof(h));
  return 0;
}

extern "C" int cocclSymmMulticastJoin(cocclSymmBuffer* b, const void* handle) {
  if (!b || !b->vmm || !handle || b->own.chunks.empty()) return (int)cudaErrorInvalidValue;
  if (!cocclSymmMulticastSupported()) return (int)cudaErrorNotSupported;
  const Driver& d = driver();
  McHandle h;
  memcpy(&h, handle, sizeof(h));
  if (h.magic != kVmmMagic || h.bytes != b->own.chunks[0].bytes) return (int)cudaErrorInvalidValue;
  if (b->mc.handle == 0) {  // not the creator: import the object
    const int fd = fdChannelFetch(h.pid, h.key, kFetchTimeoutMs);
    if (fd < 0) return (int)cudaErrorUnknown;
    const CUresult r = d.importHandle(&b->mc.handle, reinterpret_cast<void*>((uintptr_t)fd), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    if (r != CUDA_SUCCESS) { b->mc.handle = 0; return (int)cudaErrorUnknown; }
    b->mc.bytes = (size_t)h.bytes;
  }
  if (d.mcAddDevice(b->mc.handle, b->device) != CUDA_SUCCESS) return (int)cudaErrorUnknown;
  b->mc.added = true;
  return 0;
}

extern "C" int cocclSymmMulticastBind(cocclSymmBuffer* b, void** multicastPtr) {
  if (!b || !b->vmm || !multicastPtr || b->mc.handle == 0 || !b->mc.added || b->mc.bound) return (int)cudaErrorInvalidValue;
  const Driver& d = driver();
  if (d.mcBindMem(b->mc.handle, 0, b->own.chunks[0].handle, 0, b->mc.bytes, 0) != CUDA_SUCCESS) return (int)cudaErrorUnknown;
  b->mc.bound = true;
  const size_t g = chunkGranularity(b->device);
  bool ok = d.addressReserve(&b->mc.base, b->mc.bytes, g, 0, 0) == CUDA_SUCCESS;
  if (ok && d.map(b->mc.base, b->mc.bytes, 0, b->mc.handle, 0) != CUDA_SUCCESS) {
    d.addressFree(b->mc.base, b->mc.bytes);
    b->mc.base = 0;
    ok = false;
  }
  if (ok && grantAccess(b->mc.base, b->mc.bytes, b->device) != 0) {
    d.unmap(b->mc.base, b->mc.bytes);
    d.addressFree(b->mc.base, b->mc.bytes);
    b->mc.base = 0;
    ok = false;
  }
  if (!ok) {
    cocclSymmMulticastUnbind(b);
    return (int)cudaErrorUnknown;
  }
  *multicastPtr = reinterpret_cast<void*>(b->mc.base);
  return 0;
}

extern "C" int cocclSymmMulticastUnbind(cocclSymmBuffer* b) {
  if (!b || !b->vmm || b->mc.handle == 0) return 0;
  const Driver& d = driver();
  if (b->mc.base) {
    cudaDeviceSynchronize();  // nothing of this rank is still reducing through the object
    d.unmap(b->mc.base, b->mc.bytes);
    d.addressFree(b->mc.base, b->mc.bytes);
    b->mc.base = 0;
  }
  if (b->mc.bound) {
    d.mcUnbind(b->mc.handle, b->device, 0, b->mc.bytes);
    b->mc.bound = false;
  }
  if (b->mc.key) fdChannelWithdraw(b->mc.key);
  d.release(b->mc.handle);
  b->mc = VmmMulticast{};
  return 0;
}
