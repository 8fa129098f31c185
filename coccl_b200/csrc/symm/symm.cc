// Symmetric memory interface (symm.h): the CUDA-IPC backend, and the dispatch to the cuMem VMM backend (symm_vmm.cc)
// for buffers that were allocated by it.
#include "symm.h"
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
#include <new>
#include <vector>

#include "symm/symm_internal.h"

namespace {
// What follows the IPC handle inside an export handle.
struct SameProcess {
  unsigned long long pid;
  void* address;
  int device;
};
constexpr size_t kIpcBytes = 64;
static_assert(sizeof(cudaIpcMemHandle_t) <= kIpcBytes, "IPC handle does not fit");
static_assert(kIpcBytes + sizeof(SameProcess) <= COCCL_SYMM_HANDLE_BYTES, "export handle too small");
}  // namespace

extern "C" int cocclSymmHandleBytes(void) { return COCCL_SYMM_HANDLE_BYTES; }

namespace coccl {
static int gBackend = -1;
int symmBackend() {
  if (gBackend < 0) {
    // default: cuMem VMM where the driver offers it (buffers grow in place, multicast can be bound), CUDA IPC otherwise;
    // COCCL_SYMM_BACKEND=ipc|vmm forces one
    const char* v = getenv("COCCL_SYMM_BACKEND");
    if (v && strcmp(v, "ipc") == 0) gBackend = COCCL_SYMM_BACKEND_IPC;
    else if (v && strcmp(v, "vmm") == 0) gBackend = COCCL_SYMM_BACKEND_VMM;
    else gBackend = vmmAvailable() ? COCCL_SYMM_BACKEND_VMM : COCCL_SYMM_BACKEND_IPC;
  }
  return gBackend;
}
}  // namespace coccl

extern "C" int cocclSymmSetBackend(int backend) {
  if (backend != COCCL_SYMM_BACKEND_IPC && backend != COCCL_SYMM_BACKEND_VMM) return (int)cudaErrorInvalidValue;
  if (backend == COCCL_SYMM_BACKEND_VMM && !coccl::vmmAvailable()) return (int)cudaErrorNotSupported;
  coccl::gBackend = backend;
  return 0;
}
extern "C" int cocclSymmGetBackend(void) { return coccl::symmBackend(); }

extern "C" int cocclSymmGrow(cocclSymmBuffer* buf, size_t bytes) {
  if (!buf) return (int)cudaErrorInvalidValue;
  if (!buf->vmm) return (int)cudaErrorNotSupported;   // cudaMalloc'd memory cannot grow where it is
  return coccl::vmmGrow(buf, bytes);
}

extern "C" int cocclSymmAlloc(size_t bytes, cocclSymmBuffer** out) {
  if (out == nullptr || bytes == 0) return (int)cudaErrorInvalidValue;
  if (coccl::symmBackend() == COCCL_SYMM_BACKEND_VMM) return coccl::vmmAlloc(bytes, out);
  cocclSymmBuffer* b = new (std::nothrow) cocclSymmBuffer();
  if (!b) return (int)cudaErrorMemoryAllocation;
  cudaError_t e = cudaGetDevice(&b->device);
  if (e == cudaSuccess) e = cudaMalloc(&b->local, bytes);
  if (e == cudaSuccess) e = cudaMemset(b->local, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (b->local) cudaFree(b->local);
    delete b;
    return (int)e;
  }
  b->bytes = bytes;
  *out = b;
  return 0;
}

extern "C" int cocclSymmExport(const cocclSymmBuffer* buf, void* handle) {
  if (!buf || !handle) return (int)cudaErrorInvalidValue;
  if (buf->vmm) return coccl::vmmExport(buf, handle);
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, buf->local);
  if (e != cudaSuccess) return (int)e;
  memset(handle, 0, COCCL_SYMM_HANDLE_BYTES);
  memcpy(handle, &h, sizeof(h));
  const SameProcess sp{(unsigned long long)getpid(), buf->local, buf->device};
  memcpy(static_cast<char*>(handle) + kIpcBytes, &sp, sizeof(sp));
  return 0;
}

extern "C" int cocclSymmImport(cocclSymmBuffer* owner, int peerIndex, const void* handle, void** mapped) {
  if (!owner || !handle || !mapped || peerIndex < 0) return (int)cudaErrorInvalidValue;
  if (owner->vmm) return coccl::vmmImport(owner, peerIndex, handle, mapped);
  if ((size_t)peerIndex >= owner->imported.size()) { owner->imported.resize(peerIndex + 1, nullptr); owner->direct.resize(peerIndex + 1, 0); }
  SameProcess sp;
  memcpy(&sp, static_cast<const char*>(handle) + kIpcBytes, sizeof(sp));
  if (sp.pid == (unsigned long long)getpid() && sp.address != nullptr) {
    // ranks that are threads of one process (one thread per GPU): the exporter's pointer is valid here as it is,
    // the importing device only needs peer access to the exporter's device
    int mine = -1;
    cudaError_t e = cudaGetDevice(&mine);
    if (e != cudaSuccess) return (int)e;
    if (mine != sp.device) {
      int can = 0;
      e = cudaDeviceCanAccessPeer(&can, mine, sp.device);
      if (e != cudaSuccess || !can) { cudaGetLastError(); return (int)(e != cudaSuccess ? e : cudaErrorPeerAccessUnsupported); }
      e = cudaDeviceEnablePeerAccess(sp.device, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
      if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    }
    owner->imported[peerIndex] = sp.address;
    owner->direct[peerIndex] = 1;
    *mapped = sp.address;
    return 0;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();  // the failure must not stay behind as the thread's last error: the caller falls back
    return (int)e;
  }
  owner->imported[peerIndex] = p;
  owner->direct[peerIndex] = 0;
  *mapped = p;
  return 0;
}

extern "C" void* cocclSymmLocalPtr(const cocclSymmBuffer* buf) { return buf ? buf->local : nullptr; }
extern "C" size_t cocclSymmBytes(const cocclSymmBuffer* buf) { return buf ? buf->bytes : 0; }

extern "C" int cocclSymmCloseImports(cocclSymmBuffer* buf) {
  if (!buf) return 0;
  if (buf->vmm) return coccl::vmmCloseImports(buf);
  cudaError_t first = cudaSuccess;
  for (size_t i = 0; i < buf->imported.size(); ++i) {
    void*& p = buf->imported[i];
    if (p && !buf->direct[i]) {
      cudaError_t e = cudaIpcCloseMemHandle(p);
      if (first == cudaSuccess) first = e;
    }
    p = nullptr;
  }
  return (int)first;
}

extern "C" int cocclSymmFree(cocclSymmBuffer* buf) {
  if (!buf) return 0;
  if (buf->vmm) return coccl::vmmFree(buf);
  cudaError_t first = (cudaError_t)cocclSymmCloseImports(buf);
  if (buf->local) {
    cudaError_t e = cudaFree(buf->local);
    if (first == cudaSuccess) first = e;
  }
  delete buf;
  return (int)first;
}

// Small synchronous device->host read (status words).
extern "C" int cocclHostRead32(const void* dev, unsigned int* out) {
  return (int)cudaMemcpy(out, dev, sizeof(unsigned int), cudaMemcpyDeviceToHost);
}

// Stream-ordered read of `words` 32-bit words into pinned host memory (status words, polled later without a sync).
extern "C" int cocclAsyncRead32(void* pinnedHost, const void* dev, int words, cudaStream_t stream) {
  return (int)cudaMemcpyAsync(pinnedHost, dev, (size_t)words * sizeof(unsigned int), cudaMemcpyDeviceToHost, stream);
}

// Stream-ordered device-to-device copy between raw addresses (e.g. out of a symmetric workspace, which has no
// framework tensor behind it).
extern "C" int cocclDeviceCopy(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  if (bytes == 0) return 0;
  return (int)cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
}
