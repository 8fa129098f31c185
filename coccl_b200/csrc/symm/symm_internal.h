// Shared between the two backends of the symmetric memory (symm.cc: CUDA IPC, symm_vmm.cc: cuMem VMM).
#pragma once
#include <cuda.h>
#include <stddef.h>

#include <vector>

#include "symm/symm.h"

namespace coccl {
struct VmmChunk {              // one physical allocation
  CUmemGenericAllocationHandle handle = 0;
  size_t bytes = 0;
  unsigned long long key = 0;  // under which its descriptor is published (fd_channel.h); 0 = imported chunk
};
struct VmmMapping {            // a contiguous virtual range and the chunks mapped into it, in order
  CUdeviceptr base = 0;
  size_t reserved = 0, mapped = 0;
  std::vector<VmmChunk> chunks;
};
struct VmmMulticast {
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr base = 0;
  size_t bytes = 0;
  unsigned long long key = 0;
  bool added = false, bound = false;
};
}  // namespace coccl

struct cocclSymmBuffer {
  void* local = nullptr;
  size_t bytes = 0;
  int device = -1;
  std::vector<void*> imported;  // by peer index; nullptr = not mapped
  std::vector<char> direct;     // by peer index; 1 = same-process pointer, nothing to close
  // cuMem VMM backend only
  bool vmm = false;
  coccl::VmmMapping own;
  std::vector<coccl::VmmMapping> peers;  // by peer index
  coccl::VmmMulticast mc;
};

namespace coccl {
int symmBackend();
bool vmmAvailable();
int vmmAlloc(size_t bytes, cocclSymmBuffer** out);
int vmmGrow(cocclSymmBuffer* buf, size_t bytes);
int vmmExport(const cocclSymmBuffer* buf, void* handle);
int vmmImport(cocclSymmBuffer* owner, int peerIndex, const void* handle, void** mapped);
int vmmCloseImports(cocclSymmBuffer* buf);
int vmmFree(cocclSymmBuffer* buf);
}  // namespace coccl
