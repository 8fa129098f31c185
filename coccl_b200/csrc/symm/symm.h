// Symmetric (peer-mapped) device memory for one NVSwitch domain.
//
// Every rank allocates a buffer of the same size, exports a handle, and maps
// the buffers of all its peers, so that kernels can store encoded tiles
// straight into a peer's receive slot and set flags there. This is what NCCL
// builds for its P2P transport (src/transport/p2p.cc:199-284) and what COCCL's
// VMM workspace grants to every peer-accessible device
// (src/coccl-extend/core/memory/coccl_buffer_vmm.cc:85-102), reduced to the one
// thing the fused kernels need. Handle exchange itself is left to the caller
// (torch.distributed store, NCCL all-gather, a socket): handles are plain bytes.
//
// This interface is the CUDA-IPC backend (cudaMalloc + 64-byte IPC handles). The cuMem VMM backend with
// POSIX file descriptors and the NVSwitch multicast binding is symm_vmm.h.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// export handle: the CUDA IPC handle (64 bytes) followed by the exporter's process id, address and device, which a
// rank of the SAME process uses instead (CUDA IPC handles cannot be opened by the process that made them)
enum { COCCL_SYMM_HANDLE_BYTES = 96 };
int cocclSymmHandleBytes(void);

typedef struct cocclSymmBuffer cocclSymmBuffer;

// Allocate `bytes` of zero-initialised device memory on the current device that peers can map.
int cocclSymmAlloc(size_t bytes, cocclSymmBuffer** out);
// Copy this buffer's export handle (COCCL_SYMM_HANDLE_BYTES bytes).
int cocclSymmExport(const cocclSymmBuffer* buf, void* handle);
// Map a peer's buffer from its handle; returns the local device pointer of the mapping.
int cocclSymmImport(cocclSymmBuffer* owner, int peerIndex, const void* handle, void** mapped);
void* cocclSymmLocalPtr(const cocclSymmBuffer* buf);
size_t cocclSymmBytes(const cocclSymmBuffer* buf);
// Unmap every imported peer; the local allocation stays. CUDA leaves freeing exported memory that a peer still
// has mapped undefined, so a collective teardown is: every rank closes its imports, all ranks meet, then each
// frees its own allocation.
int cocclSymmCloseImports(cocclSymmBuffer* buf);
// Unmap every imported peer (if still mapped) and free the local allocation.
int cocclSymmFree(cocclSymmBuffer* buf);

#ifdef __cplusplus
}
#endif
