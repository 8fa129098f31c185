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
// Two backends sit behind this interface. CUDA IPC (COCCL_SYMM_BACKEND=ipc, or where cuMem is missing): cudaMalloc +
// 64-byte IPC handles; growing means a new allocation and a new mapping on every peer. cuMem VMM (the default): physical
// chunks from cuMemCreate, exported as POSIX file descriptors that travel between processes over a Unix socket
// (fd_channel.h), mapped into a virtual range that is reserved larger than the buffer, so that cocclSymmGrow adds
// chunks behind the existing ones and every pointer stays valid; such a buffer can also be bound to an NVSwitch
// multicast object (cocclSymmMulticast*), which gives the multimem kernels one address that reaches every rank.
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

enum { COCCL_SYMM_BACKEND_IPC = 0, COCCL_SYMM_BACKEND_VMM = 1 };
// Backend of the buffers allocated from now on (existing buffers keep theirs). VMM is refused with
// cudaErrorNotSupported where the driver lacks cuMem or POSIX-descriptor handles.
int cocclSymmSetBackend(int backend);
int cocclSymmGetBackend(void);
// VMM buffers only: make the buffer at least `bytes` long WITHOUT moving it. The local pointer and every mapping a
// peer holds stay valid; peers see the new part after they import the buffer's next export handle (the import maps
// only the chunks it does not have yet and returns the same pointer). Collective use: every rank grows, exports,
// the handles are exchanged, every rank imports every peer again.
int cocclSymmGrow(cocclSymmBuffer* buf, size_t bytes);

// ---- NVSwitch multicast over a VMM buffer (collective; the caller moves the small handles between the ranks) ----
// 1. the root calls cocclSymmMulticastCreate(buf, nRanks, handle) and sends `handle` to every rank;
// 2. every rank (the root too) calls cocclSymmMulticastJoin(buf, handle): imports the object where needed and adds
//    its device; ALL ranks must have joined before any of them binds (the caller's barrier);
// 3. every rank calls cocclSymmMulticastBind(buf, &ptr): binds the first chunk of its buffer and maps the object;
//    `ptr` is the multicast address of byte 0 of the buffer;
// 4. teardown: every rank calls cocclSymmMulticastUnbind while all ranks are still alive, the ranks meet, then the
//    buffers are freed as usual. A rank must not exit with its memory still bound.
// The multicast range covers the buffer as it was when the object was created (later growth is not part of it).
int cocclSymmMulticastSupported(void);
int cocclSymmMulticastCreate(cocclSymmBuffer* buf, int nRanks, void* handle);
int cocclSymmMulticastJoin(cocclSymmBuffer* buf, const void* handle);
int cocclSymmMulticastBind(cocclSymmBuffer* buf, void** multicastPtr);
int cocclSymmMulticastUnbind(cocclSymmBuffer* buf);

#ifdef __cplusplus
}
#endif
