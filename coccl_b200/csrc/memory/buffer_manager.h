// Workspace buffers of the staged pipeline.
//
//  * BufferManager: per-communicator pool behind a global mutex; hands out leases
//    {ptr, bytes, owner, block, slice}, "registered" ones (peer-mapped / registered with the
//    transport, used for edges that a collective reads or writes) and "unregistered" ones (raw
//    boundary temps). Implements the pipeline's WorkspaceProvider.
//  * SliceBackend ("legacy"): device blocks cut into slices {Free, InUse, Pending}. Releasing a
//    slice records an event and leaves it Pending; a Pending slice is handed to a request on the
//    SAME stream without waiting, to another stream only once its event has completed; adjacent
//    free slices merge.
//  * VmmBackend: one virtual range per block, physical chunks of `physical_chunk_bytes` created
//    with cuMemCreate, mapped and made accessible to every peer-accessible device; a block grows
//    IN PLACE by reserving a larger range and re-mapping the old handles plus new ones.
//
// Behavioural model: src/coccl-extend/core/memory/coccl_buffer_management.cc:22-195,
// coccl_buffer_legacy.cc:11-225, coccl_buffer_vmm.cc:16-448. All CUDA entry points go through
// function tables so that the host tests can substitute fakes and assert the call order
// (the reference does the same in tests/coccl-tests/src/coccl_vmm_buffer_test.cc:48-120).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "pipeline/pipeline.h"

namespace coccl {

struct EventApi {
  cudaError_t (*create)(cudaEvent_t* e);
  cudaError_t (*record)(cudaEvent_t e, cudaStream_t s);
  cudaError_t (*query)(cudaEvent_t e);  // cudaSuccess = complete, cudaErrorNotReady = pending
  cudaError_t (*sync)(cudaEvent_t e);
  cudaError_t (*destroy)(cudaEvent_t e);
};
const EventApi& cudaEventApi();

struct VmmDriverApi {
  CUresult (*getGranularity)(size_t* g, const CUmemAllocationProp* prop, CUmemAllocationGranularity_flags f);
  CUresult (*addressReserve)(CUdeviceptr* p, size_t size, size_t align, CUdeviceptr hint, unsigned long long flags);
  CUresult (*addressFree)(CUdeviceptr p, size_t size);
  CUresult (*create)(CUmemGenericAllocationHandle* h, size_t size, const CUmemAllocationProp* prop, unsigned long long flags);
  CUresult (*release)(CUmemGenericAllocationHandle h);
  CUresult (*map)(CUdeviceptr p, size_t size, size_t offset, CUmemGenericAllocationHandle h, unsigned long long flags);
  CUresult (*unmap)(CUdeviceptr p, size_t size);
  CUresult (*setAccess)(CUdeviceptr p, size_t size, const CUmemAccessDesc* desc, size_t count);
  // devices that can reach `device` (itself included)
  int (*peerDevices)(int device, int* out, int capacity);
  // whether the device supports VMM (and VMM with GPUDirect RDMA where the transport needs it)
  bool (*supported)(int device);
};
// Driver entry points resolved at run time (no link-time dependency on libcuda).
const VmmDriverApi* cudaVmmDriverApi();

class BufferBackend {
 public:
  virtual ~BufferBackend() {}
  virtual ncclResult_t acquire(size_t bytes, cudaStream_t stream, void** ptr, int* block, int* slice) = 0;
  virtual ncclResult_t release(int block, int slice, cudaStream_t stream) = 0;
  virtual size_t reservedBytes() const = 0;
  virtual const char* name() const = 0;
};

// ---------------------------------------------------------------------------------------------
class SliceBackend : public BufferBackend {
 public:
  enum class State { Free, InUse, Pending };
  struct Slice { size_t offset, bytes; State state; cudaEvent_t event; cudaStream_t stream; };
  struct Block { char* base; size_t bytes; std::vector<Slice> slices; };

  SliceBackend(const DeviceAllocator* alloc, const EventApi* events, size_t blockBytes);
  ~SliceBackend() override;
  ncclResult_t acquire(size_t bytes, cudaStream_t stream, void** ptr, int* block, int* slice) override;
  ncclResult_t release(int block, int slice, cudaStream_t stream) override;
  size_t reservedBytes() const override;
  const char* name() const override { return "slices"; }
  const std::vector<Block>& blocks() const { return blocks_; }

 private:
  bool reusable(Slice& s, cudaStream_t stream);
  void mergeFree(Block& b);
  const DeviceAllocator* alloc_;
  const EventApi* events_;
  size_t blockBytes_;
  std::vector<Block> blocks_;
};

// ---------------------------------------------------------------------------------------------
class VmmBackend : public BufferBackend {
 public:
  VmmBackend(const VmmDriverApi* api, int device, size_t chunkBytes);
  ~VmmBackend() override;
  // One growing block: every acquire returns the block base; callers hold at most one lease at a time
  // per backend instance (the manager keeps one instance per communicator and kind).
  ncclResult_t acquire(size_t bytes, cudaStream_t stream, void** ptr, int* block, int* slice) override;
  ncclResult_t release(int block, int slice, cudaStream_t stream) override;
  size_t reservedBytes() const override { return mapped_; }
  const char* name() const override { return "vmm"; }
  size_t granularity() const { return granularity_; }
  size_t chunks() const { return handles_.size(); }

 private:
  ncclResult_t init();
  ncclResult_t grow(size_t bytes);
  ncclResult_t mapRange(CUdeviceptr base, size_t fromChunk, size_t toChunk);
  const VmmDriverApi* api_;
  int device_;
  size_t chunkBytes_, granularity_ = 0;
  bool ready_ = false, busy_ = false;
  CUdeviceptr base_ = 0;
  size_t reserved_ = 0, mapped_ = 0;
  std::vector<CUmemGenericAllocationHandle> handles_;
};

// ---------------------------------------------------------------------------------------------
struct BufferLease {
  void* ptr = nullptr;
  size_t bytes = 0;
  Comm* owner = nullptr;
  bool registered = false;
  int block = -1, slice = -1;
};

struct BufferOptions {
  size_t legacyBlockBytes = 0;           // 0 = size blocks to the request (rounded to 2 MiB)
  size_t physicalChunkBytes = 8ull << 20;
  size_t poolLimitBytes = 0;             // parsed, reported, not enforced (as in the reference)
  bool preferVmm = true;
  const DeviceAllocator* alloc = nullptr;
  const EventApi* events = nullptr;
  const VmmDriverApi* vmm = nullptr;
};

class BufferManager : public WorkspaceProvider {
 public:
  explicit BufferManager(const BufferOptions& opt);
  ~BufferManager() override;
  ncclResult_t commInit(Comm* comm);
  ncclResult_t commDestroy(Comm* comm);
  ncclResult_t getBuffer(Comm* comm, size_t bytes, bool registered, cudaStream_t stream, BufferLease* lease);
  ncclResult_t releaseBuffer(BufferLease* lease, cudaStream_t stream);
  // WorkspaceProvider
  ncclResult_t acquire(Comm* comm, size_t bytes, bool registered, cudaStream_t stream, void** ptr, void** lease) override;
  void release(void* lease, cudaStream_t stream) override;
  size_t reservedBytes(Comm* comm) const;
  const char* backendName(Comm* comm, bool registered) const;

 private:
  struct Pool { std::unique_ptr<BufferBackend> registered, unregistered; };
  Pool* poolFor(Comm* comm);
  BufferOptions opt_;
  mutable std::mutex mutex_;
  std::map<Comm*, Pool> pools_;
};

}  // namespace coccl
