#include "memory/buffer_manager.h"

#include <algorithm>

#include "runtime/log.h"

namespace coccl {

// ------------------------------------------------------------------ event API
static cudaError_t evCreate(cudaEvent_t* e) { return cudaEventCreateWithFlags(e, cudaEventDisableTiming); }
static cudaError_t evRecord(cudaEvent_t e, cudaStream_t s) { return cudaEventRecord(e, s); }
static cudaError_t evQuery(cudaEvent_t e) { return cudaEventQuery(e); }
static cudaError_t evSync(cudaEvent_t e) { return cudaEventSynchronize(e); }
static cudaError_t evDestroy(cudaEvent_t e) { return cudaEventDestroy(e); }
const EventApi& cudaEventApi() {
  static const EventApi a = {&evCreate, &evRecord, &evQuery, &evSync, &evDestroy};
  return a;
}

// ------------------------------------------------------------------ slice backend
SliceBackend::SliceBackend(const DeviceAllocator* alloc, const EventApi* events, size_t blockBytes)
    : alloc_(alloc), events_(events), blockBytes_(blockBytes) {}

SliceBackend::~SliceBackend() {
  for (Block& b : blocks_) {
    for (Slice& s : b.slices)
      if (s.event) { events_->sync(s.event); events_->destroy(s.event); }
    alloc_->freeSync(b.base);
  }
}

size_t SliceBackend::reservedBytes() const {
  size_t n = 0;
  for (const Block& b : blocks_) n += b.bytes;
  return n;
}

bool SliceBackend::reusable(Slice& s, cudaStream_t stream) {
  if (s.state == State::Free) return true;
  if (s.state != State::Pending) return false;
  if (s.stream == stream) return true;  // stream order already protects the previous user
  if (events_->query(s.event) == cudaSuccess) {
    s.state = State::Free;
    return true;
  }
  return false;
}

void SliceBackend::mergeFree(Block& b) {
  for (size_t i = 0; i + 1 < b.slices.size();) {
    Slice& a = b.slices[i];
    Slice& n = b.slices[i + 1];
    auto settled = [&](Slice& s) {
      if (s.state == State::Pending && events_->query(s.event) == cudaSuccess) s.state = State::Free;
      return s.state == State::Free;
    };
    if (settled(a) && settled(n)) {
      a.bytes += n.bytes;
      if (n.event) events_->destroy(n.event);
      b.slices.erase(b.slices.begin() + i + 1);
    } else {
      ++i;
    }
  }
}

ncclResult_t SliceBackend::acquire(size_t bytes, cudaStream_t stream, void** ptr, int* block, int* slice) {
  const size_t need = alignUpSize(bytes ? bytes : 1, kWorkspaceAlign);
  for (int pass = 0; pass < 2; ++pass) {
    for (size_t bi = 0; bi < blocks_.size(); ++bi) {
      Block& b = blocks_[bi];
      if (pass == 1) mergeFree(b);
      for (size_t si = 0; si < b.slices.size(); ++si) {
        Slice& s = b.slices[si];
        if (s.bytes < need || !reusable(s, stream)) continue;
        if (s.bytes > need) {  // split: the remainder inherits the state (a Pending tail stays Pending)
          Slice rest = s;
          rest.offset = s.offset + need;
          rest.bytes = s.bytes - need;
          rest.event = nullptr;
          if (s.state == State::Pending) {
            // the tail must wait for the same event; give it its own, recorded now on the old stream
            if (events_->create(&rest.event) != cudaSuccess) return ncclUnhandledCudaError;
            events_->record(rest.event, s.stream);
          }
          s.bytes = need;
          b.slices.insert(b.slices.begin() + si + 1, rest);
        }
        Slice& got = b.slices[si];
        got.state = State::InUse;
        got.stream = stream;
        *ptr = b.base + got.offset;
        *block = (int)bi;
        *slice = (int)got.offset;  // slices are identified by their offset: indices move when neighbours merge
        return ncclSuccess;
      }
    }
  }
  // new block
  size_t blockBytes = blockBytes_ ? std::max(blockBytes_, need) : alignUpSize(need, 2ull << 20);
  void* base = nullptr;
  if (alloc_->mallocSync(&base, blockBytes) != cudaSuccess) return ncclUnhandledCudaError;
  Block b;
  b.base = static_cast<char*>(base);
  b.bytes = blockBytes;
  b.slices.push_back({0, need, State::InUse, nullptr, stream});
  if (blockBytes > need) b.slices.push_back({need, blockBytes - need, State::Free, nullptr, nullptr});
  blocks_.push_back(b);
  COCCL_INFO(kLogMemory, "slice backend: new block of %zu B (total %zu B)", blockBytes, reservedBytes());
  *ptr = base;
  *block = (int)blocks_.size() - 1;
  *slice = 0;
  return ncclSuccess;
}

ncclResult_t SliceBackend::release(int block, int slice, cudaStream_t stream) {
  if (block < 0 || (size_t)block >= blocks_.size()) return ncclInvalidArgument;
  Block& b = blocks_[block];
  for (Slice& s : b.slices) {
    if ((int)s.offset != slice || s.state != State::InUse) continue;
    if (s.event == nullptr && events_->create(&s.event) != cudaSuccess) return ncclUnhandledCudaError;
    if (events_->record(s.event, stream) != cudaSuccess) return ncclUnhandledCudaError;
    s.state = State::Pending;
    s.stream = stream;
    return ncclSuccess;
  }
  return ncclInvalidArgument;
}

// ------------------------------------------------------------------ VMM backend
VmmBackend::VmmBackend(const VmmDriverApi* api, int device, size_t chunkBytes)
    : api_(api), device_(device), chunkBytes_(chunkBytes ? chunkBytes : (8ull << 20)) {}

VmmBackend::~VmmBackend() {
  if (base_ && mapped_) api_->unmap(base_, mapped_);
  for (CUmemGenericAllocationHandle h : handles_) api_->release(h);
  if (base_) api_->addressFree(base_, reserved_);
}

static CUmemAllocationProp vmmProp(int device) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

ncclResult_t VmmBackend::init() {
  if (ready_) return ncclSuccess;
  CUmemAllocationProp prop = vmmProp(device_);
  size_t g = 0;
  if (api_->getGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0) return ncclSystemError;
  granularity_ = g;
  chunkBytes_ = alignUpSize(chunkBytes_, g);
  ready_ = true;
  return ncclSuccess;
}

ncclResult_t VmmBackend::mapRange(CUdeviceptr base, size_t fromChunk, size_t toChunk) {
  int peers[64];
  const int n = api_->peerDevices(device_, peers, 64);
  std::vector<CUmemAccessDesc> access((size_t)n);
  for (int i = 0; i < n; ++i) {
    access[i].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access[i].location.id = peers[i];
    access[i].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  }
  for (size_t c = fromChunk; c < toChunk; ++c)
    if (api_->map(base + c * chunkBytes_, chunkBytes_, 0, handles_[c], 0) != CUDA_SUCCESS) return ncclSystemError;
  if (toChunk > fromChunk &&
      api_->setAccess(base + fromChunk * chunkBytes_, (toChunk - fromChunk) * chunkBytes_, access.data(), access.size()) != CUDA_SUCCESS)
    return ncclSystemError;
  return ncclSuccess;
}

ncclResult_t VmmBackend::grow(size_t bytes) {
  const size_t wantChunks = (bytes + chunkBytes_ - 1) / chunkBytes_;
  const size_t oldChunks = handles_.size();
  if (wantChunks <= oldChunks) return ncclSuccess;
  CUmemAllocationProp prop = vmmProp(device_);
  for (size_t c = oldChunks; c < wantChunks; ++c) {
    CUmemGenericAllocationHandle h;
    if (api_->create(&h, chunkBytes_, &prop, 0) != CUDA_SUCCESS) return ncclSystemError;
    handles_.push_back(h);
  }
  const size_t newBytes = wantChunks * chunkBytes_;
  if (newBytes > reserved_) {
    // grow in place: a larger range takes over the existing physical chunks, then the new ones
    CUdeviceptr nb = 0;
    if (api_->addressReserve(&nb, newBytes, granularity_, 0, 0) != CUDA_SUCCESS) return ncclSystemError;
    if (base_) {
      if (mapped_ && api_->unmap(base_, mapped_) != CUDA_SUCCESS) return ncclSystemError;
      api_->addressFree(base_, reserved_);
    }
    base_ = nb;
    reserved_ = newBytes;
    mapped_ = 0;
    ncclResult_t r = mapRange(base_, 0, wantChunks);
    if (r != ncclSuccess) return r;
  } else {
    ncclResult_t r = mapRange(base_, oldChunks, wantChunks);
    if (r != ncclSuccess) return r;
  }
  mapped_ = newBytes;
  COCCL_INFO(kLogMemory, "vmm backend: %zu chunks of %zu B mapped at %p", wantChunks, chunkBytes_, (void*)base_);
  return ncclSuccess;
}

ncclResult_t VmmBackend::acquire(size_t bytes, cudaStream_t, void** ptr, int* block, int* slice) {
  ncclResult_t r = init();
  if (r != ncclSuccess) return r;
  if (busy_) return ncclInvalidUsage;
  if ((r = grow(bytes ? bytes : 1)) != ncclSuccess) return r;
  busy_ = true;
  *ptr = reinterpret_cast<void*>(base_);
  *block = 0;
  *slice = 0;
  return ncclSuccess;
}

ncclResult_t VmmBackend::release(int, int, cudaStream_t) {
  busy_ = false;
  return ncclSuccess;
}

// ------------------------------------------------------------------ manager
BufferManager::BufferManager(const BufferOptions& opt) : opt_(opt) {
  if (opt_.alloc == nullptr) opt_.alloc = &cudaDeviceAllocator();
  if (opt_.events == nullptr) opt_.events = &cudaEventApi();
}
BufferManager::~BufferManager() {}

ncclResult_t BufferManager::commInit(Comm* comm) {
  std::lock_guard<std::mutex> lock(mutex_);
  pools_[comm];
  return ncclSuccess;
}

ncclResult_t BufferManager::commDestroy(Comm* comm) {
  std::lock_guard<std::mutex> lock(mutex_);
  pools_.erase(comm);
  return ncclSuccess;
}

BufferManager::Pool* BufferManager::poolFor(Comm* comm) {
  Pool& p = pools_[comm];
  if (!p.unregistered) p.unregistered.reset(new SliceBackend(opt_.alloc, opt_.events, opt_.legacyBlockBytes));
  if (!p.registered) {
    const VmmDriverApi* vmm = opt_.vmm;
    if (opt_.preferVmm && vmm != nullptr && vmm->supported(comm->cudaDev))
      p.registered.reset(new VmmBackend(vmm, comm->cudaDev, opt_.physicalChunkBytes));
    else
      p.registered.reset(new SliceBackend(opt_.alloc, opt_.events, opt_.legacyBlockBytes));
  }
  return &p;
}

ncclResult_t BufferManager::getBuffer(Comm* comm, size_t bytes, bool registered, cudaStream_t stream, BufferLease* lease) {
  if (comm == nullptr || lease == nullptr) return ncclInvalidArgument;
  std::lock_guard<std::mutex> lock(mutex_);
  Pool* p = poolFor(comm);
  BufferBackend* b = registered ? p->registered.get() : p->unregistered.get();
  BufferLease l;
  ncclResult_t r = b->acquire(bytes, stream, &l.ptr, &l.block, &l.slice);
  if (r == ncclInvalidUsage && registered) {
    // the growing block is already leased (nested pipelines): fall back to slices for this request
    b = p->unregistered.get();
    r = b->acquire(bytes, stream, &l.ptr, &l.block, &l.slice);
    registered = false;
  }
  if (r != ncclSuccess) return r;
  l.bytes = bytes;
  l.owner = comm;
  l.registered = registered;
  *lease = l;
  return ncclSuccess;
}

ncclResult_t BufferManager::releaseBuffer(BufferLease* lease, cudaStream_t stream) {
  if (lease == nullptr || lease->owner == nullptr) return ncclInvalidArgument;
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = pools_.find(lease->owner);
  if (it == pools_.end()) return ncclInvalidArgument;
  BufferBackend* b = lease->registered ? it->second.registered.get() : it->second.unregistered.get();
  ncclResult_t r = b->release(lease->block, lease->slice, stream);
  *lease = BufferLease();
  return r;
}

ncclResult_t BufferManager::acquire(Comm* comm, size_t bytes, bool registered, cudaStream_t stream, void** ptr, void** lease) {
  BufferLease* l = new BufferLease();
  ncclResult_t r = getBuffer(comm, bytes, registered, stream, l);
  if (r != ncclSuccess) {
    delete l;
    return r;
  }
  *ptr = l->ptr;
  *lease = l;
  return ncclSuccess;
}

void BufferManager::release(void* lease, cudaStream_t stream) {
  BufferLease* l = static_cast<BufferLease*>(lease);
  if (l == nullptr) return;
  releaseBuffer(l, stream);
  delete l;
}

size_t BufferManager::reservedBytes(Comm* comm) const {
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = pools_.find(comm);
  if (it == pools_.end()) return 0;
  size_t n = 0;
  if (it->second.registered) n += it->second.registered->reservedBytes();
  if (it->second.unregistered) n += it->second.unregistered->reservedBytes();
  return n;
}

const char* BufferManager::backendName(Comm* comm, bool registered) const {
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = pools_.find(comm);
  if (it == pools_.end()) return "none";
  const auto& b = registered ? it->second.registered : it->second.unregistered;
  return b ? b->name() : "none";
}

}  // namespace coccl
