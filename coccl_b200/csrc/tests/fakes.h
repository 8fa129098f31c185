// Fakes shared by the host tests: an in-memory transport that records calls, a configurable
// compressor plugin, a host allocator, fake CUDA events and a fake VMM driver with a call log.
#pragma once
#include <stdlib.h>
#include <string.h>
#include <map>
#include <string>
#include <vector>

#include "compressor_plugin/coccl_compressor_plugin.h"
#include "memory/buffer_manager.h"
#include "runtime/runtime.h"

namespace fakes {

// ------------------------------------------------------------------ transport
struct FakeTransport : coccl::Transport {
  std::vector<std::string> log;
  int nativeCalls = 0, groupDepth = 0, splits = 0;
  ncclResult_t fail = ncclSuccess;
  ncclResult_t note(const char* what) { log.push_back(what); ++nativeCalls; return fail; }
  ncclResult_t allGather(coccl::Comm*, const void*, void*, size_t, ncclDataType_t, cudaStream_t) override { return note("allGather"); }
  ncclResult_t reduceScatter(coccl::Comm*, const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, cudaStream_t) override { return note("reduceScatter"); }
  ncclResult_t allReduce(coccl::Comm*, const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, cudaStream_t) override { return note("allReduce"); }
  ncclResult_t allToAll(coccl::Comm*, const void*, void*, size_t, ncclDataType_t, cudaStream_t) override { return note("allToAll"); }
  ncclResult_t send(coccl::Comm*, const void*, size_t, ncclDataType_t, int, cudaStream_t) override { return note("send"); }
  ncclResult_t recv(coccl::Comm*, void*, size_t, ncclDataType_t, int, cudaStream_t) override { return note("recv"); }
  ncclResult_t groupStart() override { ++groupDepth; return ncclSuccess; }
  ncclResult_t groupEnd() override { --groupDepth; log.push_back("groupEnd"); return ncclSuccess; }
  ncclResult_t p2pBatch(coccl::Comm*, const coccl::P2POp*, int, cudaStream_t) override { return note("p2pBatch"); }
  ncclResult_t split(coccl::Comm* parent, int color, int, coccl::Comm** child) override {
    ++splits;
    coccl::Comm* c = new coccl::Comm();
    c->transport = this;
    c->cudaDev = parent->cudaDev;
    const bool byNode = color == parent->rank / parent->localRanks;
    c->nRanks = byNode ? parent->localRanks : parent->nNodes;
    c->rank = byNode ? parent->localRank : parent->node;
    *child = c;
    return ncclSuccess;
  }
  void destroy(coccl::Comm* c) override { delete c; }
};

inline coccl::Comm makeComm(FakeTransport* t, int rank, int nRanks, int nNodes) {
  coccl::Comm c;
  c.rank = rank; c.nRanks = nRanks; c.nNodes = nNodes; c.localRanks = nRanks / nNodes;
  c.localRank = rank % c.localRanks; c.node = rank / c.localRanks; c.transport = t; c.id = 100 + rank;
  return c;
}

// ------------------------------------------------------------------ plugin
// One process-wide configurable codec: encoded size = raw / ratio (ratio < 1 expands).
struct PluginKnobs {
  double compressRatio = 4.0, drcRatio = 4.0;
  bool framed = false, lossless = false, fusedSwizzle = false, hasReduce = true, hasDrc = true;
  bool sizeBoundUnknown = false;
  int compressCalls = 0, decompressCalls = 0, reduceCalls = 0, drcCalls = 0, parseCalls = 0;
  std::string rejectKey;  // parseConfig fails when this key is present
};
inline PluginKnobs& knobs() { static PluginKnobs k; return k; }

inline ncclResult_t fakeExecute(cocclCompressorCall* call) {
  PluginKnobs& k = knobs();
  cocclCompressorView* out = call->output;
  switch (call->operation) {
    case cocclCompressorOperationCompress: {
      ++k.compressCalls;
      size_t bytes = (size_t)((double)call->input.bytes / k.compressRatio);
      bytes = (bytes / call->input.chunks) * call->input.chunks;
      if (bytes == 0) bytes = call->input.chunks;
      if (bytes > out->capacityBytes) return ncclInvalidArgument;
      out->bytes = bytes; out->elements = bytes; out->chunks = call->input.chunks; out->datatype = ncclInt8;
      return ncclSuccess;
    }
    case cocclCompressorOperationDecompress: ++k.decompressCalls; out->bytes = out->elements * cocclTypeSize(out->datatype); return ncclSuccess;
    case cocclCompressorOperationDecompressReduce:
      if (!k.hasReduce) return ncclInvalidUsage;
      ++k.reduceCalls; out->bytes = out->elements * cocclTypeSize(out->datatype); return ncclSuccess;
    case cocclCompressorOperationDecompressReduceCompress: {
      if (!k.hasDrc) return ncclInvalidUsage;
      ++k.drcCalls;
      size_t raw = call->originalElements * cocclTypeSize(call->originalDatatype);
      size_t chunks = call->input.chunks / call->reduceChunks;
      size_t bytes = (size_t)((double)raw / k.drcRatio) / chunks * chunks;
      if (bytes == 0) bytes = chunks;
      if (bytes > out->capacityBytes) return ncclInvalidArgument;
      out->bytes = bytes; out->elements = bytes; out->chunks = chunks; out->datatype = ncclInt8;
      return ncclSuccess;
    }
  }
  return ncclInvalidArgument;
}
inline ncclResult_t fakeParse(const cocclConfigView* v, const cocclCompressorConfigContext*, void** cfg, char* err, size_t cap) {
  PluginKnobs& k = knobs();
  ++k.parseCalls;
  for (size_t i = 0; v && i < v->count; ++i)
    if (!k.rejectKey.empty() && k.rejectKey == v->pairs[i].key) { snprintf(err, cap, "option '%s' rejected", v->pairs[i].key); return ncclInvalidArgument; }
  *cfg = malloc(4);
  return ncclSuccess;
}
inline void fakeDestroy(void* c) { free(c); }
inline ncclResult_t fakeBound(const cocclCompressorSizeQuery* q, size_t* bytes) {
  PluginKnobs& k = knobs();
  if (k.sizeBoundUnknown) return ncclInvalidUsage;
  const size_t raw = q->elements * cocclTypeSize(q->datatype);
  const double ratio = q->operation == cocclCompressorOperationDecompressReduceCompress ? k.drcRatio : k.compressRatio;
  size_t b = (size_t)((double)raw / ratio);
  b = (b + q->chunks - 1) / q->chunks * q->chunks;
  if (b == 0) b = q->chunks;
  *bytes = b;
  return ncclSuccess;
}
inline const cocclCompressorPlugin* fakePlugin(const char* name = "fake") {
  static std::map<std::string, cocclCompressorPlugin> made;
  static std::map<std::string, std::string> names;
  PluginKnobs& k = knobs();
  names[name] = name;
  cocclCompressorPlugin& p = made[name];
  p.abiVersion = COCCL_COMPRESSOR_ABI_VERSION;
  p.structSize = sizeof(cocclCompressorPlugin);
  p.name = names[name].c_str();
  p.capabilities = cocclCompressorCapabilityCompress | cocclCompressorCapabilityDecompress |
                   (k.hasReduce ? cocclCompressorCapabilityDecompressReduce : 0) |
                   (k.hasDrc ? cocclCompressorCapabilityDecompressReduceCompress : 0) |
                   (k.framed ? cocclCompressorCapabilityFramed : 0) |
                   (k.fusedSwizzle ? cocclCompressorCapabilityFusedHierarchicalSwizzle : 0) |
                   (k.lossless ? cocclCompressorCapabilityBytewiseLossless : 0);
  p.execute = &fakeExecute;
  p.parseConfig = &fakeParse;
  p.destroyConfig = &fakeDestroy;
  p.getEncodedSizeBound = &fakeBound;
  return &p;
}

// ------------------------------------------------------------------ allocator / events
struct AllocLog { int mallocs = 0, frees = 0, asyncMallocs = 0, asyncFrees = 0; size_t live = 0; bool failNext = false; };
inline AllocLog& allocLog() { static AllocLog l; return l; }
inline cudaError_t hostMallocAsync(void** p, size_t n, cudaStream_t) {
  if (allocLog().failNext) { allocLog().failNext = false; return cudaErrorMemoryAllocation; }
  *p = malloc(n ? n : 1); ++allocLog().asyncMallocs; return cudaSuccess;
}
inline cudaError_t hostFreeAsync(void* p, cudaStream_t) { free(p); ++allocLog().asyncFrees; return cudaSuccess; }
inline cudaError_t hostMalloc(void** p, size_t n) {
  if (allocLog().failNext) { allocLog().failNext = false; return cudaErrorMemoryAllocation; }
  *p = malloc(n ? n : 1); ++allocLog().mallocs; allocLog().live += n; return cudaSuccess;
}
inline cudaError_t hostFree(void* p) { free(p); ++allocLog().frees; return cudaSuccess; }
inline const coccl::DeviceAllocator& hostAllocator() {
  static const coccl::DeviceAllocator a = {&hostMallocAsync, &hostFreeAsync, &hostMalloc, &hostFree};
  return a;
}

// Fake events: an event completes when the test says so.
struct FakeEvent { bool done = false; cudaStream_t stream = nullptr; };
inline std::vector<FakeEvent*>& liveEvents() { static std::vector<FakeEvent*> v; return v; }
inline cudaError_t fevCreate(cudaEvent_t* e) { FakeEvent* f = new FakeEvent(); liveEvents().push_back(f); *e = reinterpret_cast<cudaEvent_t>(f); return cudaSuccess; }
inline cudaError_t fevRecord(cudaEvent_t e, cudaStream_t s) { auto* f = reinterpret_cast<FakeEvent*>(e); f->done = false; f->stream = s; return cudaSuccess; }
inline cudaError_t fevQuery(cudaEvent_t e) { return reinterpret_cast<FakeEvent*>(e)->done ? cudaSuccess : cudaErrorNotReady; }
inline cudaError_t fevSync(cudaEvent_t e) { reinterpret_cast<FakeEvent*>(e)->done = true; return cudaSuccess; }
inline cudaError_t fevDestroy(cudaEvent_t e) { (void)e; return cudaSuccess; }
inline const coccl::EventApi& fakeEvents() {
  static const coccl::EventApi a = {&fevCreate, &fevRecord, &fevQuery, &fevSync, &fevDestroy};
  return a;
}
inline void completeAllEvents() { for (FakeEvent* f : liveEvents()) f->done = true; }

// ------------------------------------------------------------------ fake VMM driver with a life-cycle log
struct VmmLog { std::vector<std::string> calls; size_t nextVa = 0x100000000ull; unsigned long long nextHandle = 1; bool supported = true; };
inline VmmLog& vmmLog() { static VmmLog l; return l; }
inline CUresult fGran(size_t* g, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) { *g = 2u << 20; vmmLog().calls.push_back("granularity"); return CUDA_SUCCESS; }
inline CUresult fReserve(CUdeviceptr* p, size_t size, size_t, CUdeviceptr, unsigned long long) { *p = vmmLog().nextVa; vmmLog().nextVa += size + (1ull << 30); vmmLog().calls.push_back("reserve:" + std::to_string(size)); return CUDA_SUCCESS; }
inline CUresult fAddrFree(CUdeviceptr, size_t size) { vmmLog().calls.push_back("addressFree:" + std::to_string(size)); return CUDA_SUCCESS; }
inline CUresult fCreate(CUmemGenericAllocationHandle* h, size_t size, const CUmemAllocationProp*, unsigned long long) { *h = vmmLog().nextHandle++; vmmLog().calls.push_back("create:" + std::to_string(size)); return CUDA_SUCCESS; }
inline CUresult fRelease(CUmemGenericAllocationHandle) { vmmLog().calls.push_back("release"); return CUDA_SUCCESS; }
inline CUresult fMap(CUdeviceptr, size_t size, size_t, CUmemGenericAllocationHandle h, unsigned long long) { vmmLog().calls.push_back("map:" + std::to_string(h) + ":" + std::to_string(size)); return CUDA_SUCCESS; }
inline CUresult fUnmap(CUdeviceptr, size_t size) { vmmLog().calls.push_back("unmap:" + std::to_string(size)); return CUDA_SUCCESS; }
inline CUresult fAccess(CUdeviceptr, size_t size, const CUmemAccessDesc*, size_t count) { vmmLog().calls.push_back("setAccess:" + std::to_string(size) + "x" + std::to_string(count)); return CUDA_SUCCESS; }
inline int fPeers(int device, int* out, int cap) { int n = 0; for (int d = 0; d < 4 && n < cap; ++d) out[n++] = (device + d) % 4; return n; }
inline bool fSupported(int) { return vmmLog().supported; }
inline const coccl::VmmDriverApi& fakeVmm() {
  static const coccl::VmmDriverApi a = {&fGran, &fReserve, &fAddrFree, &fCreate, &fRelease, &fMap, &fUnmap, &fAccess, &fPeers, &fSupported};
  return a;
}

}  // namespace fakes
