// Native transport: the system NCCL, resolved with dlopen so that libcoccl.so neither links
// against it nor interposes it. Library lookup order: $COCCL_NCCL_LIBRARY, libnccl.so.2, libnccl.so.
// Used for every call the router leaves native, for pipeline-parallel send/recv, and for the byte
// exchanges of the staged pipeline.
#include <dlfcn.h>
#include <stdlib.h>
#include <mutex>

#include "runtime/log.h"
#include "runtime/nccl_transport.h"

#include <atomic>

namespace coccl {
namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(void**, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(void*) = nullptr;
  ncclResult_t (*CommAbort)(void*) = nullptr;
  ncclResult_t (*CommSplit)(void*, int, int, void**, void*) = nullptr;
  ncclResult_t (*CommGetAsyncError)(void*, ncclResult_t*) = nullptr;
  ncclResult_t (*CommCount)(void*, int*) = nullptr;
  ncclResult_t (*CommUserRank)(void*, int*) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, void*, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, void*, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, void*, cudaStream_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, void*, cudaStream_t) = nullptr;
  ncclResult_t (*Reduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, int, void*, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, void*, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, void*, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  // optional entry points (forwarded when the library has them)
  ncclResult_t (*GetVersion)(int*) = nullptr;
  ncclResult_t (*MemAlloc)(void**, size_t) = nullptr;
  ncclResult_t (*MemFree)(void*) = nullptr;
  ncclResult_t (*CommRegister)(void*, void*, size_t, void**) = nullptr;
  ncclResult_t (*CommDeregister)(void*, void*) = nullptr;
  ncclResult_t (*RedOpCreatePreMulSum)(ncclRedOp_t*, void*, ncclDataType_t, int, void*) = nullptr;
  ncclResult_t (*RedOpDestroy)(ncclRedOp_t, void*) = nullptr;
  bool ok = false;
};

NcclApi& api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {getenv("COCCL_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      if (n == nullptr || *n == '\0') continue;
      // DEEPBIND: the native library resolves its internal references to public nccl* functions to ITSELF, also when
      // a library that exports the same names (libcoccl_nccl.so) comes first in the global search order
      a.handle = dlopen(n, RTLD_NOW | RTLD_LOCAL | RTLD_DEEPBIND);
      if (a.handle) break;
    }
    if (!a.handle) {
      COCCL_WARN("native transport: no NCCL library found (set COCCL_NCCL_LIBRARY)");
      return;
    }
#define LOAD(name) a.name = reinterpret_cast<decltype(a.name)>(dlsym(a.handle, "nccl" #name))
    LOAD(GetUniqueId); LOAD(CommInitRank); LOAD(CommDestroy); LOAD(CommAbort); LOAD(CommSplit); LOAD(CommGetAsyncError); LOAD(CommCount); LOAD(CommUserRank);
    LOAD(AllReduce); LOAD(ReduceScatter); LOAD(AllGather); LOAD(Broadcast); LOAD(Reduce); LOAD(Send); LOAD(Recv);
    LOAD(GroupStart); LOAD(GroupEnd); LOAD(GetErrorString);
    LOAD(GetVersion); LOAD(MemAlloc); LOAD(MemFree); LOAD(CommRegister); LOAD(CommDeregister);
    LOAD(RedOpCreatePreMulSum); LOAD(RedOpDestroy);
#undef LOAD
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.ReduceScatter && a.AllGather && a.Send &&
           a.Recv && a.GroupStart && a.GroupEnd;
  });
  return a;
}

uint64_t nextCommId() {
  static std::atomic<uint64_t> next{1};
  return next.fetch_add(1);
}

int envInt(const char* name, int fallback) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : fallback;
}

}  // namespace

bool NcclTransport::available() { return api().ok; }

ncclResult_t NcclTransport::uniqueId(ncclUniqueId* id) { return api().ok ? api().GetUniqueId(id) : ncclSystemError; }

const char* NcclTransport::errorString(ncclResult_t r) {
  return (api().ok && api().GetErrorString) ? api().GetErrorString(r) : "NCCL library not loaded";
}

void NcclTransport::fillTopology(Comm* c) {
  // One process per GPU; ranks are laid out node-major. LOCAL_WORLD_SIZE (torchrun) or
  // COCCL_LOCAL_RANKS tells how many ranks share a node; default: all of them.
  int local = envInt("COCCL_LOCAL_RANKS", envInt("LOCAL_WORLD_SIZE", c->nRanks));
  if (local <= 0 || local > c->nRanks || c->nRanks % local != 0) local = c->nRanks;
  c->localRanks = local;
  c->nNodes = c->nRanks / local;
  c->node = c->rank / local;
  c->localRank = c->rank % local;
  c->uniform = true;
}

ncclResult_t NcclTransport::initRank(Comm** out, int nRanks, ncclUniqueId id, int rank) {
  if (!api().ok) return ncclSystemError;
  // Inside a group the native library keeps the address it is given and writes the handle again when the group ends:
  // the slot must outlive this function, so it is the communicator object's own field.
  Comm* c = new Comm();
  ncclResult_t r = api().CommInitRank(&c->native, nRanks, id, rank);
  if (r != ncclSuccess) { delete c; return r; }
  c->rank = rank;
  c->nRanks = nRanks;
  cudaGetDevice(&c->cudaDev);
  c->transport = this;
  c->id = nextCommId();
  fillTopology(c);
  *out = c;
  return ncclSuccess;
}

ncclResult_t NcclTransport::allGather(Comm* c, const void* s, void* r, size_t n, ncclDataType_t t, cudaStream_t st) {
  return api().AllGather(s, r, n, t, c->native, st);
}
ncclResult_t NcclTransport::reduceScatter(Comm* c, const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, cudaStream_t st) {
  return api().ReduceScatter(s, r, n, t, op, c->native, st);
}
ncclResult_t NcclTransport::allReduce(Comm* c, const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, cudaStream_t st) {
  return api().AllReduce(s, r, n, t, op, c->native, st);
}
ncclResult_t NcclTransport::allToAll(Comm* c, const void* s, void* r, size_t n, ncclDataType_t t, cudaStream_t st) {
  const size_t bytes = n * cocclTypeSize(t);
  ncclResult_t res = api().GroupStart();
  for (int p = 0; p < c->nRanks && res == ncclSuccess; ++p) {
    res = api().Recv(static_cast<char*>(r) + (size_t)p * bytes, n, t, p, c->native, st);
    if (res == ncclSuccess) res = api().Send(static_cast<const char*>(s) + (size_t)p * bytes, n, t, p, c->native, st);
  }
  ncclResult_t e = api().GroupEnd();
  return res != ncclSuccess ? res : e;
}
ncclResult_t NcclTransport::send(Comm* c, const void* b, size_t n, ncclDataType_t t, int peer, cudaStream_t st) {
  return api().Send(b, n, t, peer, c->native, st);
}
ncclResult_t NcclTransport::recv(Comm* c, void* b, size_t n, ncclDataType_t t, int peer, cudaStream_t st) {
  return api().Recv(b, n, t, peer, c->native, st);
}
ncclResult_t NcclTransport::broadcast(Comm* c, const void* s, void* r, size_t n, ncclDataType_t t, int root, cudaStream_t st) {
  return api().Broadcast ? api().Broadcast(s, r, n, t, root, c->native, st) : ncclInternalError;
}
ncclResult_t NcclTransport::reduce(Comm* c, const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, int root, cudaStream_t st) {
  return api().Reduce ? api().Reduce(s, r, n, t, op, root, c->native, st) : ncclInternalError;
}
ncclResult_t NcclTransport::groupStart() { return api().GroupStart(); }
ncclResult_t NcclTransport::groupEnd() { return api().GroupEnd(); }

ncclResult_t NcclTransport::p2pBatch(Comm* c, const P2POp* ops, int n, cudaStream_t st) {
  ncclResult_t res = api().GroupStart();
  for (int i = 0; i < n && res == ncclSuccess; ++i) {
    if (ops[i].bytes == 0) continue;
    res = ops[i].send ? api().Send(ops[i].buffer, ops[i].bytes, ncclUint8, ops[i].peer, c->native, st)
                      : api().Recv(ops[i].buffer, ops[i].bytes, ncclUint8, ops[i].peer, c->native, st);
  }
  ncclResult_t e = api().GroupEnd();
  return res != ncclSuccess ? res : e;
}

ncclResult_t NcclTransport::split(Comm* parent, int color, int key, Comm** child) {
  if (!api().CommSplit) return ncclInternalError;
  Comm* c = new Comm();   // the handle slot must outlive a surrounding group (see initRank)
  ncclResult_t r = api().CommSplit(parent->native, color, key, &c->native, nullptr);
  if (r != ncclSuccess) { delete c; return r; }
  c->transport = this;
  void* native = c->native;
  c->cudaDev = parent->cudaDev;
  c->id = nextCommId();  // two splits with the same colour are two communicators: ids never repeat in a process
  int count = 1, rank = 0;
  if (api().CommCount) api().CommCount(native, &count);
  if (api().CommUserRank) api().CommUserRank(native, &rank);
  c->nRanks = count;
  c->rank = rank;
  // topology of the child is set by the caller (Runtime::hierarchy knows which split this is);
  // default: treat it as one node
  c->nNodes = 1; c->localRanks = count; c->localRank = rank; c->node = 0;
  *child = c;
  return ncclSuccess;
}

// Queries on a handle of the native library itself (see kCommMagic in runtime/comm.h).
ncclResult_t NcclTransport::foreignAsyncError(void* native, ncclResult_t* out) {
  return (api().ok && api().CommGetAsyncError) ? api().CommGetAsyncError(native, out) : ncclInvalidArgument;
}
ncclResult_t NcclTransport::foreignCount(void* native, int* out) {
  return (api().ok && api().CommCount) ? api().CommCount(native, out) : ncclInvalidArgument;
}
ncclResult_t NcclTransport::foreignUserRank(void* native, int* out) {
  return (api().ok && api().CommUserRank) ? api().CommUserRank(native, out) : ncclInvalidArgument;
}

void NcclTransport::destroy(Comm* c) {
  if (c == nullptr) return;
  if (c->native && api().ok) api().CommDestroy(c->native);
  delete c;
}

ncclResult_t NcclTransport::asyncError(Comm* c, ncclResult_t* out) {
  if (api().CommGetAsyncError) return api().CommGetAsyncError(c->native, out);
  *out = ncclSuccess;
  return ncclSuccess;
}

ncclResult_t NcclTransport::abort(Comm* c) {
  ncclResult_t r = (api().CommAbort && c->native) ? api().CommAbort(c->native) : ncclSuccess;
  c->native = nullptr;
  delete c;
  return r;
}

ncclResult_t NcclTransport::version(int* v) {
  if (v == nullptr) return ncclInvalidArgument;
  if (api().ok && api().GetVersion) return api().GetVersion(v);
  *v = 22105;  // the API level this library implements (NCCL 2.21.5, the reference's base)
  return ncclSuccess;
}
ncclResult_t NcclTransport::memAlloc(void** p, size_t bytes) {
  if (p == nullptr) return ncclInvalidArgument;
  if (api().ok && api().MemAlloc) return api().MemAlloc(p, bytes);
  return cudaMalloc(p, bytes) == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}
ncclResult_t NcclTransport::memFree(void* p) {
  if (api().ok && api().MemFree) return api().MemFree(p);
  return cudaFree(p) == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}
ncclResult_t NcclTransport::commRegister(Comm* c, void* buff, size_t size, void** handle) {
  if (api().ok && api().CommRegister && c->native) return api().CommRegister(c->native, buff, size, handle);
  if (handle) *handle = nullptr;  // registration is an optimisation hint: without it calls still work
  return ncclSuccess;
}
ncclResult_t NcclTransport::commDeregister(Comm* c, void* handle) {
  if (api().ok && api().CommDeregister && c->native) return api().CommDeregister(c->native, handle);
  return ncclSuccess;
}
ncclResult_t NcclTransport::redOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t t, int residence, Comm* c) {
  if (api().ok && api().RedOpCreatePreMulSum && c->native) return api().RedOpCreatePreMulSum(op, scalar, t, residence, c->native);
  return ncclInvalidUsage;
}
ncclResult_t NcclTransport::redOpDestroy(ncclRedOp_t op, Comm* c) {
  if (api().ok && api().RedOpDestroy && c->native) return api().RedOpDestroy(op, c->native);
  return ncclInvalidUsage;
}

NcclTransport& ncclTransport() {
  static NcclTransport* t = new NcclTransport();
  return *t;
}

}  // namespace coccl
