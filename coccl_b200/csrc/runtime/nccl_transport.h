// Transport over the system NCCL (see nccl_transport.cc).
#pragma once
#include "runtime/comm.h"

namespace coccl {

class NcclTransport : public Transport {
 public:
  static bool available();
  ncclResult_t uniqueId(ncclUniqueId* id);
  ncclResult_t initRank(Comm** out, int nRanks, ncclUniqueId id, int rank);
  const char* errorString(ncclResult_t r);
  bool peerMemoryCapable() const override { return true; }
  ncclResult_t asyncError(Comm* c, ncclResult_t* out);
  ncclResult_t foreignAsyncError(void* native, ncclResult_t* out);
  ncclResult_t foreignCount(void* native, int* out);
  ncclResult_t foreignUserRank(void* native, int* out);
  ncclResult_t abort(Comm* c);
  ncclResult_t broadcast(Comm* c, const void* s, void* r, size_t n, ncclDataType_t t, int root, cudaStream_t st);
  ncclResult_t reduce(Comm* c, const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, int root, cudaStream_t st);
  // pass-throughs of the rest of the NCCL surface (user-defined reductions, registration, allocation, version)
  ncclResult_t version(int* v);
  ncclResult_t memAlloc(void** p, size_t bytes);
  ncclResult_t memFree(void* p);
  ncclResult_t commRegister(Comm* c, void* buff, size_t size, void** handle);
  ncclResult_t commDeregister(Comm* c, void* handle);
  ncclResult_t redOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t t, int residence, Comm* c);
  ncclResult_t redOpDestroy(ncclRedOp_t op, Comm* c);

  ncclResult_t allGather(Comm* c, const void* send, void* recv, size_t sendCount, ncclDataType_t t, cudaStream_t s) override;
  ncclResult_t reduceScatter(Comm* c, const void* send, void* recv, size_t recvCount, ncclDataType_t t, ncclRedOp_t op, cudaStream_t s) override;
  ncclResult_t allReduce(Comm* c, const void* send, void* recv, size_t count, ncclDataType_t t, ncclRedOp_t op, cudaStream_t s) override;
  ncclResult_t allToAll(Comm* c, const void* send, void* recv, size_t sendCount, ncclDataType_t t, cudaStream_t s) override;
  ncclResult_t send(Comm* c, const void* buf, size_t count, ncclDataType_t t, int peer, cudaStream_t s) override;
  ncclResult_t recv(Comm* c, void* buf, size_t count, ncclDataType_t t, int peer, cudaStream_t s) override;
  ncclResult_t groupStart() override;
  ncclResult_t groupEnd() override;
  ncclResult_t p2pBatch(Comm* c, const P2POp* ops, int n, cudaStream_t s) override;
  ncclResult_t split(Comm* parent, int color, int key, Comm** child) override;
  void destroy(Comm* c) override;

 private:
  void fillTopology(Comm* c);
};

NcclTransport& ncclTransport();

}  // namespace coccl
