// Communicator view used by the host runtime, and the transport interface behind it.
//
// The router, planner and executor never talk to a collective library directly: native
// operations and the byte exchanges of the staged pipeline go through `Transport`, which is
// NCCL in production (runtime/nccl_transport.cc, resolved with dlopen), symmetric peer memory
// for the fused kernels, and an in-memory fake in the host tests. The reference reaches the same
// testability with link-seam fakes of ncclComm (tests/coccl-tests/src/coccl_runtime_test.cc:115-260).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "coccl/nccl_compat.h"

namespace coccl {

struct Comm;

struct P2POp {
  bool send;
  void* buffer;
  size_t bytes;
  int peer;
};

class Transport {
 public:
  virtual ~Transport() {}
  virtual ncclResult_t allGather(Comm* c, const void* send, void* recv, size_t sendCount, ncclDataType_t t, cudaStream_t s) = 0;
  virtual ncclResult_t reduceScatter(Comm* c, const void* send, void* recv, size_t recvCount, ncclDataType_t t, ncclRedOp_t op, cudaStream_t s) = 0;
  virtual ncclResult_t allReduce(Comm* c, const void* send, void* recv, size_t count, ncclDataType_t t, ncclRedOp_t op, cudaStream_t s) = 0;
  // every rank sends sendCount elements to every rank (native form: one grouped send/recv per peer,
  // src/collectives.cc:245-271)
  virtual ncclResult_t allToAll(Comm* c, const void* send, void* recv, size_t sendCount, ncclDataType_t t, cudaStream_t s) = 0;
  virtual ncclResult_t send(Comm* c, const void* buf, size_t count, ncclDataType_t t, int peer, cudaStream_t s) = 0;
  virtual ncclResult_t recv(Comm* c, void* buf, size_t count, ncclDataType_t t, int peer, cudaStream_t s) = 0;
  virtual ncclResult_t groupStart() = 0;
  virtual ncclResult_t groupEnd() = 0;
  // One grouped exchange of byte ranges (frame payloads, metadata).
  virtual ncclResult_t p2pBatch(Comm* c, const P2POp* ops, int n, cudaStream_t s) = 0;
  // ncclCommSplit equivalent: ranks with the same color form a child, ordered by key.
  virtual ncclResult_t split(Comm* parent, int color, int key, Comm** child) = 0;
  virtual void destroy(Comm* c) = 0;
  // Whether the ranks behind this transport are real GPUs of one machine whose memory can be mapped into one another
  // (the peer-memory data path of the staged pipeline asks; test doubles answer no).
  virtual bool peerMemoryCapable() const { return false; }
};

// First word of every communicator object of this library. A handle that reaches the public API without it is not
// ours: when this library's nccl* names sit in front of the native library's in the symbol search order (linked or
// preloaded in its place), the native library's own internal calls of public functions can land here with ITS handles.
constexpr uint64_t kCommMagic = 0x434f43434c423230ull;  // "COCCLB20"

struct Comm {
  uint64_t magic = kCommMagic;
  int rank = 0, nRanks = 1;
  int nNodes = 1, localRanks = 1, localRank = 0, node = 0;
  bool uniform = true;  // every node holds the same number of ranks
  int cudaDev = 0;
  Transport* transport = nullptr;
  void* native = nullptr;  // transport-private handle (ncclComm_t for the NCCL transport)
  uint64_t id = 0;
  // lazily created hierarchy (runtime/hierarchy.cc); children never own further children
  Comm* intra = nullptr;
  Comm* inter = nullptr;
  bool isChild = false;
  void* user = nullptr;  // per-comm runtime state (buffer pool, training registry entry)
};

}  // namespace coccl
