// libcoccl_nccl.so: the public API under its NCCL names, for linking or preloading in place of
// libnccl.so. Each function forwards to the cocclApi* implementation in libcoccl.so; the
// p-prefixed names are the profiling aliases NCCL exports (src/include/core.h:17-31).
#include "coccl/coccl.h"

#define COCCL_ALIAS2(ret, name, params, args)                  \
  extern "C" ret nccl##name params { return cocclApi##name args; } \
  extern "C" ret pnccl##name params { return cocclApi##name args; }

COCCL_ALIAS2(ncclResult_t, GetUniqueId, (ncclUniqueId * id), (id))
COCCL_ALIAS2(ncclResult_t, CommInitRank, (ncclComm_t * c, int n, ncclUniqueId id, int r), (c, n, id, r))
COCCL_ALIAS2(ncclResult_t, CommDestroy, (ncclComm_t c), (c))
COCCL_ALIAS2(ncclResult_t, CommFinalize, (ncclComm_t c), (c))
COCCL_ALIAS2(ncclResult_t, CommAbort, (ncclComm_t c), (c))
COCCL_ALIAS2(ncclResult_t, CommSplit, (ncclComm_t c, int color, int key, ncclComm_t* out, void* cfg), (c, color, key, out, cfg))
COCCL_ALIAS2(ncclResult_t, CommCount, (ncclComm_t c, int* n), (c, n))
COCCL_ALIAS2(ncclResult_t, CommUserRank, (ncclComm_t c, int* r), (c, r))
COCCL_ALIAS2(ncclResult_t, CommCuDevice, (ncclComm_t c, int* d), (c, d))
COCCL_ALIAS2(ncclResult_t, CommGetAsyncError, (ncclComm_t c, ncclResult_t* e), (c, e))
COCCL_ALIAS2(const char*, GetErrorString, (ncclResult_t r), (r))
COCCL_ALIAS2(const char*, GetLastError, (ncclComm_t c), (c))
COCCL_ALIAS2(ncclResult_t, AllReduce, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st), (s, r, n, t, op, c, st))
COCCL_ALIAS2(ncclResult_t, ReduceScatter, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st), (s, r, n, t, op, c, st))
COCCL_ALIAS2(ncclResult_t, AllGather, (const void* s, void* r, size_t n, ncclDataType_t t, ncclComm_t c, cudaStream_t st), (s, r, n, t, c, st))
COCCL_ALIAS2(ncclResult_t, AllToAll, (const void* s, void* r, size_t n, ncclDataType_t t, ncclComm_t c, cudaStream_t st), (s, r, n, t, c, st))
COCCL_ALIAS2(ncclResult_t, Send, (const void* s, size_t n, ncclDataType_t t, int p, ncclComm_t c, cudaStream_t st), (s, n, t, p, c, st))
COCCL_ALIAS2(ncclResult_t, Recv, (void* r, size_t n, ncclDataType_t t, int p, ncclComm_t c, cudaStream_t st), (r, n, t, p, c, st))
COCCL_ALIAS2(ncclResult_t, Broadcast, (const void* s, void* r, size_t n, ncclDataType_t t, int root, ncclComm_t c, cudaStream_t st), (s, r, n, t, root, c, st))
COCCL_ALIAS2(ncclResult_t, Reduce, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, int root, ncclComm_t c, cudaStream_t st), (s, r, n, t, op, root, c, st))
COCCL_ALIAS2(ncclResult_t, GetVersion, (int* v), (v))
COCCL_ALIAS2(ncclResult_t, CommInitAll, (ncclComm_t * c, int n, const int* devs), (c, n, devs))
COCCL_ALIAS2(ncclResult_t, CommInitRankConfig, (ncclComm_t * c, int n, ncclUniqueId id, int r, void* cfg), (c, n, id, r, cfg))
COCCL_ALIAS2(ncclResult_t, MemAlloc, (void** p, size_t n), (p, n))
COCCL_ALIAS2(ncclResult_t, MemFree, (void* p), (p))
COCCL_ALIAS2(ncclResult_t, CommRegister, (ncclComm_t c, void* b, size_t n, void** h), (c, b, n, h))
COCCL_ALIAS2(ncclResult_t, CommDeregister, (ncclComm_t c, void* h), (c, h))
COCCL_ALIAS2(ncclResult_t, RedOpCreatePreMulSum, (ncclRedOp_t * op, void* scalar, ncclDataType_t t, int residence, ncclComm_t c), (op, scalar, t, residence, c))
COCCL_ALIAS2(ncclResult_t, RedOpDestroy, (ncclRedOp_t op, ncclComm_t c), (op, c))
COCCL_ALIAS2(ncclResult_t, Bcast, (void* b, size_t n, ncclDataType_t t, int root, ncclComm_t c, cudaStream_t st), (b, n, t, root, c, st))
COCCL_ALIAS2(ncclResult_t, GroupStart, (void), ())
COCCL_ALIAS2(ncclResult_t, GroupEnd, (void), ())

// profiling aliases of the explicit compressed calls
#define COCCL_PALIAS(name, params, args) extern "C" ncclResult_t p##name params { return name args; }
COCCL_PALIAS(cocclAllReduceCompOneShot, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st), (s, r, n, t, op, c, st))
COCCL_PALIAS(cocclAllReduceCompTwoShot, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st), (s, r, n, t, op, c, st))
COCCL_PALIAS(cocclAllReduceCompTripleShot, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st), (s, r, n, t, op, c, st))
COCCL_PALIAS(cocclReduceScatterCompOneShot, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st), (s, r, n, t, op, c, st))
COCCL_PALIAS(cocclReduceScatterCompTwoShot, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st), (s, r, n, t, op, c, st))
COCCL_PALIAS(cocclAllGatherComp, (const void* s, void* r, size_t n, ncclDataType_t t, ncclComm_t c, cudaStream_t st), (s, r, n, t, c, st))
COCCL_PALIAS(cocclAllToAllComp, (const void* s, void* r, size_t n, ncclDataType_t t, ncclComm_t c, cudaStream_t st), (s, r, n, t, c, st))
COCCL_PALIAS(cocclSendComp, (const void* s, size_t n, ncclDataType_t t, int p, ncclComm_t c, cudaStream_t st), (s, n, t, p, c, st))
COCCL_PALIAS(cocclRecvDecomp, (void* r, size_t n, ncclDataType_t t, int p, ncclComm_t c, cudaStream_t st), (r, n, t, p, c, st))
