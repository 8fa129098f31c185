// Public C API: the NCCL-compatible collective calls routed through the compression-aware
// runtime, plus the explicit compressed calls.
//
// libcoccl.so exports every function under a `cocclApi` prefix (cocclApiAllReduce, ...), so that it
// can live in a process that also holds the real NCCL. libcoccl_nccl.so is a thin shim that exports
// the same functions under their NCCL names (ncclAllReduce, ..., and the p-prefixed profiling aliases),
// for linking or preloading in place of libnccl.so. API surface: src/nccl.h.in:84-486 of the reference
// (NCCL 2.21.5 calls + ncclAllToAll :437 + the nine coccl*Comp* calls :326-442).
//
// Environment: COCCL_ENABLE=0|1, COCCL_CONFIG_FILE=<policy.toml>; COCCL_DEBUG / COCCL_DEBUG_SUBSYS.
#pragma once
#include "coccl/nccl_compat.h"

#ifdef __cplusplus
extern "C" {
#endif

ncclResult_t cocclApiGetUniqueId(ncclUniqueId* id);
ncclResult_t cocclApiCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank);
ncclResult_t cocclApiCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, void* config);
ncclResult_t cocclApiCommInitAll(ncclComm_t* comms, int ndev, const int* devlist);
ncclResult_t cocclApiGetVersion(int* version);
ncclResult_t cocclApiMemAlloc(void** ptr, size_t size);
ncclResult_t cocclApiMemFree(void* ptr);
ncclResult_t cocclApiCommRegister(ncclComm_t comm, void* buff, size_t size, void** handle);
ncclResult_t cocclApiCommDeregister(ncclComm_t comm, void* handle);
ncclResult_t cocclApiRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t datatype, int residence, ncclComm_t comm);
ncclResult_t cocclApiRedOpDestroy(ncclRedOp_t op, ncclComm_t comm);
ncclResult_t cocclApiBcast(void* buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclApiCommDestroy(ncclComm_t comm);
ncclResult_t cocclApiCommFinalize(ncclComm_t comm);
ncclResult_t cocclApiCommAbort(ncclComm_t comm);
ncclResult_t cocclApiCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, void* config);
ncclResult_t cocclApiCommCount(ncclComm_t comm, int* count);
ncclResult_t cocclApiCommUserRank(ncclComm_t comm, int* rank);
ncclResult_t cocclApiCommCuDevice(ncclComm_t comm, int* device);
// Also reports a bounded wait of a fused kernel that ran out (ncclRemoteError).
ncclResult_t cocclApiCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError);
const char* cocclApiGetErrorString(ncclResult_t result);
const char* cocclApiGetLastError(ncclComm_t comm);

ncclResult_t cocclApiAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclApiReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclApiAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclApiAllToAll(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclApiSend(const void* sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclApiRecv(void* recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclApiBroadcast(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclApiReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclApiGroupStart(void);
ncclResult_t cocclApiGroupEnd(void);

// Explicit compressed calls: bypass the size threshold, still need an enabled runtime and a policy for
// the operation; an unsupported datatype runs natively and succeeds; no codec at the scopes the
// algorithm uses is ncclInvalidUsage.
ncclResult_t cocclAllReduceCompOneShot(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclAllReduceCompTwoShot(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclAllReduceCompTripleShot(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclReduceScatterCompOneShot(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclReduceScatterCompTwoShot(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclAllGatherComp(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclAllToAllComp(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclSendComp(const void* sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream);
ncclResult_t cocclRecvDecomp(void* recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream);

// Router statistics of the process (native / compressed / deferred calls, fused vs staged).
typedef struct cocclApiStats {
  unsigned long long nativeCalls, compressedCalls, deferredCalls, policyLookups, fusedCalls, stagedCalls;
} cocclApiStats;
void cocclApiGetStats(cocclApiStats* out);
// How many exchanges of encoded bytes of the staged pipeline (codecs without a fused kernel form: rANS, ZFP at rates
// without one, third-party plugins) this process served by its own peer-memory kernel instead of a library collective.
// Why compressed calls of this process ran through the staged pipeline instead of one fused kernel: the call has no
// fused form (codec without a tile codec, datatype, hierarchical algorithm, more than one node); an earlier set-up of
// the communicator had failed; this call's own set-up (mapping the peers' memory) failed.
void cocclApiStagedReasons(unsigned long long* noFusedForm, unsigned long long* afterFailedSetup, unsigned long long* setupFailed);
unsigned long long cocclApiPeerExchangeCalls(void);
// Algorithm selection from measured times ([autotune] enabled = true): at the first all-reduce of a size bucket
// (64 KiB - 256 MiB) that a fused kernel can serve, the one-shot and the two-shot kernel are timed on the call's own
// input and stream (output to scratch memory, maximum over the ranks), and calls of that bucket, or of the nearest
// measured one, take the faster. bucketsTimed: how many buckets this process timed; bucketsInTable: how many hold
// at least one time. COCCL_AUTOTUNE_MEASURE=0 turns the timing off (the cost model and heuristics decide).
void cocclApiMeasuredSelection(unsigned long long* bucketsTimed, unsigned long long* bucketsInTable);

// Training mode: what the classifier decided for this communicator. `committed` is 0 until a decision exists (all
// other fields are then zero); `active` turns 1 at the call from which every rank routes by the role. Roles:
// 0 normal, 1 data, 2 tensor, 3 pipeline parallel, 4 unknown (stays native). Outside training mode the call
// returns ncclInvalidUsage.
typedef struct cocclApiTrainingRole {
  int role, candidate, committed, active;
  double confidence, callsPerIteration, agToRsRatio;
  unsigned long long observedCalls, activationCall;
} cocclApiTrainingRole;
ncclResult_t cocclApiCommTrainingRole(ncclComm_t comm, cocclApiTrainingRole* out);

#ifdef __cplusplus
}
#endif
