// Fused fast path of the executor: one persistent kernel per collective over peer-mapped
// symmetric memory (kernels/collective_kernels.cuh) instead of the staged pipeline.
// Taken when the communicator sits on one node with at most 8 ranks, the codec exports
// cocclFusedCodecQuery and accepts the datatype, and the algorithm is flat.
#include <map>
#include <mutex>
#include <string.h>

#include "kernels/kernels_api.h"
#include "runtime/log.h"
#include "runtime/primitives.h"
#include "symm/symm.h"

namespace coccl {
namespace {

struct SymmRegion {
  cocclSymmBuffer* buf = nullptr;
  void* ptrs[COCCLK_MAX_RANKS] = {};
  size_t bytes = 0;
};

struct FusedState {
  SymmRegion signals;   // flags + status word
  SymmRegion workspace; // two parity halves
  size_t half = 0;
  unsigned epoch = 0;
  bool broken = false;
};

std::mutex gMutex;
std::map<Comm*, FusedState> gStates;

// Allocate a symmetric buffer and map every peer's; handles travel through the comm's own all-gather.
ncclResult_t openRegion(Comm* comm, size_t bytes, cudaStream_t s, SymmRegion* r) {
  if (cocclSymmAlloc(bytes, &r->buf) != 0) return ncclUnhandledCudaError;
  r->bytes = bytes;
  char mine[COCCL_SYMM_HANDLE_BYTES];
  if (cocclSymmExport(r->buf, mine) != 0) return ncclUnhandledCudaError;
  void* dMine = nullptr;
  void* dAll = nullptr;
  const size_t n = (size_t)comm->nRanks;
  ncclResult_t res = ncclSuccess;
  std::vector<char> all(n * COCCL_SYMM_HANDLE_BYTES);
  if (cudaMalloc(&dMine, COCCL_SYMM_HANDLE_BYTES) != cudaSuccess || cudaMalloc(&dAll, all.size()) != cudaSuccess) res = ncclUnhandledCudaError;
  if (res == ncclSuccess && cudaMemcpyAsync(dMine, mine, sizeof(mine), cudaMemcpyHostToDevice, s) != cudaSuccess) res = ncclUnhandledCudaError;
  if (res == ncclSuccess) res = comm->transport->allGather(comm, dMine, dAll, COCCL_SYMM_HANDLE_BYTES, ncclUint8, s);
  if (res == ncclSuccess && cudaMemcpyAsync(all.data(), dAll, all.size(), cudaMemcpyDeviceToHost, s) != cudaSuccess) res = ncclUnhandledCudaError;
  if (res == ncclSuccess && cudaStreamSynchronize(s) != cudaSuccess) res = ncclUnhandledCudaError;
  if (dMine) cudaFree(dMine);
  if (dAll) cudaFree(dAll);
  if (res != ncclSuccess) return res;
  for (int p = 0; p < comm->nRanks; ++p) {
    if (p == comm->rank) { r->ptrs[p] = cocclSymmLocalPtr(r->buf); continue; }
    if (cocclSymmImport(r->buf, p, all.data() + (size_t)p * COCCL_SYMM_HANDLE_BYTES, &r->ptrs[p]) != 0) return ncclUnhandledCudaError;
  }
  return ncclSuccess;
}

void closeRegion(SymmRegion* r) {
  if (r->buf) cocclSymmFree(r->buf);
  *r = SymmRegion();
}

int kernelDtype(ncclDataType_t t) { return t == ncclFloat32 ? 0 : t == ncclFloat16 ? 1 : t == ncclBfloat16 ? 2 : -1; }

}  // namespace

void FusedExecutor::releaseComm(Comm* comm) {
  std::lock_guard<std::mutex> lock(gMutex);
  auto it = gStates.find(comm);
  if (it == gStates.end()) return;
  cudaDeviceSynchronize();
  closeRegion(&it->second.workspace);
  closeRegion(&it->second.signals);
  gStates.erase(it);
}

ncclResult_t FusedExecutor::execute(Runtime* rt, const PreparedCall& call) {
  const CallInfo& info = call.info;
  Comm* comm = info.comm;
  CompressorPolicy* codec = flatCodec(call);
  int op = -1;
  switch (info.op) {
    case Operation::ReduceScatter: if (call.algorithm == Algorithm::RsOneShot) op = 0; break;
    case Operation::AllGather: op = 1; break;
    case Operation::AllToAll: op = 2; break;
    case Operation::AllReduce:
      if (call.algorithm == Algorithm::ArOneShot) op = 3;
      if (call.algorithm == Algorithm::ArTwoShot) op = 4;
      break;
    default: break;
  }
  cocclkCodec kc;
  const bool fusable = op >= 0 && codec != nullptr && comm->nNodes == 1 && comm->nRanks <= COCCLK_MAX_RANKS &&
                       kernelDtype(info.datatype) >= 0 && codec->plugin()->fusedQuery != nullptr &&
                       codec->plugin()->fusedQuery(codec->config(), (int)info.datatype, &kc) == 1 && cocclkTileCodecSupported(&kc);
  if (!fusable) { ++stagedCalls; return StagedExecutor::execute(rt, call); }

  std::lock_guard<std::mutex> lock(gMutex);
  FusedState& st = gStates[comm];
  if (st.broken) { ++stagedCalls; return StagedExecutor::execute(rt, call); }
  const int n = comm->nRanks;
  const long count = (op == 0 || op == 1 || op == 2) ? (long)info.count : (op == 4 ? (long)(info.count / (size_t)n) : (long)info.count);
  const long slot = cocclkSlotBytes(&kc, count);
  const long region = (slot * n + 255) / 256 * 256;
  const size_t need = (size_t)region * (op == 4 ? 2 : 1);
  if (st.signals.buf == nullptr) {
    if (openRegion(comm, (size_t)cocclkFlagBytes() + 256, info.stream, &st.signals) != ncclSuccess) {
      COCCL_WARN("fused path: cannot map peer signal memory on comm %llu; using the staged pipeline", (unsigned long long)comm->id);
      st.broken = true;
      closeRegion(&st.signals);
      ++stagedCalls;
      return StagedExecutor::execute(rt, call);
    }
  }
  if (st.half < need) {
    // every rank reaches this with the same sizes at the same call; drain before remapping
    cudaStreamSynchronize(info.stream);
    closeRegion(&st.workspace);
    const size_t half = (need + (1u << 20) - 1) / (1u << 20) * (1u << 20);
    if (openRegion(comm, 2 * half, info.stream, &st.workspace) != ncclSuccess) {
      st.broken = true;
      closeRegion(&st.workspace);
      ++stagedCalls;
      return StagedExecutor::execute(rt, call);
    }
    st.half = half;
    COCCL_INFO(kLogMemory, "fused path: comm %llu workspace 2 x %zu B mapped on %d peers", (unsigned long long)comm->id, half, n);
  }
  ++st.epoch;
  cocclkCollArgs a;
  memset(&a, 0, sizeof(a));
  a.op = op;
  a.nRanks = n;
  a.rankBase = comm->rank;
  a.dtype = kernelDtype(info.datatype);
  a.count = count;
  const long tileElems = cocclkTileElems();
  long tiles = (count + tileElems - 1) / tileElems;
  long sliceTiles = tiles * n / (148 * 3);
  if (sliceTiles < 1) sliceTiles = 1;
  if (sliceTiles > 16) sliceTiles = 16;
  while ((tiles + sliceTiles - 1) / sliceTiles > COCCLK_MAX_SLICES) sliceTiles *= 2;
  a.sliceTiles = (int)sliceTiles;
  a.epoch = st.epoch & 0x7fffffffu;
  a.timeoutNs = 20ull * 1000000000ull;
  a.codec = kc;
  a.slotBytes = slot;
  a.regionBOffset = region;
  a.in[comm->rank] = info.sendbuff;
  a.out[comm->rank] = info.recvbuff;
  for (int p = 0; p < n; ++p) {
    a.ws[p] = static_cast<uint8_t*>(st.workspace.ptrs[p]) + (size_t)(st.epoch & 1u) * st.half;
    a.flags[p] = static_cast<unsigned int*>(st.signals.ptrs[p]);
    a.status[p] = static_cast<char*>(st.signals.ptrs[p]) + cocclkFlagBytes();
  }
  const int rc = cocclkFusedCollective(&a, 1, 0, info.stream);
  if (rc != 0) return rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError;
  ++fusedCalls;
  return ncclSuccess;
}

}  // namespace coccl
