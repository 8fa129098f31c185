// Fused fast path of the executor: one persistent kernel per collective over peer-mapped
// symmetric memory (kernels/collective_kernels.cuh) instead of the staged pipeline.
// Taken when the communicator sits on one node with at most 8 ranks, the codec exports
// cocclFusedCodecQuery and accepts the datatype, and the algorithm is flat.
#include <map>
#include <mutex>
#include <string.h>
#include <vector>

#include "kernels/kernels_api.h"
#include "runtime/log.h"
#include "runtime/primitives.h"
#include "runtime/symm_workspace.h"
#include "runtime/transport_exchange.h"

namespace coccl {
namespace {

struct FusedState {
  SymmRegion signals;    // flags + status word
  SymmRegion workspace;  // two parity halves
  size_t half = 0;
  unsigned epoch = 0;
  bool broken = false;   // agreed by all ranks: the staged pipeline serves this communicator
  unsigned int* hostStatus = nullptr;  // pinned copy of the status word, refreshed after every fused launch
  std::mutex mutex;  // one call at a time per communicator; different communicators (threads of one process) run in parallel
};

std::mutex gMutex;
std::map<Comm*, FusedState> gStates;

int kernelDtype(ncclDataType_t t) { return t == ncclFloat32 ? 0 : t == ncclFloat16 ? 1 : t == ncclBfloat16 ? 2 : -1; }

}  // namespace

void FusedExecutor::releaseComm(Comm* comm) {
  std::lock_guard<std::mutex> lock(gMutex);
  auto it = gStates.find(comm);
  if (it == gStates.end()) return;
  cudaDeviceSynchronize();
  // teardown may run after a peer has gone: unmap and free locally, without a rendezvous
  it->second.workspace.closeLocal(cudaSymmApi());
  it->second.signals.closeLocal(cudaSymmApi());
  if (it->second.hostStatus) cudaFreeHost(it->second.hostStatus);
  gStates.erase(it);
}

// Kernel operation of a prepared call (-1: none) and, when a fused kernel can serve it, the codec's tile form.
static int fusedOperation(const PreparedCall& call, Algorithm algorithm, cocclkCodec* kc) {
  const CallInfo& info = call.info;
  Comm* comm = info.comm;
  CompressorPolicy* codec = flatCodec(call);
  int op = -1;
  switch (info.op) {
    case Operation::ReduceScatter: if (algorithm == Algorithm::RsOneShot) op = 0; break;
    case Operation::AllGather: op = 1; break;
    case Operation::AllToAll: op = 2; break;
    case Operation::AllReduce:
      if (algorithm == Algorithm::ArOneShot) op = 3;
      if (algorithm == Algorithm::ArTwoShot) op = 4;
      break;
    default: break;
  }
  const bool fusable = op >= 0 && codec != nullptr && comm->nNodes == 1 && comm->nRanks <= COCCLK_MAX_RANKS &&
                       kernelDtype(info.datatype) >= 0 && codec->plugin()->fusedQuery != nullptr &&
                       codec->plugin()->fusedQuery(codec->config(), (int)info.datatype, kc) == 1 && cocclkTileCodecSupported(kc);
  return fusable ? op : -1;
}

bool FusedExecutor::serves(const PreparedCall& call, Algorithm algorithm) {
  cocclkCodec kc;
  return fusedOperation(call, algorithm, &kc) >= 0;
}

ncclResult_t FusedExecutor::execute(Runtime* rt, const PreparedCall& call) {
  const CallInfo& info = call.info;
  Comm* comm = info.comm;
  cocclkCodec kc;
  const int op = fusedOperation(call, call.algorithm, &kc);
  const bool fusable = op >= 0;
  if (!fusable) { ++stagedCalls; ++stagedNoFusedForm; return StagedExecutor::execute(rt, call); }

  FusedState* stp;
  {
    std::lock_guard<std::mutex> lock(gMutex);  // guards the table only: map nodes never move
    stp = &gStates[comm];
  }
  FusedState& st = *stp;
  // The set-up below blocks on the other ranks (host-level exchange). Ranks that live in one process as threads must
  // therefore not share a lock across it: each communicator has its own.
  std::unique_lock<std::mutex> lock(st.mutex);
  if (st.broken) { lock.unlock(); ++stagedCalls; ++stagedAfterFailedSetup; return StagedExecutor::execute(rt, call); }
  const int n = comm->nRanks;
  const long count = (op == 0 || op == 1 || op == 2) ? (long)info.count : (op == 4 ? (long)(info.count / (size_t)n) : (long)info.count);
  const long slot = cocclkSlotBytes(&kc, count);
  const long region = (slot * n + 255) / 256 * 256;
  const size_t need = (size_t)region * (op == 4 ? 2 : 1);
  // Opening and growing the peer-mapped regions is collective and its outcome is agreed by all ranks
  // (runtime/symm_workspace.h). The decision to grow depends only on the call's sizes, which the collective's
  // contract makes equal on every rank, so all ranks enter the protocol at the same call.
  if (!st.signals.open() || st.half < need) {
    cudaStreamSynchronize(info.stream);  // no kernel of this rank still uses the old mapping
    TransportExchange x(comm, info.stream);
    const SymmApi& api = cudaSymmApi();
    bool ok = true;
    if (!st.signals.open()) {
      ok = st.signals.reopen(api, x, (size_t)cocclkFlagBytes() + 256);
      if (ok && st.hostStatus == nullptr && cudaHostAlloc((void**)&st.hostStatus, 64, cudaHostAllocDefault) == cudaSuccess) *st.hostStatus = 0;
    }
    if (ok && st.half < need) {
      const size_t half = (need + (1u << 20) - 1) / (1u << 20) * (1u << 20);
      ok = st.workspace.reopen(api, x, 2 * half);
      st.half = ok ? st.workspace.bytes() / 2 : 0;
      if (ok) COCCL_INFO(kLogMemory, "fused path: comm %llu workspace 2 x %zu B mapped on %d peers", (unsigned long long)comm->id, st.half, n);
    }
    if (!ok) {
      COCCL_WARN("fused path: peer memory of comm %llu could not be mapped on every rank; all ranks use the staged pipeline", (unsigned long long)comm->id);
      st.broken = true;
      st.workspace.close(api, x);
      st.signals.close(api, x);
      st.half = 0;
      lock.unlock();
      ++stagedCalls;
      ++stagedSetupFailed;
      return StagedExecutor::execute(rt, call);
    }
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
  a.epoch = st.epoch;  // full 32 bits: waitFlag compares with a wrapping signed difference
  a.timeoutNs = 20ull * 1000000000ull;
  a.codec = kc;
  a.slotBytes = slot;
  a.regionBOffset = region;
  a.in[comm->rank] = info.sendbuff;
  a.out[comm->rank] = info.recvbuff;
  for (int p = 0; p < n; ++p) {
    a.ws[p] = static_cast<uint8_t*>(st.workspace.ptr(p)) + (size_t)(st.epoch & 1u) * st.half;
    a.flags[p] = static_cast<unsigned int*>(st.signals.ptr(p));
    a.status[p] = static_cast<char*>(st.signals.ptr(p)) + cocclkFlagBytes();
  }
  const int rc = cocclkFusedCollective(&a, 1, rt->config().fusedMaxCtas, info.stream);
  if (rc != 0) return rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError;
  // the status word (written by a bounded wait that ran out) follows the kernel to pinned host memory, where
  // asyncStatus reads it without touching the device
  if (st.hostStatus) cudaMemcpyAsync(st.hostStatus, a.status[comm->rank], sizeof(unsigned int), cudaMemcpyDeviceToHost, info.stream);
  ++fusedCalls;
  return ncclSuccess;
}

unsigned int FusedExecutor::asyncStatus(Comm* comm) {
  std::lock_guard<std::mutex> lock(gMutex);
  auto it = gStates.find(comm);
  if (it == gStates.end()) return 0;
  volatile unsigned int* p = it->second.hostStatus;   // set once, under the communicator's lock, never freed before release
  return p == nullptr ? 0 : *p;
}

}  // namespace coccl
