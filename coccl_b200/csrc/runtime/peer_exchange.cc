#include "runtime/peer_exchange.h"

#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <map>

#include "kernels/kernels_api.h"
#include "runtime/log.h"
#include "runtime/transport_exchange.h"

namespace coccl {

struct PeerDataPathTable {
  std::mutex mutex;
  std::map<Comm*, PeerDataPath*> paths;   // nullptr entry = decided: this communicator stays on its transport
  static PeerDataPathTable& get() {
    static PeerDataPathTable* t = new PeerDataPathTable();
    return *t;
  }
  static PeerDataPath* make(Comm* comm) { return new PeerDataPath(comm); }
  static void destroy(PeerDataPath* p) {
    if (p == nullptr) return;
    cudaDeviceSynchronize();
    p->staging_.closeLocal(cudaSymmApi());
    p->signals_.closeLocal(cudaSymmApi());
    if (p->hostStatus_) cudaFreeHost(p->hostStatus_);
    if (p->last_) cudaEventDestroy(p->last_);
    delete p;
  }
  static bool open(PeerDataPath* p, cudaStream_t stream) {
    TransportExchange x(p->comm_, stream);
    bool ok = p->signals_.reopen(cudaSymmApi(), x, (size_t)cocclkFlagBytes() + 256);
    if (ok && cudaHostAlloc((void**)&p->hostStatus_, 64, cudaHostAllocDefault) == cudaSuccess) *p->hostStatus_ = 0;
    if (ok && cudaEventCreateWithFlags(&p->last_, cudaEventDisableTiming) != cudaSuccess) { p->last_ = nullptr; cudaGetLastError(); }
    return ok;
  }
};

namespace {
std::atomic<uint64_t> gCalls{0};

bool disabledByEnv() {
  const char* v = getenv("COCCL_STAGED_TRANSPORT");
  return v != nullptr && strcmp(v, "nccl") == 0;
}
}  // namespace

uint64_t PeerDataPath::calls() { return gCalls.load(); }

unsigned int PeerDataPath::asyncStatusOf(Comm* comm) {
  PeerDataPathTable& t = PeerDataPathTable::get();
  std::lock_guard<std::mutex> lock(t.mutex);
  auto it = t.paths.find(comm);
  return (it == t.paths.end() || it->second == nullptr) ? 0 : it->second->asyncStatus();
}

bool PeerDataPath::serves(size_t frames, size_t frameStride) {
  long pieceBytes = 0;
  return frames >= 1 && frameStride >= 16 && (frameStride & 15) == 0 &&
         cocclkExchangePieces((int)frames, (long)frameStride, &pieceBytes) >= 1;
}

PeerDataPath* PeerDataPath::of(Comm* comm, cudaStream_t stream) {
  if (comm == nullptr || comm->transport == nullptr || !comm->transport->peerMemoryCapable() || comm->nNodes != 1 || comm->nRanks < 2 ||
      comm->nRanks > COCCLK_MAX_RANKS || disabledByEnv())
    return nullptr;
  PeerDataPathTable& t = PeerDataPathTable::get();
  {
    std::lock_guard<std::mutex> lock(t.mutex);
    auto it = t.paths.find(comm);
    if (it != t.paths.end()) return it->second;
  }
  // first staged call of this communicator: every rank is here (same call sequence), the set-up is collective and its
  // outcome is agreed, so either all ranks get a data path or none does
  cudaStreamSynchronize(stream);
  PeerDataPath* p = PeerDataPathTable::make(comm);
  if (!PeerDataPathTable::open(p, stream)) {
    COCCL_WARN("staged path: peer memory of comm %llu could not be mapped on every rank; its encoded bytes travel through NCCL",
               (unsigned long long)comm->id);
    PeerDataPathTable::destroy(p);
    p = nullptr;
  }
  std::lock_guard<std::mutex> lock(t.mutex);
  t.paths[comm] = p;
  return p;
}

void PeerDataPath::release(Comm* comm) {
  PeerDataPathTable& t = PeerDataPathTable::get();
  PeerDataPath* p = nullptr;
  {
    std::lock_guard<std::mutex> lock(t.mutex);
    auto it = t.paths.find(comm);
    if (it == t.paths.end()) return;
    p = it->second;
    t.paths.erase(it);
  }
  PeerDataPathTable::destroy(p);
}

ncclResult_t PeerDataPath::exchange(bool gather, const void* send, void* recv, size_t frames, size_t frameStride,
                                    const cocclCompressorFrameMetadata* sendMeta, cocclCompressorFrameMetadata* recvMeta,
                                    cudaStream_t stream) {
  if (!serves(frames, frameStride) || (sendMeta == nullptr) != (recvMeta == nullptr)) return ncclInvalidArgument;
  if ((reinterpret_cast<uintptr_t>(send) & 15u) || (reinterpret_cast<uintptr_t>(recv) & 15u)) return ncclInvalidArgument;
  std::lock_guard<std::mutex> lock(mutex_);
  const int n = comm_->nRanks;
  const size_t need = (size_t)cocclkExchangeStagingBytes(n, (int)frames, (long)frameStride);
  if (half_ < need) {
    // collective growth (sizes are equal on every rank by the collective's contract); a failure here cannot be turned
    // into a silent per-rank fallback any more, because the peers are already committed to this path: report it
    cudaStreamSynchronize(stream);
    if (last_ != nullptr && epoch_ > 0) cudaEventSynchronize(last_);   // the previous exchange may sit on another stream
    TransportExchange x(comm_, stream);
    const size_t half = (need + (1u << 20) - 1) / (1u << 20) * (1u << 20);
    if (!staging_.reopen(cudaSymmApi(), x, 2 * half)) {
      half_ = 0;
      COCCL_WARN("staged path: staging area of comm %llu (%zu bytes) could not be mapped on every rank", (unsigned long long)comm_->id, 2 * half);
      return ncclSystemError;
    }
    half_ = staging_.bytes() / 2;
  }
  ++epoch_;
  cocclkExchangeArgs a;
  memset(&a, 0, sizeof(a));
  a.nRanks = n;
  a.rankBase = comm_->rank;
  a.gather = gather ? 1 : 0;
  a.frames = (int)frames;
  a.frameStride = (long)frameStride;
  a.pieces = cocclkExchangePieces((int)frames, (long)frameStride, &a.pieceBytes);
  a.send[comm_->rank] = static_cast<const uint8_t*>(send);
  a.recv[comm_->rank] = static_cast<uint8_t*>(recv);
  a.sendMeta[comm_->rank] = sendMeta;
  a.recvMeta[comm_->rank] = recvMeta;
  for (int p = 0; p < n; ++p) {
    a.staging[p] = static_cast<uint8_t*>(staging_.ptr(p)) + (size_t)(epoch_ & 1u) * half_;
    a.flags[p] = static_cast<unsigned int*>(signals_.ptr(p));
    a.status[p] = static_cast<char*>(signals_.ptr(p)) + cocclkFlagBytes();
  }
  a.epoch = epoch_;
  a.timeoutNs = 20ull * 1000000000ull;
  if (last_ != nullptr && epoch_ > 1) cudaStreamWaitEvent(stream, last_, 0);
  const int rc = cocclkPeerExchange(&a, 1, 0, stream);
  if (rc != 0) return rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError;
  if (last_ != nullptr) cudaEventRecord(last_, stream);
  if (hostStatus_) cudaMemcpyAsync(hostStatus_, a.status[comm_->rank], sizeof(unsigned int), cudaMemcpyDeviceToHost, stream);
  ++gCalls;
  return ncclSuccess;
}

}  // namespace coccl
