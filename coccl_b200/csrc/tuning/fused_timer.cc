#include "tuning/fused_timer.h"

#include <stdlib.h>
#include <string.h>

#include <vector>

#include "runtime/log.h"
#include "runtime/transport_exchange.h"

namespace coccl {

FusedTimer::~FusedTimer() {
  for (auto& kv : scratch_)
    if (kv.second.ptr) cudaFree(kv.second.ptr);
}

void FusedTimer::release(Comm* comm) {
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = scratch_.find(comm);
  if (it == scratch_.end()) return;
  if (it->second.ptr) cudaFree(it->second.ptr);
  scratch_.erase(it);
}

bool FusedTimer::measurable(Runtime*, const PreparedCall& call) {
  const char* env = getenv("COCCL_AUTOTUNE_MEASURE");
  if (env != nullptr && strcmp(env, "0") == 0) return false;
  const CallInfo& info = call.info;
  if (info.op != Operation::AllReduce || info.comm == nullptr || info.comm->transport == nullptr) return false;
  const size_t bytes = info.count * cocclTypeSize(info.datatype);
  if (bytes < kMinBytes || bytes > kMaxBytes) return false;
  if (!FusedExecutor::serves(call, Algorithm::ArOneShot) || !FusedExecutor::serves(call, Algorithm::ArTwoShot)) return false;
  // a stream that is being captured into a graph cannot be synchronised or timed
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(info.stream, &capture) != cudaSuccess) { cudaGetLastError(); return false; }
  return capture == cudaStreamCaptureStatusNone;
}

bool FusedTimer::time(Runtime* rt, const PreparedCall& call, Algorithm algorithm, double* seconds) {
  const CallInfo& info = call.info;
  Comm* comm = info.comm;
  const size_t bytes = info.count * cocclTypeSize(info.datatype);
  TransportExchange exchange(comm, info.stream);
  std::vector<int> flags((size_t)comm->nRanks, 0);
  auto everyone = [&](bool mine) {
    const int v = mine ? 1 : 0;
    if (!exchange.allGather(&v, flags.data(), sizeof(int))) return false;
    for (int f : flags)
      if (f == 0) return false;
    return true;
  };
  // 1. every rank has room for the output, or nobody runs anything
  bool ok = true;
  Scratch* mine_;
  {
    std::lock_guard<std::mutex> lock(mutex_);
    mine_ = &scratch_[comm];   // map nodes never move
  }
  Scratch& scratch = *mine_;
  if (scratch.capacity < bytes) {
    if (scratch.ptr) cudaFree(scratch.ptr);
    scratch = Scratch();
    if (cudaMalloc(&scratch.ptr, bytes) == cudaSuccess) scratch.capacity = bytes;
    else { cudaGetLastError(); scratch.ptr = nullptr; ok = false; }
  }
  if (!everyone(ok)) return false;
  // 2. the candidate itself, through the executor that serves real calls
  PreparedCall trial = call;
  trial.algorithm = algorithm;
  trial.info.recvbuff = scratch.ptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  ok = cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess;
  for (int i = 0; i < kWarmup && ok; ++i) ok = executor_->execute(rt, trial) == ncclSuccess;
  ok = ok && cudaEventRecord(e0, info.stream) == cudaSuccess;
  for (int i = 0; i < kIterations && ok; ++i) ok = executor_->execute(rt, trial) == ncclSuccess;
  ok = ok && cudaEventRecord(e1, info.stream) == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess;
  float ms = 0.f;
  ok = ok && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess && executor_->asyncStatus(comm) == 0;
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (!ok) cudaGetLastError();
  // 3. the slowest rank's time, the same number everywhere; one failure anywhere drops the candidate everywhere
  std::vector<double> all((size_t)comm->nRanks, 0.0);
  const double mine = ok ? (double)ms * 1e-3 / kIterations : -1.0;
  if (!exchange.allGather(&mine, all.data(), sizeof(double))) return false;
  double worst = 0.0;
  for (double t : all) {
    if (!(t > 0.0)) return false;
    if (t > worst) worst = t;
  }
  *seconds = worst;
  if (comm->rank == 0)
    COCCL_INFO(kLogTuning, "measured %s bytes=%zu ranks=%d: %.1f us", algorithmName(algorithm), bytes, comm->nRanks, worst * 1e6);
  return true;
}

}  // namespace coccl
