// Host-level all-gather of small blobs through a communicator's own transport (symm_workspace.h's HostExchange over
// NCCL): what the collective set-up of peer-mapped regions uses to move handles and outcomes between the ranks.
#pragma once
#include <cuda_runtime.h>

#include "runtime/comm.h"
#include "runtime/symm_workspace.h"

namespace coccl {

// Host-level all-gather through the communicator's own transport: the blobs travel through two small device
// buffers and come back with a stream synchronisation (rare path: region set-up and regrowth only).
class TransportExchange : public HostExchange {
 public:
  TransportExchange(Comm* comm, cudaStream_t s) : comm_(comm), stream_(s) {}
  ~TransportExchange() override {
    if (dMine_) cudaFree(dMine_);
    if (dAll_) cudaFree(dAll_);
  }
  int rank() const override { return comm_->rank; }
  int nRanks() const override { return comm_->nRanks; }
  bool allGather(const void* mine, void* all, size_t bytes) override {
    const size_t n = (size_t)comm_->nRanks;
    if (bytes > cap_) {
      if (dMine_) cudaFree(dMine_);
      if (dAll_) cudaFree(dAll_);
      dMine_ = dAll_ = nullptr;
      cap_ = 0;
      if (cudaMalloc(&dMine_, bytes) != cudaSuccess || cudaMalloc(&dAll_, bytes * n) != cudaSuccess) return false;
      cap_ = bytes;
    }
    if (cudaMemcpyAsync(dMine_, mine, bytes, cudaMemcpyHostToDevice, stream_) != cudaSuccess) return false;
    if (comm_->transport->allGather(comm_, dMine_, dAll_, bytes, ncclUint8, stream_) != ncclSuccess) return false;
    if (cudaMemcpyAsync(all, dAll_, bytes * n, cudaMemcpyDeviceToHost, stream_) != cudaSuccess) return false;
    return cudaStreamSynchronize(stream_) == cudaSuccess;
  }

 private:
  Comm* comm_;
  cudaStream_t stream_;
  void* dMine_ = nullptr;
  void* dAll_ = nullptr;
  size_t cap_ = 0;
};

}  // namespace coccl
