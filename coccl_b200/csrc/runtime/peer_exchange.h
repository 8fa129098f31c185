// Transport of the staged pipeline over peer memory (kernels/exchange_kernels.cu) instead of NCCL.
//
// The staged pipeline moves encoded bytes with an all-to-all or an all-gather between its compress and decompress
// stages. On one NVSwitch domain those bytes can be stored straight into the receiver's memory by one kernel, so that
// also codecs without a tile form (rANS, ZFP at odd rates, third-party plugins) run without a library collective on the
// compressed path, and framed codecs exchange exactly the bytes that exist WITHOUT the host reading the frame sizes
// first (the kernel reads them from the metadata the codec left on the device). The reference does this with
// ncclAllToAll / ncclAllGather and a device-to-host copy of the frame headers
// (src/coccl-extend/core/pipeline/coccl_pipeline_stage.cc:120-139, coccl_pipeline_execute.cc:218-260).
//
// One PeerDataPath exists per communicator that qualifies: one node, at most 8 ranks, peer memory mappable on EVERY
// rank (agreed collectively; otherwise every rank keeps NCCL), and COCCL_STAGED_TRANSPORT not set to "nccl".
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <mutex>

#include "compressor_plugin/detail/coccl_compressor_abi.h"
#include "runtime/comm.h"
#include "runtime/symm_workspace.h"

namespace coccl {

class PeerDataPath {
 public:
  // The data path of `comm`, or nullptr when its staged traffic stays on the communicator's transport. The first
  // call per communicator is collective (every rank of the communicator reaches it at the same staged call).
  static PeerDataPath* of(Comm* comm, cudaStream_t stream);
  // Local teardown (communicator destruction).
  static void release(Comm* comm);
  // Status word of `comm`'s exchanges (0 = fine or no data path), from pinned host memory.
  static unsigned int asyncStatusOf(Comm* comm);
  // Calls served so far in this process (all communicators).
  static uint64_t calls();

  // Whether a call with these sizes can be served; depends on sizes only, so every rank answers the same.
  static bool serves(size_t frames, size_t frameStride);

  // gather = false: block p of `send` goes to rank p; true: the one block of `send` goes to every rank. A block is
  // `frames` frames of `frameStride` bytes; sendMeta / recvMeta (device memory, one record per frame) are null for
  // data whose frames are always full. Collective when the staging area has to grow.
  ncclResult_t exchange(bool gather, const void* send, void* recv, size_t frames, size_t frameStride,
                        const cocclCompressorFrameMetadata* sendMeta, cocclCompressorFrameMetadata* recvMeta,
                        cudaStream_t stream);
  // Status word of this communicator's exchanges (0 = fine), from pinned host memory.
  unsigned int asyncStatus() const { return hostStatus_ ? *(volatile unsigned int*)hostStatus_ : 0; }

 private:
  explicit PeerDataPath(Comm* comm) : comm_(comm) {}
  Comm* comm_;
  SymmRegion signals_, staging_;
  size_t half_ = 0;
  unsigned epoch_ = 0;
  unsigned int* hostStatus_ = nullptr;
  // The pipeline issues the slices of one call on several streams; the exchanges of one communicator share flags and
  // staging halves and must run one after another on the device, in the order they were issued (the same on every rank)
  cudaEvent_t last_ = nullptr;
  std::mutex mutex_;
  friend struct PeerDataPathTable;
};

}  // namespace coccl
