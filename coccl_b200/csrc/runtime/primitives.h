// Primitive recipes: the stage list of every compressed operation / algorithm, and the
// production executor that carries prepared calls out (fused kernel when the codec and topology
// allow it, staged pipeline otherwise).
//
// Recipes (src/coccl-extend/extensions/primitives/coccl_allgather.cc:7-24, coccl_alltoall.cc:7-23,
// coccl_reducescatter.cc:12-60, coccl_allreduce.cc:12-103, coccl_hierarchical_reduction.cc:15-63):
//   AllGather              Compress(1) -> AllGather -> Decompress(N)            in place: input rank chunk
//   AllToAll               Compress(N) -> AllToAll -> Decompress(N)
//   ReduceScatter one-shot Compress(N) -> AllToAll -> DecompressReduce(N)       in place: output rank chunk
//   ReduceScatter two-shot swizzled input; Compress -> AllToAll(intra) -> DecompReduceComp(local, inter codec)
//                          -> AllToAll(inter) -> DecompressReduce(nodes); a level without codec uses a
//                          native reduce-scatter
//   AllReduce one-shot     Compress(N) -> AllGather -> DecompressReduce(N)      always serial
//   AllReduce two-shot     Compress(N) -> AllToAll -> DecompReduceComp(N) -> AllGather -> Decompress
//   AllReduce triple-shot  hierarchical reduction (last encoder = default scope) -> AllGather -> Decompress
#pragma once
#include <atomic>
#include "memory/buffer_manager.h"
#include "pipeline/pipeline.h"
#include "runtime/runtime.h"

namespace coccl {

// Build the pipeline specification of a prepared collective (not send/recv). `intra`/`inter` are the
// hierarchy communicators, needed by the hierarchical algorithms only.
ncclResult_t buildRecipe(const PreparedCall& call, Comm* intra, Comm* inter, PipelineSpec* spec);
// Codec a flat algorithm uses: the intra scope on one node, the default scope otherwise.
CompressorPolicy* flatCodec(const PreparedCall& call);

class StagedExecutor : public Executor {
 public:
  StagedExecutor(BufferManager* buffers) : buffers_(buffers) {}
  ncclResult_t execute(Runtime* rt, const PreparedCall& call) override;
  ncclResult_t executeSendRecvBatch(Runtime* rt, const std::vector<PreparedCall>& batch) override;
 protected:
  BufferManager* buffers_;
};

// Adds the fused-kernel fast path in front of the staged one (runtime/fused_executor.cc).
class FusedExecutor : public StagedExecutor {
 public:
  FusedExecutor(BufferManager* buffers) : StagedExecutor(buffers) {}
  ncclResult_t execute(Runtime* rt, const PreparedCall& call) override;
  // Whether ONE fused kernel serves this call with this algorithm (one node, at most 8 ranks, a codec with a tile
  // form for the datatype, a flat algorithm). Depends on the call's description only: equal on every rank.
  static bool serves(const PreparedCall& call, Algorithm algorithm);
  void releaseComm(Comm* comm);
  // Status word of the communicator's last completed fused kernels (0 = fine; otherwise the {phase, peer, slice}
  // of the first bounded wait that ran out). Reads pinned host memory only.
  unsigned int asyncStatus(Comm* comm);
  // ranks that are threads of one process share the executor
  std::atomic<uint64_t> fusedCalls{0}, stagedCalls{0};
  // why calls went to the staged pipeline: no fused form for the call (codec, datatype, algorithm, more than one node);
  // the communicator's earlier set-up had failed; this call's set-up (mapping the peers' memory) failed
  std::atomic<uint64_t> stagedNoFusedForm{0}, stagedAfterFailedSetup{0}, stagedSetupFailed{0};
};

}  // namespace coccl
