// Host runtime: the router that decides, for every collective call, between the compressed
// path and the native transport; prepared calls; group batching; hierarchy cache; init/destroy.
//
// Routing rules (in order; src/coccl-extend/core/runtime/coccl_runtime.cc:181-229):
//   1 compression disabled -> native            2 call issued by the runtime itself -> native
//   3 the training classifier observes the call 4 nRanks>1, sum only, count>0, buffers non-null,
//     all-reduce count divisible by nRanks      5 logical bytes = count*size (*nRanks for AG/RS/A2A)
//   6 training mode and role unknown -> native  7 resolve codecs for default/intra/inter scopes
//     (lossy codecs take fp16/bf16/fp32; int8/int32/int64 only with a bytewise-lossless codec)
//   8 bytes <= threshold -> native              9 reduce-scatter / all-reduce pick an algorithm
//  10 inside a group the call is deferred, otherwise executed.
// Explicit calls (coccl*Comp*) skip rule 8 (coccl_runtime.cc:231-266).
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "compression/compressor_runtime.h"
#include "config/config.h"
#include "runtime/comm.h"

namespace coccl {

enum class Func : uint8_t { Collective, Send, Recv };

struct CallInfo {
  Operation op = Operation::Count;
  Func func = Func::Collective;
  const void* sendbuff = nullptr;
  void* recvbuff = nullptr;
  size_t count = 0;
  ncclDataType_t datatype = ncclFloat32;
  ncclRedOp_t redOp = ncclSum;
  int peer = -1;
  Comm* comm = nullptr;
  cudaStream_t stream = nullptr;
};

enum class Algorithm : uint8_t { None = 0, RsOneShot, RsTwoShot, ArOneShot, ArTwoShot, ArTripleShot };
const char* algorithmName(Algorithm a);

// Immutable description of a call that will run compressed.
struct PreparedCall {
  CallInfo info;
  const OperationDescriptor* desc = nullptr;
  Role role = Role::Normal;
  PolicyKey policy;
  Algorithm algorithm = Algorithm::None;
  CompressorPolicy* codecs[3] = {nullptr, nullptr, nullptr};  // by Scope
  bool datatypeOk[3] = {false, false, false};
  size_t thresholdBytes = 0;
  CompressorPolicy* codec(Scope s) const { return codecs[(size_t)s]; }
  bool anyCodec() const { return codecs[0] || codecs[1] || codecs[2]; }
};

// Which scopes an algorithm draws its codecs from: two-shot reduce-scatter uses intra+inter,
// triple-shot all-reduce all three, flat algorithms the intra scope on one node and the default
// scope otherwise; send/recv picks intra or inter by the peer's node
// (core/runtime/coccl_prepared_call.cc:7-80).
void algorithmScopes(const PreparedCall& p, Algorithm a, bool use[3]);
bool algorithmHasCompression(const PreparedCall& p, Algorithm a);
bool algorithmSupported(const PreparedCall& p, Algorithm a);
// node of a rank of `comm` (ranks are laid out node-major, localRanks per node)
int nodeOfRank(const Comm* comm, int rank);

class Runtime;

// How prepared calls are carried out (production: fused kernels or the staged pipeline; tests: fakes).
class Executor {
 public:
  virtual ~Executor() {}
  virtual ncclResult_t execute(Runtime* rt, const PreparedCall& call) = 0;
  // a batch of grouped send/recv calls executed as one unit
  virtual ncclResult_t executeSendRecvBatch(Runtime* rt, const std::vector<PreparedCall>& batch) = 0;
};

// Picks the reduce-scatter / all-reduce algorithm (tuning/selector.cc); may be replaced in tests.
class AlgorithmSelector {
 public:
  virtual ~AlgorithmSelector() {}
  virtual ncclResult_t select(Runtime* rt, PreparedCall* call) = 0;
};

// Observes calls in training mode and reports the role of a communicator (training/assist.cc).
class RoleOracle {
 public:
  virtual ~RoleOracle() {}
  virtual void observe(const CallInfo& info, int groupDepth) = 0;
  virtual Role roleOf(Comm* comm) = 0;
};

struct RouterStats {
  uint64_t policyLookups = 0, nativeCalls = 0, compressedCalls = 0, deferredCalls = 0;
};

class Runtime {
 public:
  Runtime();
  ~Runtime();

  // Enable with an already parsed configuration (processConfig() in production).
  ncclResult_t enable(const Config& cfg, int nodes, int devicesPerNode, std::string* error);
  void disable();
  bool enabled() const { return enabled_; }
  const Config& config() const { return compressors_.config(); }
  CompressorRuntime& compressors() { return compressors_; }

  void setExecutor(Executor* e) { executor_ = e; }
  void setSelector(AlgorithmSelector* s) { selector_ = s; }
  void setRoleOracle(RoleOracle* r) { roles_ = r; }
  Executor* executor() const { return executor_; }

  // Per-communicator life cycle (hierarchy cache, training registration happen lazily).
  ncclResult_t commInit(Comm* comm);
  ncclResult_t commDestroy(Comm* comm);

  // Router entry point of every public collective. *enqueued == false: the caller runs natively.
  ncclResult_t enqueueCheck(const CallInfo& info, bool* enqueued);
  // Explicit coccl*Comp* call: needs an enabled runtime and a matching policy, ignores the threshold;
  // an unsupported datatype is replayed natively; no codec at the algorithm's scopes is ncclInvalidUsage.
  ncclResult_t enqueueExplicit(const CallInfo& info, Algorithm algorithm);
  // Run a call on the native transport with the re-entrancy guard raised.
  ncclResult_t replayNative(const CallInfo& info);
  ncclResult_t executePrepared(const PreparedCall& call);

  // Group hooks (called by the API layer around the transport's own group).
  void groupStart();
  int groupDepth() const;
  bool groupHasPending() const;
  // nativePending: the transport has native work queued in this group. Decides whether the whole batch
  // must be replayed natively (native work pending, a native entry in the batch, or send/recv mixed
  // with collectives); if so it issues the replays now, inside the transport group.
  ncclResult_t groupPrepareEnd(Transport* t, bool nativePending);
  // After the transport group has been flushed: run what stayed compressed.
  ncclResult_t groupDrain();
  void groupAbort();
  void groupEnqueuePrepared(const PreparedCall& call);
  void groupEnqueueNative(const CallInfo& info);
  ncclResult_t groupEnd(Transport* t, bool nativePending);

  // Lazily split `owner` into intra-node (color = rank / localRanks) and inter-node
  // (color = rank % localRanks) communicators.
  ncclResult_t hierarchy(Comm* owner, Comm** intra, Comm** inter);

  static bool internalCall();  // true while the runtime itself is issuing transport calls
  RouterStats& stats() { return stats_; }

 private:
  ncclResult_t prepare(const CallInfo& info, PreparedCall* out, bool explicitCall, bool* native);
  ncclResult_t resolveCodecs(PreparedCall* call);
  ncclResult_t routeNativeGrouped(const CallInfo& info, bool* enqueued);
  CompressorRuntime compressors_;
  bool enabled_ = false;
  Executor* executor_ = nullptr;
  AlgorithmSelector* selector_ = nullptr;
  RoleOracle* roles_ = nullptr;
  RouterStats stats_;
};

// Process-wide instance used by the C API.
Runtime& globalRuntime();

}  // namespace coccl
