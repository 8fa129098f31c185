// Compressor runtime: loads `lib<name>.so` plugins, turns every configured policy scope into
// a ready-to-run CompressorPolicy (plugin + parsed config + threshold + per-device resources),
// serves the host API plugins call back into (scratch, persistent memory, host state) and
// wraps the four plugin operations with validation and generic fallbacks.
//
// Behavioural model: src/coccl-extend/core/compression/coccl_compressor.cc:100-517 (loading,
// 4-D policy table [role][variant][operation][scope], host API, output validation),
// coccl_compressor_size.cc:5-36 (size bound; ncclInvalidUsage from the plugin means "raw size"),
// compress.cc:7-113 (raw pass-through decode, fused op if available and not framed, otherwise
// decode to scratch + chunk reduction (+ re-encode)).
#pragma once
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "compressor_plugin/detail/coccl_compressor_abi.h"
#include "config/config.h"

namespace coccl {

// Device-memory services used by the host API; tests replace them with host-side fakes.
struct DeviceAllocator {
  cudaError_t (*mallocAsync)(void** p, size_t bytes, cudaStream_t s);
  cudaError_t (*freeAsync)(void* p, cudaStream_t s);
  cudaError_t (*mallocSync)(void** p, size_t bytes);
  cudaError_t (*freeSync)(void* p);
};
const DeviceAllocator& cudaDeviceAllocator();

struct LoadedPlugin {
  std::string name;
  std::string path;
  void* handle = nullptr;                       // dlopen handle (null for built-in / test plugins)
  const cocclCompressorPlugin* descriptor = nullptr;
  // Optional export `cocclFusedCodecQuery`: lets a codec whose kernels are the library's own tile codecs
  // describe a parsed configuration as a kernel codec, which unlocks the fused collectives for it.
  // Returns 1 and fills `out` (a cocclkCodec) when the configuration can run fused for `ncclDatatype`.
  int (*fusedQuery)(const void* config, int ncclDatatype, void* out) = nullptr;
  // Optional export `cocclFusedCodecDeltaQuery`: the same for a STATEFUL configuration that sends the change against
  // the previous result (sdp4bit subAdd). The fused all-gather has a delta form whose state is the output buffer
  // itself; `out` receives the tile codec of the deltas.
  int (*deltaQuery)(const void* config, int ncclDatatype, void* out) = nullptr;
};

// Everything the pipeline needs to run one codec for one policy scope.
class CompressorPolicy {
 public:
  CompressorPolicy(const LoadedPlugin* plugin, void* config, size_t thresholdBytes, std::string where);
  ~CompressorPolicy();
  CompressorPolicy(const CompressorPolicy&) = delete;
  CompressorPolicy& operator=(const CompressorPolicy&) = delete;

  const LoadedPlugin* plugin() const { return plugin_; }
  const void* config() const { return config_; }
  size_t thresholdBytes() const { return thresholdBytes_; }
  uint64_t capabilities() const { return plugin_->descriptor->capabilities; }
  bool has(cocclCompressorCapability c) const { return (capabilities() & c) != 0; }
  const std::string& where() const { return where_; }

  // per-device resources handed out through the host API
  struct Persistent { void* ptr = nullptr; size_t bytes = 0; };
  struct HostState { void* ptr = nullptr; cocclCompressorDestroyStateFn destroy = nullptr; };
  struct DeviceResources {
    std::map<size_t, Persistent> persistent;
    std::map<const void*, HostState> states;
    size_t scratchPeak = 0, persistentBytes = 0;
  };
  DeviceResources& resources(int device);
  void releaseResources(const DeviceAllocator& alloc);
  std::mutex& mutex() { return mutex_; }

 private:
  const LoadedPlugin* plugin_;
  void* config_;
  size_t thresholdBytes_;
  std::string where_;
  std::mutex mutex_;
  std::map<int, DeviceResources> perDevice_;
};

// Where and for whom an operation runs.
struct ExecEnv {
  cudaStream_t stream = nullptr;
  int cudaDev = 0, rank = 0, nRanks = 1, nodes = 1, devicesPerNode = 1;
  const DeviceAllocator* alloc = nullptr;  // null = CUDA
};

class CompressorRuntime {
 public:
  CompressorRuntime();
  ~CompressorRuntime();

  // Load every catalogued plugin and build the policy table. `nodes` x `devicesPerNode` is the
  // topology handed to parseConfig. Returns false with `error` set on the first failure.
  bool initialize(const Config& cfg, int nodes, int devicesPerNode, std::string* error);
  // Register an in-process plugin (tests, built-in codecs); takes no ownership.
  void addBuiltin(const cocclCompressorPlugin* descriptor);
  void shutdown();

  const LoadedPlugin* findPlugin(const std::string& name) const;
  // Policy for (role, variant, operation, scope) with scope inheritance applied; null = none.
  CompressorPolicy* resolve(Role role, Variant variant, Operation op, Scope scope) const;
  size_t thresholdFor(Role role, Variant variant, Operation op) const;
  const Config& config() const { return cfg_; }
  bool initialized() const { return initialized_; }
  const std::vector<std::unique_ptr<LoadedPlugin>>& plugins() const { return plugins_; }

 private:
  bool loadPlugin(const std::string& name, const std::string& dir, std::string* error);
  Config cfg_;
  bool initialized_ = false;
  std::vector<std::unique_ptr<LoadedPlugin>> plugins_;
  std::vector<std::unique_ptr<CompressorPolicy>> policies_;
  // [policy id][scope] -> policy (after inheritance)
  CompressorPolicy* table_[kPolicyCount][static_cast<size_t>(Scope::Count)] = {};
};

// --- size bound -----------------------------------------------------------------------------
// Upper bound of the encoded size of (elements, chunks, datatype). A plugin that answers
// ncclInvalidUsage (no bound known) yields the raw size; the bound must divide evenly into chunks.
ncclResult_t encodedSizeBound(const CompressorPolicy* policy, cocclCompressorOperation op, size_t elements,
                              size_t chunks, ncclDataType_t datatype, size_t* bytes);

// --- operations -----------------------------------------------------------------------------
ncclResult_t compress(CompressorPolicy* policy, const cocclCompressorView& input, cocclCompressorView* output,
                      const ExecEnv& env);
ncclResult_t decompress(CompressorPolicy* policy, const cocclCompressorView& input, cocclCompressorView* output,
                        const ExecEnv& env);
// output = sum over `reduceChunks` encoded copies; fused plugin op when offered (and the codec is not
// framed), otherwise decode everything to scratch and reduce with the generic chunk-sum kernel.
ncclResult_t decompressReduce(CompressorPolicy* policy, const cocclCompressorView& input,
                              cocclCompressorView* output, size_t reduceChunks, const ExecEnv& env);
// ... and re-encode the sum with `encoder` (may be the same policy).
ncclResult_t decompressReduceCompress(CompressorPolicy* decoder, CompressorPolicy* encoder,
                                      const cocclCompressorView& input, cocclCompressorView* output,
                                      size_t reduceChunks, ncclDataType_t originalDatatype, size_t originalElements,
                                      const ExecEnv& env);

// Hook for the generic reduction (tests substitute a host version). Signature of cocclkReduceChunks.
using ReduceChunksFn = int (*)(const void*, void*, long, int, long, int, cudaStream_t);
void setReduceChunksHook(ReduceChunksFn fn);

}  // namespace coccl
