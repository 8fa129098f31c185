// Policy model: COCCL_ENABLE / COCCL_CONFIG_FILE and the TOML schema (normal and training
// modes, per-operation default/intra/inter compressor scopes, size threshold, pipeline depth,
// buffer and autotune knobs). Schema and validation rules follow
// src/coccl-extend/core/config/coccl_config.cc:27-37 (unknown keys are errors at every level),
// :149-196 (codec options reach plugins as strings), :198-318 (scopes; a disabled scope may not
// name a compressor), :320-429 (training), :431-583 (sections, catalog check) and :624-636
// (scope inheritance: explicit intra/inter wins, else default).
#pragma once
#include <stddef.h>
#include <stdint.h>
#include <array>
#include <map>
#include <string>
#include <vector>

#include "coccl/operation.h"

namespace coccl {

enum class Mode { Normal, Training };
enum class DpStrategy { Ddp, Sdp, Fsdp };
enum class RsAlgorithmPolicy { Auto, OneShot, TwoShot };
enum class ArAlgorithmPolicy { Auto, OneShot, TwoShot, TripleShot };
enum class Role : uint8_t { Normal = 0, DataParallel, TensorParallel, PipelineParallel, Unknown, Count };

using OptionMap = std::map<std::string, std::string>;

struct ScopeEntry {
  bool configured = false;  // the table exists in the file
  bool enabled = false;
  std::string compressor;
  OptionMap options;        // every scalar rendered as text
};

struct PolicySlot {
  std::array<ScopeEntry, static_cast<size_t>(Scope::Count)> scopes;
  size_t thresholdBytes = 8ull << 20;
  const ScopeEntry& configured(Scope s) const { return scopes[static_cast<size_t>(s)]; }
};

struct EffectiveScope {
  const ScopeEntry* entry = nullptr;
  Scope source = Scope::Default;
  bool enabled() const { return entry != nullptr && entry->enabled; }
};
// intra/inter inherit the default scope unless configured themselves
EffectiveScope effectiveScope(const PolicySlot& slot, Scope scope);

enum class PolicyId : uint8_t {
  NormalAllGather = 0, NormalReduceScatter, NormalAllReduce, NormalAllToAll, NormalSendRecv,
  DpAllGather, DpReduceScatter, DpAllReduce,
  TpAllGather, TpReduceScatter, TpAllReduce,
  PpSendRecvForward, PpSendRecvBackward,
  Count
};
constexpr size_t kPolicyCount = static_cast<size_t>(PolicyId::Count);

struct PolicyInfo {
  PolicyId id;
  const char* path;   // TOML path, e.g. "training.dp.reduce_scatter"
  Mode mode;
  Role role;
  PolicyKey key;      // operation + variant (scope left Default)
};
const PolicyInfo& policyInfo(PolicyId id);
// Slot lookup used by the router: which slot serves (mode, role, operation, variant)?
bool findPolicy(Mode mode, Role role, Operation op, Variant variant, PolicyId* id);

constexpr int kMinPipelineDepth = 1;
constexpr int kMaxPipelineDepth = 16;

struct Config {
  // [runtime]
  Mode mode = Mode::Normal;
  size_t thresholdBytes = 8ull << 20;
  // [compressor_plugins]
  std::vector<std::string> compressors;
  std::string libraryPath;  // resolved against the config file's directory
  // [pipeline]
  int pipelineDepth = 1;
  // [runtime] fused_kernel_max_ctas: CTAs one fused kernel may occupy per GPU; 0 = as many as stay resident. A job that
  // overlaps collectives with compute (or runs two communicators at once) leaves the rest of the SMs to the other work,
  // so that the fused kernel's CTAs, which wait on one another's flags, are all resident.
  int fusedMaxCtas = 0;
  // [buffer]
  size_t poolLimitBytes = 0, legacyBlockBytes = 0, physicalChunkBytes = 8ull << 20;
  // [autotune]
  bool autotune = true;
  size_t profileMinBytes = 256ull << 10, profileMaxBytes = 8ull << 30;
  int autotuneWarmup = 3, autotuneIterations = 10;
  RsAlgorithmPolicy rsAlgorithm = RsAlgorithmPolicy::Auto;
  ArAlgorithmPolicy arAlgorithm = ArAlgorithmPolicy::Auto;
  // [training]
  int observationIterations = 5;
  int dpSize = 1, tpSize = 1, ppSize = 1;
  DpStrategy dpStrategy = DpStrategy::Sdp;
  bool sequenceParallel = false;
  // policy slots
  std::array<PolicySlot, kPolicyCount> slots;

  const PolicySlot& slot(PolicyId id) const { return slots[static_cast<size_t>(id)]; }
};

bool loadConfigText(const std::string& text, const std::string& baseDir, Config* out, std::string* error);
bool loadConfigFile(const std::string& path, Config* out, std::string* error);

// Flat "key = value" rendering of the effective configuration, one line per setting, with a
// "# <path>.<scope> source=<scope>" comment for every policy scope that resolves to a codec.
std::string formatConfig(const Config& cfg);

// Process-wide singleton. Reads COCCL_ENABLE (unset/0/1) and COCCL_CONFIG_FILE exactly once;
// an invalid value or file leaves compression disabled for the life of the process.
struct ProcessConfig {
  bool enabled = false;
  bool valid = true;
  std::string error;
  Config config;
};
const ProcessConfig& processConfig();
// Re-evaluate the environment (tests only).
void resetProcessConfigForTesting();

}  // namespace coccl
