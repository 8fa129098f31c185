// Routing sessions (include/coccl/router.h): a private Runtime whose executor records the prepared call instead of
// running it. Everything between the call description and the decision — rule order, policy lookup with scope
// inheritance, datatype support, `bytes <= threshold`, algorithm selection, explicit-call semantics — is the code
// the C API runs (runtime/router.cc, tuning/autotune.cc).
#include <map>
#include <mutex>
#include <string.h>
#include <string>

#include "coccl/router.h"
#include "runtime/log.h"
#include "runtime/runtime.h"
#include "tuning/autotune.h"

using namespace coccl;

namespace {

class RecordingExecutor : public Executor {
 public:
  ncclResult_t execute(Runtime*, const PreparedCall& call) override { last = call; have = true; return ncclSuccess; }
  ncclResult_t executeSendRecvBatch(Runtime*, const std::vector<PreparedCall>& batch) override {
    if (!batch.empty()) { last = batch[0]; have = true; }
    return ncclSuccess;
  }
  PreparedCall last;
  bool have = false;
};

class FixedRole : public RoleOracle {
 public:
  void observe(const CallInfo&, int) override {}
  Role roleOf(Comm*) override { return role; }
  Role role = Role::Normal;
};

struct MeasuredKey {
  int op, dtype, nRanks, log2Bytes;
  bool operator<(const MeasuredKey& o) const {
    if (op != o.op) return op < o.op;
    if (dtype != o.dtype) return dtype < o.dtype;
    if (nRanks != o.nRanks) return nRanks < o.nRanks;
    return log2Bytes < o.log2Bytes;
  }
};
struct MeasuredEntry { int algorithm = 0; double seconds = 0.0; };

// Measured table first (nearest bucket below, else above), then the production selector.
class MeasuredSelector : public AlgorithmSelector {
 public:
  MeasuredSelector(ModelStore* store, std::map<MeasuredKey, std::map<int, double>>* table) : inner_(store), table_(table) {}
  ncclResult_t select(Runtime* rt, PreparedCall* call) override {
    const Config& cfg = rt->config();
    const bool forced = call->info.op == Operation::ReduceScatter ? cfg.rsAlgorithm != RsAlgorithmPolicy::Auto
                                                                  : cfg.arAlgorithm != ArAlgorithmPolicy::Auto;
    if (cfg.autotune && !forced && !table_->empty()) {
      const size_t bytes = call->info.count * cocclTypeSize(call->info.datatype);
      int lg = 0;
      while ((bytes >> (lg + 1)) != 0) ++lg;
      const int op = (int)call->info.op, dt = (int)call->info.datatype, n = call->info.comm->nRanks;
      const std::map<int, double>* best = nullptr;
      for (int d = 0; d < 40 && best == nullptr; ++d) {
        auto it = table_->find(MeasuredKey{op, dt, n, lg - d});
        if (it != table_->end()) best = &it->second;
      }
      for (int d = 1; d < 40 && best == nullptr; ++d) {
        auto it = table_->find(MeasuredKey{op, dt, n, lg + d});
        if (it != table_->end()) best = &it->second;
      }
      if (best != nullptr) {
        int algo = 0;
        double t = 0.0;
        for (const auto& kv : *best) {
          if (!algorithmSupported(*call, (Algorithm)kv.first)) continue;
          if (algo == 0 || kv.second < t) { algo = kv.first; t = kv.second; }
        }
        if (algo != 0) {
          call->algorithm = (Algorithm)algo;
          if (call->info.comm->rank == 0) {
            std::string all;
            for (const auto& kv : *best) all += std::string(algorithmName((Algorithm)kv.first)) + "=" + std::to_string(kv.second * 1e6) + "us ";
            COCCL_INFO(kLogTuning, "select bytes=%zu measured %s-> %s", bytes, all.c_str(), algorithmName(call->algorithm));
          }
          return ncclSuccess;
        }
      }
    }
    return inner_.select(rt, call);
  }
 private:
  AutotuneSelector inner_;
  std::map<MeasuredKey, std::map<int, double>>* table_;
};

}  // namespace

struct cocclRouter {
  std::mutex mutex;
  Runtime rt;
  RecordingExecutor exec;
  FixedRole roles;
  ModelStore models;
  std::map<MeasuredKey, std::map<int, double>> measured;          // compressed algorithms
  std::map<MeasuredKey, std::map<int, double>> measuredNative;    // uncompressed all-reduce variants
  MeasuredSelector selector{&models, &measured};
  Transport* noTransport = nullptr;
  std::string effective;
  uint64_t hash = 0;
  bool enabled = false;
};

extern "C" int cocclRouterOpen(const char* configPath, int nodes, int devicesPerNode, cocclRouter** out, char* error, size_t errorCap) {
  if (out == nullptr) return (int)ncclInvalidArgument;
  auto fail = [&](const std::string& why, ncclResult_t r) {
    if (error != nullptr && errorCap > 0) { strncpy(error, why.c_str(), errorCap - 1); error[errorCap - 1] = 0; }
    return (int)r;
  };
  cocclRouter* r = new cocclRouter();
  if (configPath != nullptr) {
    Config cfg;
    std::string err;
    if (!loadConfigFile(configPath, &cfg, &err)) { delete r; return fail(err, ncclInvalidUsage); }
    if (r->rt.enable(cfg, nodes > 0 ? nodes : 1, devicesPerNode > 0 ? devicesPerNode : 1, &err) != ncclSuccess) {
      delete r;
      return fail(err, ncclInvalidUsage);
    }
    r->enabled = true;
    r->effective = formatConfig(cfg);
  } else {
    r->effective = "compression disabled\n";
  }
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : r->effective) { h ^= c; h *= 1099511628211ull; }
  r->hash = h;
  r->rt.setExecutor(&r->exec);
  r->rt.setSelector(&r->selector);
  r->rt.setRoleOracle(&r->roles);
  *out = r;
  return 0;
}

extern "C" void cocclRouterClose(cocclRouter* r) { delete r; }
extern "C" const char* cocclRouterEffectiveConfig(cocclRouter* r) { return r ? r->effective.c_str() : ""; }
extern "C" uint64_t cocclRouterConfigHash(cocclRouter* r) { return r ? r->hash : 0; }
extern "C" int cocclRouterEnabled(cocclRouter* r) { return r != nullptr && r->enabled ? 1 : 0; }
extern "C" int cocclRouterFusedMaxCtas(cocclRouter* r) { return r != nullptr && r->enabled ? r->rt.config().fusedMaxCtas : 0; }
extern "C" int cocclRouterTrainingMode(cocclRouter* r) { return r != nullptr && r->enabled && r->rt.config().mode == Mode::Training ? 1 : 0; }

extern "C" int cocclRouterDecide(cocclRouter* r, int role, int op, int ncclDatatype, size_t count, int nRanks, int nNodes, int rank,
                                 int redOp, int explicitAlgorithm, cocclRouteDecision* out) {
  if (r == nullptr || out == nullptr || op < 0 || op >= (int)Operation::Count || nRanks < 1) return (int)ncclInvalidArgument;
  memset(out, 0, sizeof(*out));
  std::lock_guard<std::mutex> lock(r->mutex);
  Comm comm;
  comm.nRanks = nRanks;
  comm.rank = rank;
  comm.nNodes = nNodes > 0 ? nNodes : 1;
  comm.localRanks = nRanks / comm.nNodes > 0 ? nRanks / comm.nNodes : 1;
  comm.localRank = rank % comm.localRanks;
  comm.node = rank / comm.localRanks;
  comm.id = 0x726f757465ull;
  static const Role kRoles[] = {Role::Normal, Role::DataParallel, Role::TensorParallel, Role::PipelineParallel};
  r->roles.role = (role >= 0 && role < 4) ? kRoles[role] : Role::Unknown;
  out->role = (int)r->roles.role;
  CallInfo info;
  info.op = (Operation)op;
  info.func = Func::Collective;
  // the router only tests the buffers for null; nothing is dereferenced on this path
  static char dummy[16];
  info.sendbuff = dummy;
  info.recvbuff = dummy;
  info.count = count;
  info.datatype = (ncclDataType_t)ncclDatatype;
  info.redOp = (ncclRedOp_t)redOp;
  info.comm = &comm;
  const size_t width = cocclTypeSize(info.datatype);
  out->totalBytes = count * width * ((info.op == Operation::AllReduce || info.op == Operation::SendRecv) ? 1 : (size_t)nRanks);
  r->exec.have = false;
  ncclResult_t rc = ncclSuccess;
  if (r->enabled) {
    if (explicitAlgorithm >= 0) {
      rc = r->rt.enqueueExplicit(info, (Algorithm)explicitAlgorithm);
      if (rc == ncclInvalidUsage) rc = ncclSuccess;  // no policy for an explicit call: reported as native here
    } else {
      bool taken = false;
      rc = r->rt.enqueueCheck(info, &taken);
    }
  }
  if (rc != ncclSuccess) return (int)rc;
  if (r->exec.have) {
    const PreparedCall& call = r->exec.last;
    out->compressed = 1;
    out->algorithm = (int)call.algorithm;
    out->thresholdBytes = call.thresholdBytes;
    bool use[3];
    algorithmScopes(call, call.algorithm, use);
    CompressorPolicy* codec = nullptr;
    for (int s = 0; s < 3 && codec == nullptr; ++s)
      if (use[s] && call.codecs[s] != nullptr) codec = call.codecs[s];
    if (codec != nullptr) {
      strncpy(out->compressor, codec->plugin()->name.c_str(), sizeof(out->compressor) - 1);
      const LoadedPlugin* pl = codec->plugin();
      if (pl->fusedQuery != nullptr && pl->fusedQuery(codec->config(), ncclDatatype, &out->codec) == 1 &&
          cocclkTileCodecSupported(&out->codec)) {
        out->fusable = 1;
      } else if (info.op == Operation::AllGather && pl->deltaQuery != nullptr &&
                 pl->deltaQuery(codec->config(), ncclDatatype, &out->codec) == 1 && cocclkTileCodecSupported(&out->codec)) {
        out->fusable = 1;
        out->delta = 1;
      }
    }
    return 0;
  }
  // native: a small all-reduce may still prefer the multimem kernel when it was measured faster
  if (info.op == Operation::AllReduce && !r->measuredNative.empty()) {
    const size_t bytes = count * width;
    int lg = 0;
    while ((bytes >> (lg + 1)) != 0) ++lg;
    const std::map<int, double>* best = nullptr;
    for (int d = 0; d < 40 && best == nullptr; ++d) {
      auto it = r->measuredNative.find(MeasuredKey{op, ncclDatatype, nRanks, lg - d});
      if (it != r->measuredNative.end()) best = &it->second;
    }
    if (best != nullptr) {
      double t = 0.0;
      bool first = true;
      for (const auto& kv : *best)
        if (first || kv.second < t) { out->nativeVariant = kv.first; t = kv.second; first = false; }
    }
  }
  return 0;
}

extern "C" int cocclRouterSetMeasured(cocclRouter* r, int op, int ncclDatatype, int nRanks, int log2Bytes, int algorithm, double seconds) {
  if (r == nullptr || algorithm <= 0 || !(seconds > 0.0)) return (int)ncclInvalidArgument;
  std::lock_guard<std::mutex> lock(r->mutex);
  r->measured[MeasuredKey{op, ncclDatatype, nRanks, log2Bytes}][algorithm] = seconds;
  return 0;
}
extern "C" int cocclRouterSetMeasuredNative(cocclRouter* r, int ncclDatatype, int nRanks, int log2Bytes, int nativeVariant, double seconds) {
  if (r == nullptr || !(seconds > 0.0)) return (int)ncclInvalidArgument;
  std::lock_guard<std::mutex> lock(r->mutex);
  r->measuredNative[MeasuredKey{(int)Operation::AllReduce, ncclDatatype, nRanks, log2Bytes}][nativeVariant] = seconds;
  return 0;
}
extern "C" void cocclRouterStats(cocclRouter* r, uint64_t* nativeCalls, uint64_t* compressedCalls, uint64_t* policyLookups) {
  if (r == nullptr) return;
  RouterStats& s = r->rt.stats();
  if (nativeCalls) *nativeCalls = s.nativeCalls;
  if (compressedCalls) *compressedCalls = s.compressedCalls;
  if (policyLookups) *policyLookups = s.policyLookups;
}
