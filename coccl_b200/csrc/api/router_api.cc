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
#include "tuning/measured.h"

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

}  // namespace

struct cocclRouter {
  std::mutex mutex;
  Runtime rt;
  RecordingExecutor exec;
  FixedRole roles;
  ModelStore models;
  MeasuredTable measured;          // compressed algorithms, written by the front end that timed them
  MeasuredTable measuredNative;    // uncompressed all-reduce variants
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
    // the bucket of the call or the nearest measured one BELOW it: a variant that won at a larger size says nothing
    // about a smaller call
    MeasuredTable::Times best;
    const bool have = r->measuredNative.nearest(op, ncclDatatype, nRanks, count * width, &best, /*belowOnly=*/true);
    if (have) {
      double t = 0.0;
      bool first = true;
      for (const auto& kv : best)
        if (first || kv.second < t) { out->nativeVariant = kv.first; t = kv.second; first = false; }
    }
  }
  return 0;
}

extern "C" int cocclRouterSetMeasured(cocclRouter* r, int op, int ncclDatatype, int nRanks, int log2Bytes, int algorithm, double seconds) {
  if (r == nullptr || algorithm <= 0 || !(seconds > 0.0)) return (int)ncclInvalidArgument;
  std::lock_guard<std::mutex> lock(r->mutex);
  r->measured.set(op, ncclDatatype, nRanks, log2Bytes, algorithm, seconds);
  return 0;
}
extern "C" int cocclRouterSetMeasuredNative(cocclRouter* r, int ncclDatatype, int nRanks, int log2Bytes, int nativeVariant, double seconds) {
  if (r == nullptr || !(seconds > 0.0)) return (int)ncclInvalidArgument;
  std::lock_guard<std::mutex> lock(r->mutex);
  r->measuredNative.set((int)Operation::AllReduce, ncclDatatype, nRanks, log2Bytes, nativeVariant, seconds);
  return 0;
}
extern "C" void cocclRouterStats(cocclRouter* r, uint64_t* nativeCalls, uint64_t* compressedCalls, uint64_t* policyLookups) {
  if (r == nullptr) return;
  RouterStats& s = r->rt.stats();
  if (nativeCalls) *nativeCalls = s.nativeCalls;
  if (compressedCalls) *compressedCalls = s.compressedCalls;
  if (policyLookups) *policyLookups = s.policyLookups;
}
