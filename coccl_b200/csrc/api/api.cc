// Implementation of the public C API (include/coccl/coccl.h).
// Every collective builds a CallInfo and asks the router first; when the router does not take the
// call it runs on the native transport (the hook points the reference adds to NCCL's collectives,
// src/collectives.cc:17-28,49-61,141-153,187-198,211-222,233-243, and to group end, src/group.cc:103-116).
#include <algorithm>
#include <mutex>
#include <string>
#include <vector>

#include "coccl/coccl.h"
#include "memory/buffer_manager.h"
#include "runtime/log.h"
#include "runtime/nccl_transport.h"
#include "runtime/primitives.h"
#include "runtime/runtime.h"
#include "runtime/peer_exchange.h"
#include "training/assist.h"
#include "tuning/autotune.h"
#include "tuning/fused_timer.h"
#include "tuning/measured.h"

using namespace coccl;

namespace {

struct ApiState {
  std::mutex mutex;
  bool started = false;
  BufferManager* buffers = nullptr;
  FusedExecutor* executor = nullptr;
  ModelStore models;
  MeasuredTable measured;
  FusedTimer* timer = nullptr;
  MeasuredSelector* selector = nullptr;
  TrainingAssist* assist = nullptr;
  int comms = 0;
};
ApiState& state() {
  static ApiState* s = new ApiState();
  return *s;
}

thread_local int tlsNativeInGroup = 0;  // native calls issued inside the current group
thread_local std::string tlsLastError;

Comm* unwrap(ncclComm_t c) { return reinterpret_cast<Comm*>(c); }
// A handle that does not start with this library's magic word belongs to the native library (runtime/comm.h).
bool foreign(ncclComm_t c) { return c != nullptr && unwrap(c)->magic != kCommMagic; }

// cocclInit: runs once per process when the first communicator is created; later communicators
// only register themselves (core/runtime/coccl_init.cc:17-31).
ncclResult_t runtimeStart(Comm* comm) {
  ApiState& s = state();
  std::lock_guard<std::mutex> lock(s.mutex);
  Runtime& rt = globalRuntime();
  if (!s.started) {
    s.started = true;
    const ProcessConfig& pc = processConfig();
    if (pc.enabled) {
      std::string err;
      if (rt.enable(pc.config, comm->nNodes, comm->localRanks, &err) != ncclSuccess) {
        COCCL_WARN("COCCL disabled for this process: %s", err.c_str());
      } else {
        if (logEnabled(kLevelInfo, kLogInit)) {
          std::string text = formatConfig(pc.config);
          COCCL_INFO(kLogInit, "effective configuration:\n%s", text.c_str());
        }
        BufferOptions bo;
        bo.legacyBlockBytes = pc.config.legacyBlockBytes;
        bo.physicalChunkBytes = pc.config.physicalChunkBytes;
        bo.poolLimitBytes = pc.config.poolLimitBytes;
        bo.vmm = cudaVmmDriverApi();
        s.buffers = new BufferManager(bo);
        s.executor = new FusedExecutor(s.buffers);
        // measured one-shot / two-shot times of the fused kernels first, the cost model and heuristics behind them
        s.timer = new FusedTimer(s.executor);
        s.selector = new MeasuredSelector(&s.models, &s.measured, s.timer);
        rt.setExecutor(s.executor);
        rt.setSelector(s.selector);
        if (pc.config.mode == Mode::Training) {
          s.assist = new TrainingAssist(ClassifierParams::from(pc.config), pc.config.observationIterations);
          rt.setRoleOracle(s.assist);
        }
      }
    }
  }
  ++s.comms;
  if (!rt.enabled()) return ncclSuccess;
  rt.commInit(comm);
  if (s.buffers) s.buffers->commInit(comm);
  if (s.assist) s.assist->registerComm(comm);
  return ncclSuccess;
}

void runtimeStop(Comm* comm) {
  ApiState& s = state();
  std::lock_guard<std::mutex> lock(s.mutex);
  Runtime& rt = globalRuntime();
  if (rt.enabled()) {
    if (s.executor) s.executor->releaseComm(comm);
    if (s.timer) s.timer->release(comm);
    PeerDataPath::release(comm);
    for (Comm* child : {comm->intra, comm->inter}) if (child != nullptr) PeerDataPath::release(child);
    if (s.assist) s.assist->unregisterComm(comm);
    rt.commDestroy(comm);
    if (s.buffers) s.buffers->commDestroy(comm);
  }
  if (--s.comms == 0 && rt.enabled()) destroyPipelineResources();
}

ncclResult_t route(CallInfo info) {
  if (info.comm == nullptr || info.comm->magic != kCommMagic) return ncclInvalidArgument;
  Runtime& rt = globalRuntime();
  bool taken = false;
  ncclResult_t r = rt.enqueueCheck(info, &taken);
  if (r != ncclSuccess) return r;
  if (taken) return ncclSuccess;
  if (rt.groupDepth() > 0) ++tlsNativeInGroup;
  return rt.replayNative(info);
}

CallInfo makeInfo(Operation op, Func f, const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t red, int peer, ncclComm_t c, cudaStream_t st) {
  CallInfo i;
  i.op = op; i.func = f; i.sendbuff = s; i.recvbuff = r; i.count = n; i.datatype = t; i.redOp = red; i.peer = peer;
  i.comm = unwrap(c); i.stream = st;
  return i;
}

ncclResult_t explicitCall(CallInfo info, Algorithm a) {
  if (info.comm == nullptr || info.comm->magic != kCommMagic) return ncclInvalidArgument;
  return globalRuntime().enqueueExplicit(info, a);
}

}  // namespace

extern "C" {

ncclResult_t cocclApiGetUniqueId(ncclUniqueId* id) { return ncclTransport().uniqueId(id); }

ncclResult_t cocclApiCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank) {
  if (comm == nullptr) return ncclInvalidArgument;
  Comm* c = nullptr;
  ncclResult_t r = ncclTransport().initRank(&c, nranks, id, rank);
  if (r != ncclSuccess) return r;
  runtimeStart(c);
  // measured models for the algorithm selector (collective: every rank is here)
  Runtime& rt = globalRuntime();
  if (rt.enabled() && rt.config().autotune && nranks > 1) {
    cudaStream_t s = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) == cudaSuccess) {
      if (profileModels(&rt, c, &state().models, s) != ncclSuccess)
        COCCL_WARN("autotune profiling failed; algorithm selection uses heuristics");
      cudaStreamDestroy(s);
    }
  }
  *comm = reinterpret_cast<ncclComm_t>(c);
  return ncclSuccess;
}

// ncclCommInitRankConfig: the configuration of NCCL 2.21 (blocking mode, CGA cluster size, CTA limits, network name,
// split sharing; src/nccl.h.in:84-120) tunes NCCL's own kernels; the communicator here is always created blocking.
ncclResult_t cocclApiCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, void* /*config*/) {
  return cocclApiCommInitRank(comm, nranks, id, rank);
}

// ncclCommInitAll: one process, one thread, ndev communicators (src/init.cc:1846 of the reference). The collective
// start-up measurements of the autotuner need every rank to run at once, which a single thread cannot do: the
// communicators created here select algorithms by heuristics (or by what the policy file forces).
ncclResult_t cocclApiCommInitAll(ncclComm_t* comms, int ndev, const int* devlist) {
  if (comms == nullptr || ndev <= 0) return ncclInvalidArgument;
  ncclUniqueId id;
  ncclResult_t r = ncclTransport().uniqueId(&id);
  if (r != ncclSuccess) return r;
  int previous = 0;
  cudaGetDevice(&previous);
  std::vector<Comm*> made((size_t)ndev, nullptr);
  r = ncclTransport().groupStart();
  for (int i = 0; i < ndev && r == ncclSuccess; ++i) {
    if (cudaSetDevice(devlist ? devlist[i] : i) != cudaSuccess) { r = ncclUnhandledCudaError; break; }
    r = ncclTransport().initRank(&made[(size_t)i], ndev, id, i);
  }
  ncclResult_t e = ncclTransport().groupEnd();
  if (r == ncclSuccess) r = e;
  for (int i = 0; i < ndev; ++i) {
    if (made[(size_t)i] == nullptr) continue;
    if (r == ncclSuccess) {
      runtimeStart(made[(size_t)i]);
      comms[i] = reinterpret_cast<ncclComm_t>(made[(size_t)i]);
    } else {
      ncclTransport().destroy(made[(size_t)i]);
    }
  }
  cudaSetDevice(previous);
  return r;
}

ncclResult_t cocclApiGetVersion(int* version) { return ncclTransport().version(version); }
ncclResult_t cocclApiMemAlloc(void** ptr, size_t size) { return ncclTransport().memAlloc(ptr, size); }
ncclResult_t cocclApiMemFree(void* ptr) { return ncclTransport().memFree(ptr); }
ncclResult_t cocclApiCommRegister(ncclComm_t comm, void* buff, size_t size, void** handle) {
  if (!comm) return ncclInvalidArgument;
  return ncclTransport().commRegister(unwrap(comm), buff, size, handle);
}
ncclResult_t cocclApiCommDeregister(ncclComm_t comm, void* handle) {
  if (!comm) return ncclInvalidArgument;
  return ncclTransport().commDeregister(unwrap(comm), handle);
}
// A pre-multiplied sum is not the plain sum the codecs reduce: calls that use it are left native by the router
// (rule "sum only", coccl_runtime.cc:159-167); the operator itself lives in the native library.
ncclResult_t cocclApiRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t datatype, int residence, ncclComm_t comm) {
  if (!comm || !op) return ncclInvalidArgument;
  return ncclTransport().redOpCreatePreMulSum(op, scalar, datatype, residence, unwrap(comm));
}
ncclResult_t cocclApiRedOpDestroy(ncclRedOp_t op, ncclComm_t comm) {
  if (!comm) return ncclInvalidArgument;
  return ncclTransport().redOpDestroy(op, unwrap(comm));
}

ncclResult_t cocclApiCommDestroy(ncclComm_t comm) {
  Comm* c = unwrap(comm);
  if (c == nullptr) return ncclSuccess;
  runtimeStop(c);
  c->transport->destroy(c);
  return ncclSuccess;
}
ncclResult_t cocclApiCommFinalize(ncclComm_t comm) {
  Comm* c = unwrap(comm);
  if (c == nullptr) return ncclInvalidArgument;
  return cudaDeviceSynchronize() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}
ncclResult_t cocclApiCommAbort(ncclComm_t comm) {
  Comm* c = unwrap(comm);
  if (c == nullptr) return ncclSuccess;
  runtimeStop(c);
  return ncclTransport().abort(c);
}
ncclResult_t cocclApiCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, void*) {
  Comm* c = unwrap(comm);
  if (c == nullptr || newcomm == nullptr) return ncclInvalidArgument;
  Comm* child = nullptr;
  ncclResult_t r = c->transport->split(c, color, key, &child);
  if (r != ncclSuccess) return r;
  runtimeStart(child);
  *newcomm = reinterpret_cast<ncclComm_t>(child);
  return ncclSuccess;
}
ncclResult_t cocclApiCommCount(ncclComm_t comm, int* n) {
  if (!comm || !n) return ncclInvalidArgument;
  if (foreign(comm)) return ncclTransport().foreignCount(comm, n);
  *n = unwrap(comm)->nRanks;
  return ncclSuccess;
}
ncclResult_t cocclApiCommUserRank(ncclComm_t comm, int* r) {
  if (!comm || !r) return ncclInvalidArgument;
  if (foreign(comm)) return ncclTransport().foreignUserRank(comm, r);
  *r = unwrap(comm)->rank;
  return ncclSuccess;
}
ncclResult_t cocclApiCommCuDevice(ncclComm_t comm, int* d) {
  if (!comm || !d || foreign(comm)) return ncclInvalidArgument;
  *d = unwrap(comm)->cudaDev;
  return ncclSuccess;
}
ncclResult_t cocclApiCommGetAsyncError(ncclComm_t comm, ncclResult_t* e) {
  if (!comm || !e) return ncclInvalidArgument;
  if (foreign(comm)) return ncclTransport().foreignAsyncError(comm, e);
  // a fused kernel whose wait on a peer ran out reports here as a remote error (the reference inherits NCCL's
  // abort flag polling for this, src/device/prims_simple.h:97-132 and src/init.cc:2286)
  if (state().executor != nullptr) {
    unsigned int w = state().executor->asyncStatus(unwrap(comm));
    if (w == 0) w = PeerDataPath::asyncStatusOf(unwrap(comm));
    if (w != 0) {
      COCCL_WARN("comm %llu: a fused collective gave up waiting (phase %u, peer %u, slice %u)", (unsigned long long)unwrap(comm)->id,
                 (w >> 23) & 0xffu, (w >> 15) & 0xffu, w & 0x7fffu);
      *e = ncclRemoteError;
      return ncclSuccess;
    }
  }
  return ncclTransport().asyncError(unwrap(comm), e);
}
const char* cocclApiGetErrorString(ncclResult_t r) { return ncclTransport().errorString(r); }
const char* cocclApiGetLastError(ncclComm_t) { return lastWarning(); }

ncclResult_t cocclApiAllReduce(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  return route(makeInfo(Operation::AllReduce, Func::Collective, s, r, n, t, op, -1, c, st));
}
ncclResult_t cocclApiReduceScatter(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  return route(makeInfo(Operation::ReduceScatter, Func::Collective, s, r, n, t, op, -1, c, st));
}
ncclResult_t cocclApiAllGather(const void* s, void* r, size_t n, ncclDataType_t t, ncclComm_t c, cudaStream_t st) {
  return route(makeInfo(Operation::AllGather, Func::Collective, s, r, n, t, ncclSum, -1, c, st));
}
ncclResult_t cocclApiAllToAll(const void* s, void* r, size_t n, ncclDataType_t t, ncclComm_t c, cudaStream_t st) {
  return route(makeInfo(Operation::AllToAll, Func::Collective, s, r, n, t, ncclSum, -1, c, st));
}
ncclResult_t cocclApiSend(const void* s, size_t n, ncclDataType_t t, int peer, ncclComm_t c, cudaStream_t st) {
  return route(makeInfo(Operation::SendRecv, Func::Send, s, nullptr, n, t, ncclSum, peer, c, st));
}
ncclResult_t cocclApiRecv(void* r, size_t n, ncclDataType_t t, int peer, ncclComm_t c, cudaStream_t st) {
  return route(makeInfo(Operation::SendRecv, Func::Recv, nullptr, r, n, t, ncclSum, peer, c, st));
}
ncclResult_t cocclApiBroadcast(const void* s, void* r, size_t n, ncclDataType_t t, int root, ncclComm_t c, cudaStream_t st) {
  if (!c) return ncclInvalidArgument;
  if (globalRuntime().groupDepth() > 0) ++tlsNativeInGroup;
  return ncclTransport().broadcast(unwrap(c), s, r, n, t, root, st);
}
// ncclBcast: the in-place form of ncclBroadcast
ncclResult_t cocclApiBcast(void* buff, size_t n, ncclDataType_t t, int root, ncclComm_t c, cudaStream_t st) {
  return cocclApiBroadcast(buff, buff, n, t, root, c, st);
}
ncclResult_t cocclApiReduce(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, int root, ncclComm_t c, cudaStream_t st) {
  if (!c) return ncclInvalidArgument;
  if (globalRuntime().groupDepth() > 0) ++tlsNativeInGroup;
  return ncclTransport().reduce(unwrap(c), s, r, n, t, op, root, st);
}

ncclResult_t cocclApiGroupStart(void) {
  Runtime& rt = globalRuntime();
  if (rt.groupDepth() == 0) tlsNativeInGroup = 0;
  rt.groupStart();
  return ncclTransport().groupStart();
}
ncclResult_t cocclApiGroupEnd(void) {
  Runtime& rt = globalRuntime();
  const bool nativePending = tlsNativeInGroup > 0;
  ncclResult_t r = rt.groupEnd(&ncclTransport(), nativePending);
  if (rt.groupDepth() == 0) tlsNativeInGroup = 0;
  return r;
}

ncclResult_t cocclAllReduceCompOneShot(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  return explicitCall(makeInfo(Operation::AllReduce, Func::Collective, s, r, n, t, op, -1, c, st), Algorithm::ArOneShot);
}
ncclResult_t cocclAllReduceCompTwoShot(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  return explicitCall(makeInfo(Operation::AllReduce, Func::Collective, s, r, n, t, op, -1, c, st), Algorithm::ArTwoShot);
}
ncclResult_t cocclAllReduceCompTripleShot(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  return explicitCall(makeInfo(Operation::AllReduce, Func::Collective, s, r, n, t, op, -1, c, st), Algorithm::ArTripleShot);
}
ncclResult_t cocclReduceScatterCompOneShot(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  return explicitCall(makeInfo(Operation::ReduceScatter, Func::Collective, s, r, n, t, op, -1, c, st), Algorithm::RsOneShot);
}
ncclResult_t cocclReduceScatterCompTwoShot(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  return explicitCall(makeInfo(Operation::ReduceScatter, Func::Collective, s, r, n, t, op, -1, c, st), Algorithm::RsTwoShot);
}
ncclResult_t cocclAllGatherComp(const void* s, void* r, size_t n, ncclDataType_t t, ncclComm_t c, cudaStream_t st) {
  return explicitCall(makeInfo(Operation::AllGather, Func::Collective, s, r, n, t, ncclSum, -1, c, st), Algorithm::None);
}
ncclResult_t cocclAllToAllComp(const void* s, void* r, size_t n, ncclDataType_t t, ncclComm_t c, cudaStream_t st) {
  return explicitCall(makeInfo(Operation::AllToAll, Func::Collective, s, r, n, t, ncclSum, -1, c, st), Algorithm::None);
}
ncclResult_t cocclSendComp(const void* s, size_t n, ncclDataType_t t, int peer, ncclComm_t c, cudaStream_t st) {
  return explicitCall(makeInfo(Operation::SendRecv, Func::Send, s, nullptr, n, t, ncclSum, peer, c, st), Algorithm::None);
}
ncclResult_t cocclRecvDecomp(void* r, size_t n, ncclDataType_t t, int peer, ncclComm_t c, cudaStream_t st) {
  return explicitCall(makeInfo(Operation::SendRecv, Func::Recv, nullptr, r, n, t, ncclSum, peer, c, st), Algorithm::None);
}

void cocclApiGetStats(cocclApiStats* out) {
  if (out == nullptr) return;
  RouterStats& s = globalRuntime().stats();
  out->nativeCalls = s.nativeCalls;
  out->compressedCalls = s.compressedCalls;
  out->deferredCalls = s.deferredCalls;
  out->policyLookups = s.policyLookups;
  out->fusedCalls = state().executor ? state().executor->fusedCalls.load() : 0;
  out->stagedCalls = state().executor ? state().executor->stagedCalls.load() : 0;
}

void cocclApiStagedReasons(unsigned long long* noFusedForm, unsigned long long* afterFailedSetup, unsigned long long* setupFailed) {
  FusedExecutor* e = state().executor;
  if (noFusedForm) *noFusedForm = e ? e->stagedNoFusedForm.load() : 0;
  if (afterFailedSetup) *afterFailedSetup = e ? e->stagedAfterFailedSetup.load() : 0;
  if (setupFailed) *setupFailed = e ? e->stagedSetupFailed.load() : 0;
}

unsigned long long cocclApiPeerExchangeCalls(void) { return (unsigned long long)PeerDataPath::calls(); }

void cocclApiMeasuredSelection(unsigned long long* bucketsTimed, unsigned long long* bucketsInTable) {
  ApiState& s = state();
  std::lock_guard<std::mutex> lock(s.mutex);
  if (bucketsTimed) *bucketsTimed = s.selector ? s.selector->measuredBuckets() : 0;
  if (bucketsInTable) *bucketsInTable = (unsigned long long)s.measured.size();
}

ncclResult_t cocclApiCommTrainingRole(ncclComm_t comm, cocclApiTrainingRole* out) {
  if (comm == nullptr || out == nullptr) return ncclInvalidArgument;
  *out = cocclApiTrainingRole{};
  ApiState& s = state();
  std::lock_guard<std::mutex> lock(s.mutex);
  if (s.assist == nullptr) return ncclInvalidUsage;
  Comm* c = unwrap(comm);
  Classification k;
  uint64_t activation = 0;
  if (!s.assist->query(c, &k, &activation)) return ncclSuccess;  // nothing decided yet
  out->role = (int)k.role;
  out->candidate = (int)k.candidate;
  out->committed = 1;
  out->active = s.assist->roleOf(c) == k.role && k.role != Role::Unknown ? 1 : 0;
  out->confidence = k.confidence;
  out->callsPerIteration = k.callsPerIteration;
  out->agToRsRatio = k.agToRsRatio;
  out->observedCalls = k.observedCalls;
  out->activationCall = activation;
  return ncclSuccess;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Single-process codec harness: load one plugin, parse its options, and run
// compress -> (decompressReduce | decompress) through the same glue the pipeline uses.
// options: "key=value,key=value". Returns the encoded size through *encodedBytes.
extern "C" ncclResult_t cocclApiCodecRoundTrip(const char* pluginDir, const char* name, const char* options,
                                               const void* in, void* out, size_t elements, size_t chunks, int ncclDatatype,
                                               size_t reduceChunks, int rounds, size_t* encodedBytes, cudaStream_t stream) {
  if (!pluginDir || !name || !in || !out || chunks == 0 || elements % chunks != 0) return ncclInvalidArgument;
  Config cfg;
  cfg.mode = Mode::Normal;
  cfg.compressors = {name};
  cfg.libraryPath = pluginDir;
  ScopeEntry& e = cfg.slots[(size_t)PolicyId::NormalAllGather].scopes[0];
  e.configured = e.enabled = true;
  e.compressor = name;
  std::string opts = options ? options : "";
  size_t pos = 0;
  while (pos < opts.size()) {
    size_t comma = opts.find(',', pos);
    std::string kv = opts.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos);
    size_t eq = kv.find('=');
    if (eq != std::string::npos) e.options[kv.substr(0, eq)] = kv.substr(eq + 1);
    if (comma == std::string::npos) break;
    pos = comma + 1;
  }
  CompressorRuntime rt;
  std::string err;
  if (!rt.initialize(cfg, 1, 1, &err)) {
    COCCL_WARN("codec harness: %s", err.c_str());
    return ncclInvalidUsage;
  }
  CompressorPolicy* codec = rt.resolve(Role::Normal, Variant::Default, Operation::AllGather, Scope::Default);
  if (codec == nullptr) return ncclInvalidUsage;
  const ncclDataType_t dt = (ncclDataType_t)ncclDatatype;
  const size_t width = cocclTypeSize(dt);
  size_t bound = 0;
  ncclResult_t r = encodedSizeBound(codec, cocclCompressorOperationCompress, elements, chunks, dt, &bound);
  if (r != ncclSuccess) return r;
  const bool framed = codec->has(cocclCompressorCapabilityFramed);
  const size_t cap = std::max(bound, elements * width);
  void* enc = nullptr;
  void* meta = nullptr;
  if (cudaMalloc(&enc, cap + 256) != cudaSuccess || cudaMalloc(&meta, chunks * 16 + 256) != cudaSuccess) return ncclUnhandledCudaError;
  ExecEnv env;
  env.stream = stream;
  cudaGetDevice(&env.cudaDev);
  const size_t red = reduceChunks ? reduceChunks : 1;
  for (int round = 0; round < (rounds > 0 ? rounds : 1) && r == ncclSuccess; ++round) {
    cocclCompressorView iv{const_cast<void*>(in), elements * width, elements * width, elements, chunks, dt, nullptr, 0};
    cocclCompressorView ev{enc, cap, 0, cap, chunks, ncclInt8, framed ? (cocclCompressorFrameMetadata*)meta : nullptr, framed ? bound / chunks : 0};
    r = compress(codec, iv, &ev, env);
    if (r != ncclSuccess) break;
    if (encodedBytes) *encodedBytes = ev.bytes;
    cocclCompressorView ov{out, elements / red * width, 0, elements / red, chunks / red, dt, nullptr, 0};
    r = red > 1 ? decompressReduce(codec, ev, &ov, red, env) : decompress(codec, ev, &ov, env);
  }
  if (cudaStreamSynchronize(stream) != cudaSuccess && r == ncclSuccess) r = ncclUnhandledCudaError;
  if (r == ncclSuccess && framed && encodedBytes) {
    // a framed codec reserves fixed slots; what it actually produced is in the frame metadata
    std::vector<cocclCompressorFrameMetadata> hm(chunks);
    if (cudaMemcpy(hm.data(), meta, chunks * sizeof(cocclCompressorFrameMetadata), cudaMemcpyDeviceToHost) == cudaSuccess) {
      size_t total = 0;
      for (const auto& m : hm) total += (size_t)m.payloadBytes;
      *encodedBytes = total;
    }
  }
  cudaFree(enc);
  cudaFree(meta);
  return r;
}
