#include <limits>

#include "runtime/log.h"
#include "runtime/runtime.h"

namespace coccl {

static thread_local bool tlsInternal = false;

struct InternalGuard {
  bool previous;
  InternalGuard() : previous(tlsInternal) { tlsInternal = true; }
  ~InternalGuard() { tlsInternal = previous; }
};

bool Runtime::internalCall() { return tlsInternal; }

const char* algorithmName(Algorithm a) {
  switch (a) {
    case Algorithm::None: return "none";
    case Algorithm::RsOneShot: return "reduce_scatter_oneshot";
    case Algorithm::RsTwoShot: return "reduce_scatter_twoshot";
    case Algorithm::ArOneShot: return "all_reduce_oneshot";
    case Algorithm::ArTwoShot: return "all_reduce_twoshot";
    case Algorithm::ArTripleShot: return "all_reduce_tripleshot";
  }
  return "?";
}

int nodeOfRank(const Comm* comm, int rank) {
  return comm->localRanks > 0 ? rank / comm->localRanks : 0;
}

static Scope flatScope(const CallInfo& info) {
  if (info.op == Operation::SendRecv)
    return nodeOfRank(info.comm, info.peer) == info.comm->node ? Scope::Intra : Scope::Inter;
  return info.comm->nNodes == 1 ? Scope::Intra : Scope::Default;
}

void algorithmScopes(const PreparedCall& p, Algorithm a, bool use[3]) {
  use[0] = use[1] = use[2] = false;
  if (a == Algorithm::RsTwoShot) { use[(int)Scope::Intra] = use[(int)Scope::Inter] = true; return; }
  if (a == Algorithm::ArTripleShot) { use[0] = use[1] = use[2] = true; return; }
  use[(int)flatScope(p.info)] = true;
}

bool algorithmHasCompression(const PreparedCall& p, Algorithm a) {
  bool use[3];
  algorithmScopes(p, a, use);
  for (int s = 0; s < 3; ++s)
    if (use[s] && p.codecs[s] != nullptr) return true;
  return false;
}

bool algorithmSupported(const PreparedCall& p, Algorithm a) {
  if (!algorithmHasCompression(p, a)) return false;
  bool use[3];
  algorithmScopes(p, a, use);
  for (int s = 0; s < 3; ++s)
    if (use[s] && p.codecs[s] != nullptr && !p.datatypeOk[s]) return false;
  return true;
}

namespace {

bool floatingType(ncclDataType_t t) { return t == ncclFloat16 || t == ncclFloat32 || t == ncclBfloat16; }

bool datatypeSupported(ncclDataType_t t, const CompressorPolicy* c) {
  if (floatingType(t)) return true;
  if (t != ncclInt8 && t != ncclInt32 && t != ncclInt64) return false;
  return c->has(cocclCompressorCapabilityBytewiseLossless);
}

bool shapeSupported(const CallInfo& info, const OperationDescriptor& d) {
  if (info.count == 0) return false;
  if (info.op == Operation::SendRecv)
    return info.func == Func::Send ? info.sendbuff != nullptr : (info.func == Func::Recv && info.recvbuff != nullptr);
  if (info.sendbuff == nullptr || info.recvbuff == nullptr) return false;
  return !d.has(kTraitCountDivisibleByRanks) || info.count % (size_t)info.comm->nRanks == 0;
}

bool callSupported(const CallInfo& info, const OperationDescriptor& d) {
  if (info.comm->nRanks <= 1) return false;
  if (d.has(kTraitReduction) && info.redOp != ncclSum) return false;
  return shapeSupported(info, d);
}

bool totalBytes(const CallInfo& info, const OperationDescriptor& d, size_t* bytes) {
  const size_t width = cocclTypeSize(info.datatype);
  if (width == 0 || info.count > std::numeric_limits<size_t>::max() / width) return false;
  size_t v = info.count * width;
  if (d.has(kTraitScaleBytesByRanks)) {
    if (v > std::numeric_limits<size_t>::max() / (size_t)info.comm->nRanks) return false;
    v *= (size_t)info.comm->nRanks;
  }
  *bytes = v;
  return true;
}

bool tunable(Operation op) { return op == Operation::ReduceScatter || op == Operation::AllReduce; }

bool sendRecvForward(const CallInfo& info) {
  return info.func == Func::Send ? info.comm->rank < info.peer : info.comm->rank > info.peer;
}

}  // namespace

Runtime::Runtime() {}
Runtime::~Runtime() { disable(); }

ncclResult_t Runtime::enable(const Config& cfg, int nodes, int devicesPerNode, std::string* error) {
  if (enabled_) disable();  // plugins registered in-process before the first enable are kept
  std::string err;
  if (!compressors_.initialize(cfg, nodes, devicesPerNode, &err)) {
    if (error) *error = err;
    COCCL_WARN("compressor runtime failed to start: %s", err.c_str());
    compressors_.shutdown();
    return ncclInvalidUsage;
  }
  enabled_ = true;
  return ncclSuccess;
}

void Runtime::disable() {
  enabled_ = false;
  compressors_.shutdown();
}

ncclResult_t Runtime::resolveCodecs(PreparedCall* call) {
  const CallInfo& info = call->info;
  Variant v = Variant::Default;
  if (info.op == Operation::SendRecv && call->role == Role::PipelineParallel)
    v = sendRecvForward(info) ? Variant::Forward : Variant::Backward;
  call->policy = PolicyKey{info.op, v, Scope::Default};
  bool any = false;
  for (int s = 0; s < 3; ++s) {
    ++stats_.policyLookups;
    CompressorPolicy* c = compressors_.resolve(call->role, v, info.op, (Scope)s);
    call->codecs[s] = c;
    call->datatypeOk[s] = false;
    if (c == nullptr) continue;
    any = true;
    call->datatypeOk[s] = datatypeSupported(info.datatype, c);
    call->thresholdBytes = c->thresholdBytes();
    COCCL_INFO(kLogRuntime, "route comm=%llu role=%d operation=%s scope=%s compressor=%s", (unsigned long long)info.comm->id,
               (int)call->role, call->desc->name, scopeName((Scope)s), c->plugin()->name.c_str());
  }
  return any ? ncclSuccess : ncclInvalidUsage;
}

ncclResult_t Runtime::enqueueCheck(const CallInfo& info, bool* enqueued) {
  if (enqueued == nullptr) return ncclInvalidArgument;
  *enqueued = false;
  if (!enabled_) return ncclSuccess;
  if (tlsInternal) return ncclSuccess;
  if (info.comm == nullptr) return ncclSuccess;
  const bool training = config().mode == Mode::Training;
  if (training && roles_ != nullptr) roles_->observe(info, groupDepth());

  const OperationDescriptor* d = describe(info.op);
  if (d == nullptr || !callSupported(info, *d)) return routeNativeGrouped(info, enqueued);
  size_t bytes = 0;
  if (!totalBytes(info, *d, &bytes)) return routeNativeGrouped(info, enqueued);

  PreparedCall call;
  call.info = info;
  call.desc = d;
  call.role = Role::Normal;
  if (training) {
    call.role = roles_ != nullptr ? roles_->roleOf(info.comm) : Role::Unknown;
    if (call.role == Role::Unknown) return routeNativeGrouped(info, enqueued);
  }
  if (resolveCodecs(&call) != ncclSuccess) return routeNativeGrouped(info, enqueued);
  if (bytes <= call.thresholdBytes) return routeNativeGrouped(info, enqueued);
  if (tunable(info.op)) {
    if (selector_ == nullptr || selector_->select(this, &call) != ncclSuccess) return routeNativeGrouped(info, enqueued);
  } else if (!algorithmSupported(call, Algorithm::None)) {
    return routeNativeGrouped(info, enqueued);
  }
  ncclResult_t r = groupDepth() > 0 ? (groupEnqueuePrepared(call), ncclSuccess) : executePrepared(call);
  if (r != ncclSuccess) return r;
  *enqueued = true;
  return ncclSuccess;
}

ncclResult_t Runtime::enqueueExplicit(const CallInfo& info, Algorithm algorithm) {
  if (info.comm == nullptr || !enabled_) return ncclInvalidUsage;
  const OperationDescriptor* d = describe(info.op);
  if (d == nullptr || !callSupported(info, *d)) return ncclInvalidUsage;
  PreparedCall call;
  call.info = info;
  call.desc = d;
  call.role = Role::Normal;
  if (config().mode == Mode::Training) {
    call.role = roles_ != nullptr ? roles_->roleOf(info.comm) : Role::Unknown;
    if (call.role == Role::Unknown) return ncclInvalidUsage;
  }
  call.algorithm = algorithm;
  ncclResult_t r = resolveCodecs(&call);
  if (r != ncclSuccess) return r;
  if (algorithm == Algorithm::None && tunable(info.op)) {
    if (selector_ == nullptr) return ncclInvalidUsage;
    if ((r = selector_->select(this, &call)) != ncclSuccess) return r;
  }
  if (!algorithmHasCompression(call, call.algorithm)) return ncclInvalidUsage;
  if (!algorithmSupported(call, call.algorithm)) return replayNative(info);  // datatype the codec cannot take
  if (groupDepth() > 0) {
    groupEnqueuePrepared(call);
    return ncclSuccess;
  }
  return executePrepared(call);
}

ncclResult_t Runtime::replayNative(const CallInfo& info) {
  InternalGuard guard;
  ++stats_.nativeCalls;
  Transport* t = info.comm->transport;
  if (t == nullptr) return ncclInvalidArgument;
  switch (info.op) {
    case Operation::AllGather: return t->allGather(info.comm, info.sendbuff, info.recvbuff, info.count, info.datatype, info.stream);
    case Operation::ReduceScatter: return t->reduceScatter(info.comm, info.sendbuff, info.recvbuff, info.count, info.datatype, info.redOp, info.stream);
    case Operation::AllReduce: return t->allReduce(info.comm, info.sendbuff, info.recvbuff, info.count, info.datatype, info.redOp, info.stream);
    case Operation::AllToAll: return t->allToAll(info.comm, info.sendbuff, info.recvbuff, info.count, info.datatype, info.stream);
    case Operation::SendRecv:
      return info.func == Func::Send ? t->send(info.comm, info.sendbuff, info.count, info.datatype, info.peer, info.stream)
                                     : t->recv(info.comm, info.recvbuff, info.count, info.datatype, info.peer, info.stream);
    default: return ncclInvalidArgument;
  }
}

ncclResult_t Runtime::executePrepared(const PreparedCall& call) {
  if (call.desc == nullptr || !call.anyCodec() || executor_ == nullptr) return ncclInvalidArgument;
  InternalGuard guard;
  ++stats_.compressedCalls;
  return executor_->execute(this, call);
}

ncclResult_t Runtime::commInit(Comm*) { return ncclSuccess; }

ncclResult_t Runtime::commDestroy(Comm* comm) {
  if (comm == nullptr) return ncclSuccess;
  for (Comm** child : {&comm->intra, &comm->inter}) {
    if (*child != nullptr && (*child)->transport != nullptr) (*child)->transport->destroy(*child);
    *child = nullptr;
  }
  return ncclSuccess;
}

ncclResult_t Runtime::hierarchy(Comm* owner, Comm** intra, Comm** inter) {
  if (owner == nullptr || owner->transport == nullptr) return ncclInvalidArgument;
  if (owner->isChild) return ncclInvalidUsage;
  InternalGuard guard;
  if (owner->intra == nullptr) {
    ncclResult_t r = owner->transport->split(owner, owner->rank / owner->localRanks, owner->rank, &owner->intra);
    if (r != ncclSuccess) return r;
    owner->intra->isChild = true;
    owner->intra->nNodes = 1;
    owner->intra->localRanks = owner->intra->nRanks;
    owner->intra->localRank = owner->intra->rank;
    owner->intra->node = 0;
  }
  if (owner->inter == nullptr) {
    ncclResult_t r = owner->transport->split(owner, owner->rank % owner->localRanks, owner->rank, &owner->inter);
    if (r != ncclSuccess) return r;
    owner->inter->isChild = true;
    owner->inter->nNodes = owner->inter->nRanks;
    owner->inter->localRanks = 1;
    owner->inter->localRank = 0;
    owner->inter->node = owner->inter->rank;
  }
  if (intra) *intra = owner->intra;
  if (inter) *inter = owner->inter;
  return ncclSuccess;
}

Runtime& globalRuntime() {
  static Runtime* rt = new Runtime();
  return *rt;
}

}  // namespace coccl
