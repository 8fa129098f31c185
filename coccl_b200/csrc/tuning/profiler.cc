// Start-up profiler of the autotuner (see autotune.h).
#include <algorithm>
#include <set>

#include "runtime/log.h"
#include "tuning/autotune.h"

namespace coccl {
namespace {

struct DeviceBuf {
  void* p = nullptr;
  ~DeviceBuf() { if (p) cudaFree(p); }
  bool alloc(size_t n) { return cudaMalloc(&p, n) == cudaSuccess; }
};

// max over ranks of a host double, through a device all-gather on the comm's transport
bool maxOverRanks(Comm* comm, double* v, cudaStream_t s) {
  DeviceBuf mine, all;
  if (!mine.alloc(sizeof(double)) || !all.alloc(sizeof(double) * comm->nRanks)) return false;
  if (cudaMemcpyAsync(mine.p, v, sizeof(double), cudaMemcpyHostToDevice, s) != cudaSuccess) return false;
  if (comm->transport->allGather(comm, mine.p, all.p, sizeof(double), ncclUint8, s) != ncclSuccess) return false;
  std::vector<double> host(comm->nRanks);
  if (cudaMemcpyAsync(host.data(), all.p, sizeof(double) * comm->nRanks, cudaMemcpyDeviceToHost, s) != cudaSuccess) return false;
  if (cudaStreamSynchronize(s) != cudaSuccess) return false;
  *v = *std::max_element(host.begin(), host.end());
  return true;
}
bool minOverRanks(Comm* comm, double* v, cudaStream_t s) {
  double neg = -*v;
  if (!maxOverRanks(comm, &neg, s)) return false;
  *v = -neg;
  return true;
}

struct Timer {
  cudaEvent_t a = nullptr, b = nullptr;
  Timer() { cudaEventCreate(&a); cudaEventCreate(&b); }
  ~Timer() { if (a) cudaEventDestroy(a); if (b) cudaEventDestroy(b); }
};

// Ring exchange with the next/previous peer: one grouped send+recv per iteration.
bool profileP2p(Comm* comm, int next, int prev, const std::vector<size_t>& sizes, int warmup, int iters,
                cudaStream_t s, LinearModel* out) {
  const size_t maxBytes = sizes.back();
  DeviceBuf sendBuf, recvBuf;
  if (!sendBuf.alloc(maxBytes) || !recvBuf.alloc(maxBytes)) return false;
  cudaMemsetAsync(sendBuf.p, 0x3f, maxBytes, s);
  Timer t;
  std::vector<std::pair<double, double>> samples;
  for (size_t bytes : sizes) {
    P2POp ops[2] = {{false, recvBuf.p, bytes, prev}, {true, sendBuf.p, bytes, next}};
    for (int i = 0; i < warmup; ++i)
      if (comm->transport->p2pBatch(comm, ops, 2, s) != ncclSuccess) return false;
    cudaEventRecord(t.a, s);
    for (int i = 0; i < iters; ++i)
      if (comm->transport->p2pBatch(comm, ops, 2, s) != ncclSuccess) return false;
    cudaEventRecord(t.b, s);
    if (cudaEventSynchronize(t.b) != cudaSuccess) return false;
    float ms = 0;
    cudaEventElapsedTime(&ms, t.a, t.b);
    double sec = (double)ms * 1e-3 / iters;
    if (!maxOverRanks(comm, &sec, s)) return false;
    samples.push_back({(double)bytes, sec});
  }
  *out = fitLinear(samples);
  return out->valid;
}

// Compress + decompress round trip of 0x3f-filled fp32 data.
bool profileCodec(Runtime*, Comm* comm, CompressorPolicy* codec, const std::vector<size_t>& sizes, int warmup,
                  int iters, cudaStream_t s, CodecModel* out) {
  const size_t maxBytes = sizes.back();
  size_t bound = 0;
  if (encodedSizeBound(codec, cocclCompressorOperationCompress, maxBytes / 4, 1, ncclFloat32, &bound) != ncclSuccess) return false;
  DeviceBuf raw, enc, back, meta;
  if (!raw.alloc(maxBytes) || !enc.alloc(std::max(bound, maxBytes) + 256) || !back.alloc(maxBytes) || !meta.alloc(256)) return false;
  cudaMemsetAsync(raw.p, 0x3f, maxBytes, s);
  ExecEnv env;
  env.stream = s;
  env.cudaDev = comm->cudaDev;
  env.rank = comm->rank;
  env.nRanks = comm->nRanks;
  env.nodes = comm->nNodes;
  env.devicesPerNode = comm->localRanks;
  const bool framed = codec->has(cocclCompressorCapabilityFramed);
  Timer t;
  std::vector<std::pair<double, double>> samples;
  std::vector<double> ratios;
  for (size_t bytes : sizes) {
    const size_t elems = bytes / 4;
    if (elems == 0) continue;
    size_t cap = 0;
    if (encodedSizeBound(codec, cocclCompressorOperationCompress, elems, 1, ncclFloat32, &cap) != ncclSuccess) return false;
    cocclCompressorView in{raw.p, elems * 4, elems * 4, elems, 1, ncclFloat32, nullptr, 0};
    cocclCompressorView e{enc.p, cap, 0, cap, 1, ncclInt8, framed ? (cocclCompressorFrameMetadata*)meta.p : nullptr, framed ? cap : 0};
    cocclCompressorView o{back.p, elems * 4, 0, elems, 1, ncclFloat32, nullptr, 0};
    auto once = [&]() {
      cocclCompressorView ee = e, oo = o;
      if (compress(codec, in, &ee, env) != ncclSuccess) return false;
      if (decompress(codec, ee, &oo, env) != ncclSuccess) return false;
      if (!framed && ee.bytes > 0) ratios.push_back((double)(elems * 4) / (double)ee.bytes);
      return true;
    };
    for (int i = 0; i < warmup; ++i) if (!once()) return false;
    cudaEventRecord(t.a, s);
    for (int i = 0; i < iters; ++i) if (!once()) return false;
    cudaEventRecord(t.b, s);
    if (cudaEventSynchronize(t.b) != cudaSuccess) return false;
    float ms = 0;
    cudaEventElapsedTime(&ms, t.a, t.b);
    double sec = (double)ms * 1e-3 / iters;
    if (!maxOverRanks(comm, &sec, s)) return false;
    samples.push_back({(double)elems * 4, sec});
  }
  out->roundTrip = fitLinear(samples);
  if (ratios.empty()) ratios.push_back(1.0);
  std::sort(ratios.begin(), ratios.end());
  out->ratio = ratios[ratios.size() / 2];
  return out->valid();
}

}  // namespace

ncclResult_t profileModels(Runtime* rt, Comm* comm, ModelStore* store, cudaStream_t stream) {
  if (rt == nullptr || comm == nullptr || store == nullptr || comm->transport == nullptr) return ncclInvalidArgument;
  const Config& cfg = rt->config();
  if (!cfg.autotune || comm->nRanks <= 1) return ncclSuccess;
  // never profile with more than a quarter of the free memory of the most loaded rank
  size_t freeB = 0, totalB = 0;
  if (cudaMemGetInfo(&freeB, &totalB) != cudaSuccess) return ncclUnhandledCudaError;
  double limit = (double)std::min(cfg.profileMaxBytes, freeB / 4);
  if (!minOverRanks(comm, &limit, stream)) return ncclSystemError;
  const size_t maxBytes = (size_t)limit / 256 * 256;
  if (maxBytes < cfg.profileMinBytes) {
    COCCL_WARN("autotune: not enough free memory to profile; using heuristics");
    return ncclSuccess;
  }
  const std::vector<size_t> sizes = profileSizes(cfg.profileMinBytes, maxBytes);
  const int warm = cfg.autotuneWarmup, iters = cfg.autotuneIterations;

  if (comm->localRanks > 1) {
    const int base = comm->node * comm->localRanks;
    const int next = base + (comm->localRank + 1) % comm->localRanks;
    const int prev = base + (comm->localRank + comm->localRanks - 1) % comm->localRanks;
    LinearModel m;
    if (profileP2p(comm, next, prev, sizes, warm, iters, stream, &m)) store->setP2p(false, m);
    else COCCL_WARN("autotune: intra-node p2p profile failed; using heuristics");
  }
  if (comm->nNodes > 1 && comm->uniform) {
    const int next = ((comm->node + 1) % comm->nNodes) * comm->localRanks + comm->localRank;
    const int prev = ((comm->node + comm->nNodes - 1) % comm->nNodes) * comm->localRanks + comm->localRank;
    LinearModel m;
    if (profileP2p(comm, next, prev, sizes, warm, iters, stream, &m)) store->setP2p(true, m);
    else COCCL_WARN("autotune: inter-node p2p profile failed; using heuristics");
  }
  // every codec that a reduce-scatter or all-reduce policy can select
  std::set<CompressorPolicy*> codecs;
  for (Role role : {Role::Normal, Role::DataParallel, Role::TensorParallel})
    for (Operation op : {Operation::ReduceScatter, Operation::AllReduce})
      for (int s = 0; s < 3; ++s)
        if (CompressorPolicy* c = rt->compressors().resolve(role, Variant::Default, op, (Scope)s)) codecs.insert(c);
  for (CompressorPolicy* c : codecs) {
    CodecModel m;
    if (profileCodec(rt, comm, c, sizes, warm, iters, stream, &m)) {
      store->setCodec(c, m);
      if (comm->rank == 0)
        COCCL_INFO(kLogTuning, "model %s: alpha=%.3g s beta=%.3g s/B ratio=%.2f", c->where().c_str(), m.roundTrip.alpha,
                   m.roundTrip.beta, m.ratio);
    } else {
      COCCL_WARN("autotune: codec profile of %s failed; using heuristics", c->where().c_str());
    }
  }
  return ncclSuccess;
}

}  // namespace coccl
