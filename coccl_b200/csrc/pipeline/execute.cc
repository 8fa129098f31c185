#include <string.h>
#include <mutex>

#include "kernels/kernels_api.h"
#include "pipeline/pipeline.h"
#include "runtime/log.h"
#include "runtime/peer_exchange.h"

namespace coccl {

// ------------------------------------------------------------------ frame exchange
bool frameMetadataValid(const cocclCompressorFrameMetadata& m, size_t strideBytes) {
  return m.payloadBytes > 0 && m.payloadBytes <= strideBytes &&
         (m.encoding == cocclCompressorFrameEncoded || m.encoding == cocclCompressorFrameRaw);
}

ncclResult_t buildFrameExchange(bool allGather, int rank, int nRanks, size_t framesPerRank, size_t stride,
                                const cocclCompressorFrameMetadata* sendMeta, const cocclCompressorFrameMetadata* recvMeta,
                                std::vector<FrameTransfer>* sends, std::vector<FrameTransfer>* recvs) {
  sends->clear();
  recvs->clear();
  if (nRanks <= 0 || framesPerRank == 0 || stride == 0) return ncclInvalidArgument;
  // all-to-all: my frames [p*f, (p+1)*f) go to rank p and land in its slots [rank*f, ...);
  // all-gather: my f frames go to everyone and land in slots [rank*f, ...).
  const size_t sendFrames = allGather ? framesPerRank : framesPerRank * (size_t)nRanks;
  for (size_t i = 0; i < sendFrames; ++i)
    if (!frameMetadataValid(sendMeta[i], stride)) return ncclInvalidUsage;
  for (size_t i = 0; i < framesPerRank * (size_t)nRanks; ++i)
    if (!frameMetadataValid(recvMeta[i], stride)) return ncclInvalidUsage;
  for (int p = 0; p < nRanks; ++p) {
    for (size_t f = 0; f < framesPerRank; ++f) {
      const size_t sendSlot = allGather ? f : (size_t)p * framesPerRank + f;
      const size_t recvSlot = (size_t)p * framesPerRank + f;
      sends->push_back({p, sendSlot * stride, (size_t)sendMeta[sendSlot].payloadBytes, 0, 0});
      recvs->push_back({p, 0, 0, recvSlot * stride, (size_t)recvMeta[recvSlot].payloadBytes});
    }
  }
  (void)rank;
  return ncclSuccess;
}

// ------------------------------------------------------------------ edges and stage handlers
namespace {

struct Edge {
  void* ptr = nullptr;
  size_t capacity = 0, bytes = 0, elements = 0, chunks = 0;
  ncclDataType_t datatype = ncclInt8;
  CompressorPolicy* codec = nullptr;
  cocclCompressorFrameMetadata* meta = nullptr;
  size_t frameStride = 0;
  cocclCompressorView view() const { return {ptr, capacity, bytes, elements, chunks, datatype, meta, frameStride}; }
};

bool overlaps(const void* a, size_t an, const void* b, size_t bn) {
  const char* x = static_cast<const char*>(a);
  const char* y = static_cast<const char*>(b);
  return x < y + bn && y < x + an;
}

struct SliceCtx {
  const PipelineSpec* spec;
  const PipelinePlan* plan;
  const PipelineRuntime* rt;
  size_t sliceIndex;
  SliceShape shape;
  char* arena;     // this slice's registered arena
  char* ringSlot;  // this slice's raw ring slot (split mode) or null
  Edge edge;       // current edge, mutated stage by stage
};

ExecEnv envFor(const SliceCtx& c, cudaStream_t s) {
  ExecEnv e;
  Comm* o = c.spec->ownerComm;
  e.stream = s;
  e.cudaDev = o->cudaDev;
  e.rank = o->rank;
  e.nRanks = o->nRanks;
  e.nodes = o->nNodes;
  e.devicesPerNode = o->localRanks;
  e.alloc = c.rt->alloc;
  return e;
}

// Where a stage writes: its temp, or the user's output for the last stage.
void outputFor(const SliceCtx& c, const StagePlan& p, bool last, Edge* out) {
  const size_t width = cocclTypeSize(c.spec->datatype);
  *out = Edge();
  if (last) {
    // without output staging the final edge is one chunk (or the whole unsliced message)
    out->ptr = static_cast<char*>(c.spec->output) + c.shape.offsetElems * width;
    out->capacity = p.outBoundBytes;
  } else {
    char* base = p.inRawRing ? c.ringSlot : c.arena;
    out->ptr = base + p.tempOffset;
    out->capacity = p.outBoundBytes;
    if (p.framed) {
      out->meta = reinterpret_cast<cocclCompressorFrameMetadata*>(base + p.tempOffset + p.metaOffset);
      out->frameStride = p.frameStrideBytes;
    }
  }
  out->chunks = p.outChunks;
  if (p.outEncoded) {
    out->datatype = ncclInt8;
    out->elements = p.outBoundBytes;
    out->codec = p.edgeCodec;
  } else {
    out->datatype = c.spec->datatype;
    out->elements = p.outChunks * p.outElemsPerChunk;
    out->bytes = out->elements * width;
  }
}

ncclResult_t toResult(int rc) { return rc == 0 ? ncclSuccess : (rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError); }

// Host copy of a device metadata array (framed codecs): needs the stream to be drained first.
ncclResult_t readMetadata(const cocclCompressorFrameMetadata* dev, size_t n, cudaStream_t s,
                          std::vector<cocclCompressorFrameMetadata>* host) {
  host->resize(n);
  if (cudaMemcpyAsync(host->data(), dev, n * sizeof(cocclCompressorFrameMetadata), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return ncclUnhandledCudaError;
  return cudaStreamSynchronize(s) == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}

ncclResult_t exchangeFramed(SliceCtx& c, const Stage& st, const StagePlan& p, Edge& in, Edge& out, cudaStream_t s) {
  Comm* comm = st.comm;
  const bool gather = st.kind == StageKind::AllGather;
  const int n = comm->nRanks;
  const size_t framesPerRank = gather ? in.chunks : in.chunks / (size_t)n;
  // one node: the kernel reads the sizes on the device and stores the frames into the receivers' memory; no host
  // round trip, no library collective
  if (PeerDataPath::serves(framesPerRank, in.frameStride)) {
    if (PeerDataPath* path = PeerDataPath::of(comm, s)) {
      ncclResult_t pr = path->exchange(gather, in.ptr, out.ptr, framesPerRank, in.frameStride, in.meta, out.meta, s);
      if (pr != ncclSuccess) return pr;
      out.bytes = p.outChunks * in.frameStride;
      out.elements = out.bytes;
      out.frameStride = in.frameStride;
      out.datatype = in.datatype;
      return ncclSuccess;
    }
  }
  // 1. metadata travels first, as ordinary fixed-size bytes
  ncclResult_t r = gather
      ? comm->transport->allGather(comm, in.meta, out.meta, in.chunks * kFrameMetaBytes, ncclUint8, s)
      : comm->transport->allToAll(comm, in.meta, out.meta, framesPerRank * kFrameMetaBytes, ncclUint8, s);
  if (r != ncclSuccess) return r;
  // 2. the host learns the real payload sizes
  std::vector<cocclCompressorFrameMetadata> sendMeta, recvMeta;
  if ((r = readMetadata(in.meta, in.chunks, s, &sendMeta)) != ncclSuccess) return r;
  if ((r = readMetadata(out.meta, p.outChunks, s, &recvMeta)) != ncclSuccess) return r;
  std::vector<FrameTransfer> sends, recvs;
  r = buildFrameExchange(gather, comm->rank, n, framesPerRank, in.frameStride, sendMeta.data(), recvMeta.data(), &sends, &recvs);
  if (r != ncclSuccess) return r;
  // 3. one grouped exchange of exactly the bytes that exist
  std::vector<P2POp> ops;
  for (const FrameTransfer& t : recvs) ops.push_back({false, static_cast<char*>(out.ptr) + t.recvOffset, t.recvBytes, t.peer});
  for (const FrameTransfer& t : sends) ops.push_back({true, static_cast<char*>(in.ptr) + t.sendOffset, t.sendBytes, t.peer});
  r = comm->transport->p2pBatch(comm, ops.data(), (int)ops.size(), s);
  if (r != ncclSuccess) return r;
  out.bytes = p.outChunks * in.frameStride;
  out.elements = out.bytes;
  out.frameStride = in.frameStride;
  out.datatype = in.datatype;
  return ncclSuccess;
}

ncclResult_t runStage(SliceCtx& c, size_t planIndex, const StagePlan& p, bool last, cudaStream_t s) {
  const PipelineSpec& spec = *c.spec;
  const size_t width = cocclTypeSize(spec.datatype);
  Edge out;
  outputFor(c, p, last, &out);
  Edge& in = c.edge;
  if (p.kind != StageKind::Pack && p.kind != StageKind::Unpack && in.ptr != nullptr && out.ptr != nullptr &&
      in.ptr != out.ptr && overlaps(in.ptr, in.bytes, out.ptr, out.capacity) && in.ptr != spec.input)
    return ncclInvalidUsage;  // a stage may not write over the bytes it is reading
  const bool staged = c.plan->stageInput;
  const Stage* st = nullptr;
  if (p.kind != StageKind::Pack && p.kind != StageKind::Unpack) st = &spec.stages[planIndex - (staged ? 1 : 0)];
  ExecEnv env = envFor(c, s);
  ncclResult_t r = ncclSuccess;
  switch (p.kind) {
    case StageKind::Pack: {
      Comm* o = spec.ownerComm;
      r = toResult(cocclkPackSlice(spec.input, out.ptr, c.shape.elems * width, spec.rawChunkCount * width,
                                   c.shape.offsetElems * width, (int)spec.inputChunks,
                                   c.plan->swizzle ? o->localRanks : 0, o->nNodes, 0, s));
      break;
    }
    case StageKind::Unpack:
      r = toResult(cocclkPackSlice(in.ptr, spec.output, c.shape.elems * width, spec.rawChunkCount * width,
                                   c.shape.offsetElems * width, (int)p.inChunks, 0, 1, 1, s));
      break;
    case StageKind::Compress: {
      cocclCompressorView ov = out.view();
      r = compress(st->codec, in.view(), &ov, env);
      out.bytes = ov.bytes; out.elements = ov.elements; out.chunks = ov.chunks; out.datatype = ov.datatype;
      break;
    }
    case StageKind::AllToAll:
    case StageKind::AllGather: {
      const bool framed = in.meta != nullptr;
      if (framed) { r = exchangeFramed(c, *st, p, in, out, s); break; }
      Comm* comm = st->comm;
      const bool a2a = p.kind == StageKind::AllToAll;
      const size_t block = a2a ? in.bytes / (size_t)comm->nRanks : in.bytes;   // bytes from one rank to one rank
      PeerDataPath* path = PeerDataPath::serves(1, block) &&
                                   (!a2a || in.bytes % (size_t)comm->nRanks == 0)
                               ? PeerDataPath::of(comm, s) : nullptr;
      if (path != nullptr) {
        r = path->exchange(!a2a, in.ptr, out.ptr, 1, block, nullptr, nullptr, s);
      } else if (a2a) {
        r = comm->transport->allToAll(comm, in.ptr, out.ptr, block, ncclUint8, s);
      } else {
        r = comm->transport->allGather(comm, in.ptr, out.ptr, in.bytes, ncclUint8, s);
      }
      if (a2a) {
        out.bytes = in.bytes;
        out.chunks = in.chunks;
      } else {
        out.bytes = in.bytes * (size_t)comm->nRanks;
        out.chunks = in.chunks * (size_t)comm->nRanks;
      }
      out.elements = in.datatype == spec.datatype ? out.bytes / width : out.bytes;
      out.datatype = in.datatype;
      out.codec = in.codec;
      break;
    }
    case StageKind::DecompressReduce: {
      cocclCompressorView ov = out.view();
      r = decompressReduce(in.codec, in.view(), &ov, st->reduceChunks, env);
      break;
    }
    case StageKind::DecompReduceComp: {
      cocclCompressorView ov = out.view();
      const size_t reducedChunks = in.chunks / st->reduceChunks;
      r = decompressReduceCompress(in.codec, st->codec, in.view(), &ov, st->reduceChunks, spec.datatype,
                                   reducedChunks * c.shape.elems, env);
      out.bytes = ov.bytes; out.elements = ov.elements; out.chunks = ov.chunks; out.datatype = ov.datatype;
      out.codec = st->codec;
      break;
    }
    case StageKind::Decompress: {
      cocclCompressorView ov = out.view();
      r = decompress(in.codec, in.view(), &ov, env);
      break;
    }
    case StageKind::ReduceScatter: {
      Comm* comm = st->comm;
      r = comm->transport->reduceScatter(comm, in.ptr, out.ptr, out.elements, spec.datatype, ncclSum, s);
      break;
    }
  }
  if (r != ncclSuccess) {
    COCCL_WARN("%s: stage %s of slice %zu failed (%d)", spec.name, stageName(p.kind), c.sliceIndex, (int)r);
    return r;
  }
  c.edge = out;
  return ncclSuccess;
}

void initialEdge(SliceCtx& c) {
  const PipelineSpec& spec = *c.spec;
  const size_t width = cocclTypeSize(spec.datatype);
  c.edge = Edge();
  c.edge.ptr = const_cast<char*>(static_cast<const char*>(spec.input)) + c.shape.offsetElems * width;
  c.edge.chunks = spec.inputChunks;
  c.edge.elements = spec.inputChunks * c.shape.elems;
  c.edge.bytes = c.edge.elements * width;
  c.edge.capacity = c.edge.bytes;
  c.edge.datatype = spec.datatype;
}

// ------------------------------------------------------------------ streams and events
struct StreamPool {
  std::mutex m;
  std::vector<cudaStream_t> streams;  // [0] pack, [1] unpack, [2..8] stage streams
  bool ready = false;
  ncclResult_t ensure() {
    std::lock_guard<std::mutex> lock(m);
    if (ready) return ncclSuccess;
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    streams.resize(9);
    for (int i = 0; i < 9; ++i)
      if (cudaStreamCreateWithPriority(&streams[i], cudaStreamNonBlocking, i < 2 ? lo : hi) != cudaSuccess)
        return ncclUnhandledCudaError;
    ready = true;
    return ncclSuccess;
  }
  void destroy() {
    std::lock_guard<std::mutex> lock(m);
    for (cudaStream_t s : streams) cudaStreamDestroy(s);
    streams.clear();
    ready = false;
  }
};
StreamPool gStreams;

cudaStream_t streamForStage(const StagePlan& p, size_t index) {
  if (p.kind == StageKind::Pack) return gStreams.streams[0];
  if (p.kind == StageKind::Unpack) return gStreams.streams[1];
  return gStreams.streams[2 + index % 7];
}

struct Workspace {
  void* arena = nullptr; void* arenaLease = nullptr;
  void* ring = nullptr; void* ringLease = nullptr;
};

ncclResult_t acquireWorkspace(const PipelineSpec& spec, const PipelinePlan& plan, const PipelineRuntime& rt, Workspace* w) {
  if (plan.registeredBytes) {
    ncclResult_t r = rt.workspace->acquire(spec.ownerComm, plan.registeredBytes, true, spec.stream, &w->arena, &w->arenaLease);
    if (r != ncclSuccess) return r;
  }
  if (plan.unregisteredBytes) {
    ncclResult_t r = rt.workspace->acquire(spec.ownerComm, plan.unregisteredBytes, false, spec.stream, &w->ring, &w->ringLease);
    if (r != ncclSuccess) return r;
  }
  return ncclSuccess;
}
void releaseWorkspace(const PipelineRuntime& rt, Workspace* w, cudaStream_t s) {
  if (w->arenaLease) rt.workspace->release(w->arenaLease, s);
  if (w->ringLease) rt.workspace->release(w->ringLease, s);
  *w = Workspace();
}

SliceCtx makeSlice(const PipelineSpec& spec, const PipelinePlan& plan, const PipelineRuntime& rt, const Workspace& w, size_t s) {
  SliceCtx c{&spec, &plan, &rt, s, plan.slices[s], nullptr, nullptr, Edge()};
  c.arena = static_cast<char*>(w.arena) + s * plan.sliceArenaBytes;
  c.ringSlot = w.ring ? static_cast<char*>(w.ring) + (s % 2) * plan.rawRingSlotBytes : nullptr;
  initialEdge(c);
  return c;
}

ncclResult_t runSerial(const PipelineSpec& spec, const PipelinePlan& plan, const PipelineRuntime& rt, const Workspace& w) {
  for (size_t s = 0; s < plan.slices.size(); ++s) {
    SliceCtx c = makeSlice(spec, plan, rt, w, s);
    const auto& stages = plan.stagesFor(s);
    for (size_t i = 0; i < stages.size(); ++i) {
      ncclResult_t r = runStage(c, i, stages[i], i + 1 == stages.size(), spec.stream);
      if (r != ncclSuccess) return r;
    }
  }
  return ncclSuccess;
}

// Overlapped schedule. Every stage index owns a stream; slice s of stage i waits for slice s of
// stage i-1 (event) and, by stream order, for slice s-1 of stage i. Slice-major issue order keeps
// the queues short; framed codecs are issued stage-major so that the host reads of frame metadata
// of all slices of a stage happen back to back. A raw-ring slot is reused only after the slice
// that last used it has finished (its final event).
ncclResult_t runOverlap(const PipelineSpec& spec, const PipelinePlan& plan, const PipelineRuntime& rt, const Workspace& w, bool stageMajor) {
  if (gStreams.ensure() != ncclSuccess) return ncclUnhandledCudaError;
  const size_t nSlices = plan.slices.size();
  const size_t nStages = plan.regular.size();
  std::vector<cudaEvent_t> events(nSlices * nStages, nullptr);
  cudaEvent_t inputReady = nullptr;
  ncclResult_t result = ncclSuccess;
  auto ev = [&](size_t stage, size_t slice) -> cudaEvent_t& { return events[stage * nSlices + slice]; };
  auto check = [&](cudaError_t e) { if (e != cudaSuccess && result == ncclSuccess) result = ncclUnhandledCudaError; return e == cudaSuccess; };
  check(cudaEventCreateWithFlags(&inputReady, cudaEventDisableTiming));
  for (auto& e : events) check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  std::vector<SliceCtx> ctx;
  for (size_t s = 0; s < nSlices; ++s) ctx.push_back(makeSlice(spec, plan, rt, w, s));
  if (result == ncclSuccess) {
    check(cudaEventRecord(inputReady, spec.stream));
    auto issue = [&](size_t i, size_t s) {
      if (result != ncclSuccess) return;
      const auto& stages = plan.stagesFor(s);
      cudaStream_t st = streamForStage(stages[i], i);
      if (i == 0) check(cudaStreamWaitEvent(st, inputReady, 0));
      else check(cudaStreamWaitEvent(st, ev(i - 1, s), 0));
      if (stages[i].inRawRing && s >= 2) check(cudaStreamWaitEvent(st, ev(nStages - 1, s - 2), 0));
      if (result != ncclSuccess) return;
      ncclResult_t r = runStage(ctx[s], i, stages[i], i + 1 == nStages, st);
      if (r != ncclSuccess) { result = r; return; }
      check(cudaEventRecord(ev(i, s), st));
    };
    if (stageMajor) {
      for (size_t i = 0; i < nStages; ++i) for (size_t s = 0; s < nSlices; ++s) issue(i, s);
    } else {
      for (size_t s = 0; s < nSlices; ++s) for (size_t i = 0; i < nStages; ++i) issue(i, s);
    }
    if (result == ncclSuccess)
      for (size_t s = 0; s < nSlices; ++s) check(cudaStreamWaitEvent(spec.stream, ev(nStages - 1, s), 0));
  }
  if (result != ncclSuccess) cudaDeviceSynchronize();  // nothing may still touch the workspace when it is released
  for (auto& e : events) if (e) cudaEventDestroy(e);
  if (inputReady) cudaEventDestroy(inputReady);
  return result;
}

ncclResult_t run(const PipelineSpec& spec, const PipelineRuntime& rt, int depth) {
  if (rt.workspace == nullptr) return ncclInvalidArgument;
  PipelinePlan plan;
  std::string err;
  ncclResult_t r = preparePipeline(spec, depth, &plan, &err);
  if (r != ncclSuccess) {
    COCCL_WARN("pipeline plan failed: %s", err.c_str());
    return r;
  }
  COCCL_TRACE(kLogPipeline, "%s: depth %d%s, arena %zu B x %d, raw ring %zu B, %s workspace", spec.name, plan.depth,
              plan.serial ? " (serial: buffers overlap)" : "", plan.sliceArenaBytes, plan.depth, plan.unregisteredBytes,
              plan.mode == WorkspaceMode::Split ? "split" : "unified");
  Workspace w;
  r = acquireWorkspace(spec, plan, rt, &w);
  if (r == ncclSuccess) {
    if (plan.depth == 1) r = runSerial(spec, plan, rt, w);
    else r = runOverlap(spec, plan, rt, w, plan.framed);
    if (r != ncclSuccess && plan.depth == 1) cudaDeviceSynchronize();
  }
  releaseWorkspace(rt, &w, spec.stream);
  return r;
}

}  // namespace

ncclResult_t runPipeline(const PipelineSpec& spec, const PipelineRuntime& rt) {
  // On one node the raw boundary copies of a sliced run cost more than slice overlap recovers,
  // unless the codec is framed (its host metadata reads are what slicing hides).
  bool framed = false;
  for (const Stage& st : spec.stages)
    if (st.codec && st.codec->has(cocclCompressorCapabilityFramed)) framed = true;
  const bool singleNode = spec.ownerComm != nullptr && spec.ownerComm->nNodes == 1;
  const int depth = (singleNode && !framed) ? 1 : rt.configuredDepth;
  return run(spec, rt, depth);
}

ncclResult_t runPipelineSerial(const PipelineSpec& spec, const PipelineRuntime& rt) { return run(spec, rt, 1); }

void destroyPipelineResources() { gStreams.destroy(); }

}  // namespace coccl
