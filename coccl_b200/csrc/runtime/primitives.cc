#include "runtime/primitives.h"

#include "runtime/log.h"

namespace coccl {

CompressorPolicy* flatCodec(const PreparedCall& call) {
  return call.info.comm->nNodes == 1 ? call.codec(Scope::Intra) : call.codec(Scope::Default);
}

namespace {

// Stages of the hierarchical reduction: intra-node level, then inter-node level. `last` is the codec
// that encodes what leaves the inter level (null: the inter level ends in raw data).
ncclResult_t hierarchicalReduction(const PreparedCall& call, Comm* intra, Comm* inter, CompressorPolicy* last,
                                   std::vector<Stage>* st) {
  if (intra == nullptr || inter == nullptr) return ncclInvalidArgument;
  CompressorPolicy* ci = call.codec(Scope::Intra);
  CompressorPolicy* cx = call.codec(Scope::Inter);
  const size_t local = (size_t)intra->nRanks, nodes = (size_t)inter->nRanks;
  // level 1: every local peer receives its group of `nodes` chunks from each local rank
  if (ci != nullptr) {
    st->push_back(Stage::compress(ci));
    st->push_back(Stage::allToAll(intra));
    if (cx != nullptr) st->push_back(Stage::decompReduceComp(local, cx));
    else st->push_back(Stage::decompressReduce(local));
  } else {
    st->push_back(Stage::reduceScatter(intra));  // a level without codec reduces natively
    if (cx != nullptr) st->push_back(Stage::compress(cx));
  }
  // level 2: one chunk per node peer
  if (cx != nullptr) {
    st->push_back(Stage::allToAll(inter));
    if (last != nullptr) st->push_back(Stage::decompReduceComp(nodes, last));
    else st->push_back(Stage::decompressReduce(nodes));
  } else {
    st->push_back(Stage::reduceScatter(inter));
    if (last != nullptr) st->push_back(Stage::compress(last));
  }
  return ncclSuccess;
}

}  // namespace

ncclResult_t buildRecipe(const PreparedCall& call, Comm* intra, Comm* inter, PipelineSpec* spec) {
  const CallInfo& info = call.info;
  Comm* comm = info.comm;
  const size_t n = (size_t)comm->nRanks;
  *spec = PipelineSpec();
  spec->input = info.sendbuff;
  spec->output = info.recvbuff;
  spec->datatype = info.datatype;
  spec->ownerComm = comm;
  spec->stream = info.stream;
  CompressorPolicy* flat = flatCodec(call);
  switch (info.op) {
    case Operation::AllGather:
      if (flat == nullptr) return ncclInvalidUsage;
      spec->name = "AllGather";
      spec->rawChunkCount = info.count;
      spec->inputChunks = 1;
      spec->stages = {Stage::compress(flat), Stage::allGather(comm), Stage::decompress()};
      spec->inPlace = InPlaceLayout::InputRankChunk;
      return ncclSuccess;
    case Operation::AllToAll:
      if (flat == nullptr) return ncclInvalidUsage;
      spec->name = "AllToAll";
      spec->rawChunkCount = info.count;
      spec->inputChunks = n;
      spec->stages = {Stage::compress(flat), Stage::allToAll(comm), Stage::decompress()};
      return ncclSuccess;
    case Operation::ReduceScatter:
      spec->rawChunkCount = info.count;
      spec->inputChunks = n;
      spec->inPlace = InPlaceLayout::OutputRankChunk;
      if (call.algorithm == Algorithm::RsTwoShot) {
        spec->name = "ReduceScatterTwoShot";
        spec->inputLayout = InputLayout::HierarchicalSwizzle;
        return hierarchicalReduction(call, intra, inter, nullptr, &spec->stages);
      }
      if (flat == nullptr) return ncclInvalidUsage;
      spec->name = "ReduceScatterOneShot";
      spec->stages = {Stage::compress(flat), Stage::allToAll(comm), Stage::decompressReduce(n)};
      return ncclSuccess;
    case Operation::AllReduce:
      if (info.count % n != 0) return ncclInvalidUsage;
      spec->rawChunkCount = info.count / n;
      spec->inputChunks = n;
      spec->inPlace = InPlaceLayout::SameBuffer;
      if (call.algorithm == Algorithm::ArOneShot) {
        if (flat == nullptr) return ncclInvalidUsage;
        spec->name = "AllReduceOneShot";
        spec->stages = {Stage::compress(flat), Stage::allGather(comm), Stage::decompressReduce(n)};
        return ncclSuccess;
      }
      if (call.algorithm == Algorithm::ArTripleShot) {
        CompressorPolicy* def = call.codec(Scope::Default);
        if (def == nullptr) return ncclInvalidUsage;
        spec->name = "AllReduceTripleShot";
        spec->inputLayout = InputLayout::HierarchicalSwizzle;
        ncclResult_t r = hierarchicalReduction(call, intra, inter, def, &spec->stages);
        if (r != ncclSuccess) return r;
        spec->stages.push_back(Stage::allGather(comm));
        spec->stages.push_back(Stage::decompress());
        return ncclSuccess;
      }
      if (flat == nullptr) return ncclInvalidUsage;
      spec->name = "AllReduceTwoShot";
      spec->stages = {Stage::compress(flat), Stage::allToAll(comm), Stage::decompReduceComp(n, flat), Stage::allGather(comm),
                      Stage::decompress()};
      return ncclSuccess;
    default:
      return ncclInvalidArgument;
  }
}

ncclResult_t StagedExecutor::execute(Runtime* rt, const PreparedCall& call) {
  if (call.info.op == Operation::SendRecv) return executeSendRecvBatch(rt, {call});
  Comm* intra = nullptr;
  Comm* inter = nullptr;
  if (call.algorithm == Algorithm::RsTwoShot || call.algorithm == Algorithm::ArTripleShot) {
    ncclResult_t r = rt->hierarchy(call.info.comm, &intra, &inter);
    if (r != ncclSuccess) return r;
  }
  PipelineSpec spec;
  ncclResult_t r = buildRecipe(call, intra, inter, &spec);
  if (r != ncclSuccess) return r;
  PipelineRuntime prt;
  prt.workspace = buffers_;
  prt.configuredDepth = rt->config().pipelineDepth;
  // the one-shot all-reduce moves N times the data: slicing it only multiplies the copies
  if (call.algorithm == Algorithm::ArOneShot) return runPipelineSerial(spec, prt);
  return runPipeline(spec, prt);
}

// Compressed point-to-point batch (core: src/coccl-extend/extensions/primitives/coccl_sendrecv.cc:103-277).
// Per call a slot [payload | 256-aligned 16-byte header] is leased. Senders compress into the slot and
// write the header (framed codecs do it on the device, fixed-size codecs get it from the host); the
// headers are exchanged first, read back by the host (one stream synchronisation), then the payloads
// travel with their actual sizes, and receivers decompress (raw payloads are copied).
ncclResult_t StagedExecutor::executeSendRecvBatch(Runtime* rt, const std::vector<PreparedCall>& batch) {
  if (batch.empty()) return ncclSuccess;
  struct Slot {
    BufferLease lease;
    char* payload = nullptr;
    cocclCompressorFrameMetadata* meta = nullptr;
    size_t capacity = 0;
    CompressorPolicy* codec = nullptr;
    cocclCompressorView encoded{};
  };
  std::vector<Slot> slots(batch.size());
  cudaStream_t stream = batch[0].info.stream;
  Comm* comm = batch[0].info.comm;
  ncclResult_t result = ncclSuccess;
  auto env = [&](const CallInfo& i) {
    ExecEnv e;
    e.stream = i.stream; e.cudaDev = i.comm->cudaDev; e.rank = i.comm->rank; e.nRanks = i.comm->nRanks;
    e.nodes = i.comm->nNodes; e.devicesPerNode = i.comm->localRanks;
    return e;
  };
  // 1. lease slots, compress on the sending side
  for (size_t k = 0; k < batch.size() && result == ncclSuccess; ++k) {
    const PreparedCall& c = batch[k];
    const CallInfo& i = c.info;
    Slot& s = slots[k];
    const Scope scope = nodeOfRank(i.comm, i.peer) == i.comm->node ? Scope::Intra : Scope::Inter;
    s.codec = c.codec(scope);
    if (s.codec == nullptr) { result = ncclInvalidUsage; break; }
    const size_t raw = i.count * cocclTypeSize(i.datatype);
    size_t bound = 0;
    if ((result = encodedSizeBound(s.codec, cocclCompressorOperationCompress, i.count, 1, i.datatype, &bound)) != ncclSuccess) break;
    s.capacity = alignUpSize(bound > raw ? bound : raw, kWorkspaceAlign);
    if ((result = buffers_->getBuffer(i.comm, s.capacity + kWorkspaceAlign, true, i.stream, &s.lease)) != ncclSuccess) break;
    s.payload = static_cast<char*>(s.lease.ptr);
    s.meta = reinterpret_cast<cocclCompressorFrameMetadata*>(s.payload + s.capacity);
    if (i.func != Func::Send) continue;
    const bool framed = s.codec->has(cocclCompressorCapabilityFramed);
    cocclCompressorView in{const_cast<void*>(i.sendbuff), raw, raw, i.count, 1, i.datatype, nullptr, 0};
    s.encoded = cocclCompressorView{s.payload, s.capacity, 0, s.capacity, 1, ncclInt8, framed ? s.meta : nullptr, framed ? s.capacity : 0};
    if ((result = compress(s.codec, in, &s.encoded, env(i))) != ncclSuccess) break;
    if (!framed) {
      cocclCompressorFrameMetadata h{s.encoded.bytes,
                                     s.encoded.datatype == COCCL_COMPRESSOR_RAW_PASSTHROUGH ? (uint32_t)cocclCompressorFrameRaw
                                                                                             : (uint32_t)cocclCompressorFrameEncoded, 0};
      if (cudaMemcpyAsync(s.meta, &h, sizeof(h), cudaMemcpyHostToDevice, i.stream) != cudaSuccess) result = ncclUnhandledCudaError;
    }
  }
  // 2. headers
  std::vector<P2POp> ops;
  if (result == ncclSuccess) {
    for (size_t k = 0; k < batch.size(); ++k)
      ops.push_back({batch[k].info.func == Func::Send, slots[k].meta, sizeof(cocclCompressorFrameMetadata), batch[k].info.peer});
    result = comm->transport->p2pBatch(comm, ops.data(), (int)ops.size(), stream);
  }
  // 3. the host learns the payload sizes
  std::vector<cocclCompressorFrameMetadata> heads(batch.size());
  if (result == ncclSuccess) {
    for (size_t k = 0; k < batch.size() && result == ncclSuccess; ++k)
      if (cudaMemcpyAsync(&heads[k], slots[k].meta, sizeof(heads[k]), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
        result = ncclUnhandledCudaError;
    if (result == ncclSuccess && cudaStreamSynchronize(stream) != cudaSuccess) result = ncclUnhandledCudaError;
    for (size_t k = 0; k < batch.size() && result == ncclSuccess; ++k)
      if (!frameMetadataValid(heads[k], slots[k].capacity)) result = ncclInvalidUsage;
  }
  // 4. payloads with their actual sizes
  if (result == ncclSuccess) {
    ops.clear();
    for (size_t k = 0; k < batch.size(); ++k)
      ops.push_back({batch[k].info.func == Func::Send, slots[k].payload, (size_t)heads[k].payloadBytes, batch[k].info.peer});
    result = comm->transport->p2pBatch(comm, ops.data(), (int)ops.size(), stream);
  }
  // 5. receivers decode
  for (size_t k = 0; k < batch.size() && result == ncclSuccess; ++k) {
    const CallInfo& i = batch[k].info;
    if (i.func != Func::Recv) continue;
    Slot& s = slots[k];
    const size_t raw = i.count * cocclTypeSize(i.datatype);
    const bool isRaw = heads[k].encoding == cocclCompressorFrameRaw;
    const bool framed = s.codec->has(cocclCompressorCapabilityFramed);
    cocclCompressorView in{s.payload, s.capacity, (size_t)heads[k].payloadBytes, (size_t)heads[k].payloadBytes, 1,
                           isRaw ? COCCL_COMPRESSOR_RAW_PASSTHROUGH : ncclInt8, framed ? s.meta : nullptr, framed ? s.capacity : 0};
    cocclCompressorView out{i.recvbuff, raw, 0, i.count, 1, i.datatype, nullptr, 0};
    result = decompress(s.codec, in, &out, env(i));
  }
  if (result != ncclSuccess) {
    COCCL_WARN("compressed send/recv batch of %zu calls failed (%d)", batch.size(), (int)result);
    cudaDeviceSynchronize();
  }
  for (Slot& s : slots)
    if (s.lease.owner != nullptr) buffers_->releaseBuffer(&s.lease, stream);
  (void)rt;
  return result;
}

}  // namespace coccl
