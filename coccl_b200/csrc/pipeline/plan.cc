#include <algorithm>
#include <limits>

#include "pipeline/pipeline.h"

namespace coccl {

const char* stageName(StageKind k) {
  switch (k) {
    case StageKind::Compress: return "Compress";
    case StageKind::AllToAll: return "AllToAll";
    case StageKind::AllGather: return "AllGather";
    case StageKind::DecompReduceComp: return "DecompReduceComp";
    case StageKind::DecompressReduce: return "DecompressReduce";
    case StageKind::Decompress: return "Decompress";
    case StageKind::ReduceScatter: return "ReduceScatter";
    case StageKind::Pack: return "Pack";
    case StageKind::Unpack: return "Unpack";
  }
  return "?";
}

int clampPipelineDepth(int requested, size_t rawChunkCount) {
  int d = requested;
  if (d <= 1) return 1;
  if (d > kMaxPipelineDepth) return 1;  // out of range falls back to serial, it is not clamped
  if (rawChunkCount < (size_t)d) d = (int)rawChunkCount;
  return d < 1 ? 1 : d;
}

namespace {

bool mulOk(size_t a, size_t b, size_t* out) {
  if (a != 0 && b > std::numeric_limits<size_t>::max() / a) return false;
  *out = a * b;
  return true;
}

// Walk the stages symbolically for a slice of `elems` elements per chunk.
ncclResult_t planStages(const PipelineSpec& spec, size_t elems, bool stageInput, bool stageOutput,
                        std::vector<StagePlan>* out, bool* anyFramed, std::string* error) {
  out->clear();
  const size_t width = cocclTypeSize(spec.datatype);
  size_t chunks = spec.inputChunks;
  bool encoded = false;
  CompressorPolicy* edgeCodec = nullptr;
  size_t edgeBytes = 0;   // bound of the current edge payload (encoded) or exact bytes (raw)
  size_t chunkElems = elems;
  auto fail = [&](const std::string& m) {
    if (error) *error = std::string(spec.name) + ": " + m;
    return ncclInvalidUsage;
  };
  if (!mulOk(chunks * width, elems, &edgeBytes)) return fail("message size overflows");

  if (stageInput) {
    StagePlan p;
    p.kind = StageKind::Pack;
    p.inChunks = p.outChunks = chunks;
    p.outElemsPerChunk = elems;
    p.outBoundBytes = edgeBytes;
    out->push_back(p);
  }
  for (size_t i = 0; i < spec.stages.size(); ++i) {
    const Stage& st = spec.stages[i];
    StagePlan p;
    p.kind = st.kind;
    p.inChunks = chunks;
    switch (st.kind) {
      case StageKind::Compress: {
        if (encoded || st.codec == nullptr) return fail("Compress needs a raw input and a codec");
        size_t bound = 0;
        ncclResult_t r = encodedSizeBound(st.codec, cocclCompressorOperationCompress, chunks * chunkElems, chunks,
                                          spec.datatype, &bound);
        if (r != ncclSuccess) return fail("codec gave no usable size bound");
        p.framed = st.codec->has(cocclCompressorCapabilityFramed);
        if (!p.framed && bound > edgeBytes) bound = edgeBytes;  // a fixed-size codec falls back to raw bytes
        p.outChunks = chunks;
        p.outEncoded = true;
        p.outBoundBytes = bound;
        encoded = true;
        edgeCodec = st.codec;
        edgeBytes = bound;
        break;
      }
      case StageKind::AllToAll: {
        if (st.comm == nullptr || chunks % (size_t)st.comm->nRanks != 0) return fail("AllToAll needs chunks divisible by the group size");
        p.outChunks = chunks;
        p.outEncoded = encoded;
        p.outBoundBytes = edgeBytes;
        p.framed = encoded && edgeCodec && edgeCodec->has(cocclCompressorCapabilityFramed);
        break;
      }
      case StageKind::AllGather: {
        if (st.comm == nullptr) return fail("AllGather needs a communicator");
        if (!mulOk(edgeBytes, (size_t)st.comm->nRanks, &edgeBytes)) return fail("gathered size overflows");
        chunks *= (size_t)st.comm->nRanks;
        p.outChunks = chunks;
        p.outEncoded = encoded;
        p.outBoundBytes = edgeBytes;
        p.framed = encoded && edgeCodec && edgeCodec->has(cocclCompressorCapabilityFramed);
        break;
      }
      case StageKind::DecompressReduce: {
        if (!encoded || st.reduceChunks == 0 || chunks % st.reduceChunks != 0) return fail("DecompressReduce needs encoded chunks divisible by reduceChunks");
        chunks /= st.reduceChunks;
        encoded = false;
        if (!mulOk(chunks * width, chunkElems, &edgeBytes)) return fail("size overflows");
        p.outChunks = chunks;
        p.outElemsPerChunk = chunkElems;
        p.outBoundBytes = edgeBytes;
        edgeCodec = nullptr;
        break;
      }
      case StageKind::DecompReduceComp: {
        if (!encoded || st.codec == nullptr || st.reduceChunks == 0 || chunks % st.reduceChunks != 0)
          return fail("DecompReduceComp needs encoded chunks divisible by reduceChunks and an encoder");
        chunks /= st.reduceChunks;
        size_t raw = 0;
        if (!mulOk(chunks * width, chunkElems, &raw)) return fail("size overflows");
        size_t generic = 0, fused = 0;
        if (encodedSizeBound(st.codec, cocclCompressorOperationCompress, chunks * chunkElems, chunks, spec.datatype, &generic) != ncclSuccess)
          return fail("codec gave no usable size bound");
        if (encodedSizeBound(st.codec, cocclCompressorOperationDecompressReduceCompress, chunks * chunkElems, chunks, spec.datatype, &fused) != ncclSuccess)
          fused = generic;
        size_t bound = std::max(generic, fused);
        p.framed = st.codec->has(cocclCompressorCapabilityFramed);
        if (!p.framed && bound > raw) bound = raw;
        p.outChunks = chunks;
        p.outEncoded = true;
        p.outBoundBytes = bound;
        edgeCodec = st.codec;
        edgeBytes = bound;
        break;
      }
      case StageKind::Decompress: {
        if (!encoded) return fail("Decompress needs an encoded input");
        encoded = false;
        if (!mulOk(chunks * width, chunkElems, &edgeBytes)) return fail("size overflows");
        p.outChunks = chunks;
        p.outElemsPerChunk = chunkElems;
        p.outBoundBytes = edgeBytes;
        edgeCodec = nullptr;
        break;
      }
      case StageKind::ReduceScatter: {
        if (encoded || st.comm == nullptr || chunks % (size_t)st.comm->nRanks != 0) return fail("ReduceScatter needs raw chunks divisible by the group size");
        chunks /= (size_t)st.comm->nRanks;
        if (!mulOk(chunks * width, chunkElems, &edgeBytes)) return fail("size overflows");
        p.outChunks = chunks;
        p.outElemsPerChunk = chunkElems;
        p.outBoundBytes = edgeBytes;
        break;
      }
      default:
        return fail("Pack/Unpack are inserted by the planner, not listed by primitives");
    }
    p.edgeCodec = edgeCodec;
    if (p.framed) {
      *anyFramed = true;
      p.frameStrideBytes = p.outBoundBytes / p.outChunks;
      p.metaOffset = alignUpSize(p.outBoundBytes, kWorkspaceAlign);
      p.tempBytes = alignUpSize(p.metaOffset + p.outChunks * kFrameMetaBytes, kWorkspaceAlign);
    } else {
      p.tempBytes = alignUpSize(p.outBoundBytes, kWorkspaceAlign);
    }
    out->push_back(p);
  }
  if (encoded) return fail("the last stage must produce raw data");
  if (stageOutput) {
    StagePlan p;
    p.kind = StageKind::Unpack;
    p.inChunks = p.outChunks = chunks;
    p.outElemsPerChunk = chunkElems;
    p.outBoundBytes = edgeBytes;
    out->push_back(p);
  }
  // the last producing stage writes the user buffer unless its output is staged; Unpack always does
  for (size_t i = 0; i < out->size(); ++i) {
    StagePlan& p = (*out)[i];
    const bool last = i + 1 == out->size();
    if (p.kind == StageKind::Pack) p.tempBytes = alignUpSize(p.outBoundBytes, kWorkspaceAlign);
    if (last) p.tempBytes = 0;
  }
  return ncclSuccess;
}

// Temps ping-pong between the two ends of the slice arena; the arena is as large as the
// largest pair of temps that are alive at the same time (a stage's input and its output).
size_t layoutArena(std::vector<StagePlan>* stages, bool split) {
  size_t arena = 0;
  size_t prev = 0;
  for (size_t i = 0; i < stages->size(); ++i) {
    StagePlan& p = (*stages)[i];
    const bool boundary = (p.kind == StageKind::Pack) || (i + 2 == stages->size() && stages->back().kind == StageKind::Unpack);
    if (split && boundary && !p.outEncoded) {
      p.inRawRing = true;
      p.tempOffset = 0;
      prev = 0;
      continue;
    }
    p.inRawRing = false;
    arena = std::max(arena, prev + p.tempBytes);
    prev = p.tempBytes;
  }
  // offsets: even temps at 0, odd temps at the end
  bool low = true;
  for (StagePlan& p : *stages) {
    if (p.inRawRing || p.tempBytes == 0) continue;
    p.tempOffset = low ? 0 : arena - p.tempBytes;
    low = !low;
  }
  return arena;
}

size_t ringSlot(const std::vector<StagePlan>& stages) {
  size_t slot = 0;
  for (const StagePlan& p : stages)
    if (p.inRawRing) slot = std::max(slot, p.tempBytes);
  return slot;
}

}  // namespace

bool finalShape(const PipelineSpec& spec, size_t* chunksOut) {
  size_t chunks = spec.inputChunks;
  for (const Stage& st : spec.stages) {
    switch (st.kind) {
      case StageKind::AllGather: if (!st.comm) return false; chunks *= (size_t)st.comm->nRanks; break;
      case StageKind::DecompressReduce:
      case StageKind::DecompReduceComp: if (st.reduceChunks == 0 || chunks % st.reduceChunks) return false; chunks /= st.reduceChunks; break;
      case StageKind::ReduceScatter: if (!st.comm || chunks % (size_t)st.comm->nRanks) return false; chunks /= (size_t)st.comm->nRanks; break;
      default: break;
    }
  }
  *chunksOut = chunks;
  return true;
}

bool userBuffersRequireSerial(const PipelineSpec& spec, size_t outputChunks, int rank) {
  const size_t width = cocclTypeSize(spec.datatype);
  const size_t chunkBytes = spec.rawChunkCount * width;
  const char* in = static_cast<const char*>(spec.input);
  const char* out = static_cast<const char*>(spec.output);
  const char* inEnd = in + chunkBytes * spec.inputChunks;
  const char* outEnd = out + chunkBytes * outputChunks;
  const bool overlap = in < outEnd && out < inEnd;
  if (!overlap) return false;  // disjoint buffers never force the serial path
  switch (spec.inPlace) {
    case InPlaceLayout::SameBuffer: return !(in == out && spec.inputChunks == outputChunks);
    case InPlaceLayout::InputRankChunk: return !(spec.inputChunks == 1 && in == out + (size_t)rank * chunkBytes);
    case InPlaceLayout::OutputRankChunk: return !(outputChunks == 1 && out == in + (size_t)rank * chunkBytes);
    default: return true;
  }
}

ncclResult_t preparePipeline(const PipelineSpec& spec, int requestedDepth, PipelinePlan* plan, std::string* error) {
  auto fail = [&](const std::string& m) {
    if (error) *error = std::string(spec.name) + ": " + m;
    return ncclInvalidArgument;
  };
  if (spec.input == nullptr || spec.output == nullptr || spec.rawChunkCount == 0 || spec.inputChunks == 0 ||
      spec.stages.empty() || cocclTypeSize(spec.datatype) == 0 || spec.ownerComm == nullptr)
    return fail("incomplete pipeline specification");
  *plan = PipelinePlan();
  size_t finalChunks = 0;
  if (!finalShape(spec, &finalChunks)) return fail("stage list does not compose");

  int depth = clampPipelineDepth(requestedDepth, spec.rawChunkCount);
  plan->serial = userBuffersRequireSerial(spec, finalChunks, spec.ownerComm->rank);
  if (plan->serial) depth = 1;
  plan->depth = depth;

  // slices: the same element range of every rank chunk; the last slice takes the remainder
  const size_t quotient = spec.rawChunkCount / (size_t)depth;
  for (int s = 0; s < depth; ++s) {
    SliceShape sh;
    sh.offsetElems = (size_t)s * quotient;
    sh.elems = (s + 1 == depth) ? spec.rawChunkCount - sh.offsetElems : quotient;
    plan->slices.push_back(sh);
  }

  plan->swizzle = spec.inputLayout == InputLayout::HierarchicalSwizzle;
  if (plan->swizzle && spec.stages[0].kind == StageKind::Compress && spec.stages[0].codec != nullptr &&
      spec.stages[0].codec->has(cocclCompressorCapabilityFusedHierarchicalSwizzle))
    plan->swizzle = false;  // the codec applies the swizzle while it compresses
  plan->stageInput = spec.inputChunks > 1 && (depth > 1 || plan->swizzle);
  if (plan->swizzle && spec.inputChunks == 1) plan->swizzle = false;
  plan->stageOutput = depth > 1 && finalChunks > 1;

  bool framed = false;
  ncclResult_t r = planStages(spec, plan->slices[0].elems, plan->stageInput, plan->stageOutput, &plan->regular, &framed, error);
  if (r != ncclSuccess) return r;
  if (plan->slices.back().elems != plan->slices[0].elems) {
    r = planStages(spec, plan->slices.back().elems, plan->stageInput, plan->stageOutput, &plan->tail, &framed, error);
    if (r != ncclSuccess) return r;
  }
  plan->framed = framed;

  // workspace: unified (everything in the registered slice arena) or split (raw boundary temps in a
  // 2-slot unregistered ring); regular and tail slices are planned separately and merged by maximum
  auto evaluate = [&](bool split, size_t* arena, size_t* slot) {
    std::vector<StagePlan> a = plan->regular, b = plan->tail;
    *arena = layoutArena(&a, split);
    *slot = ringSlot(a);
    if (!b.empty()) {
      *arena = std::max(*arena, layoutArena(&b, split));
      *slot = std::max(*slot, ringSlot(b));
    }
  };
  size_t uArena = 0, uSlot = 0, sArena = 0, sSlot = 0;
  evaluate(false, &uArena, &uSlot);
  evaluate(true, &sArena, &sSlot);
  const size_t unifiedTotal = uArena * (size_t)depth;
  const size_t splitTotal = sArena * (size_t)depth + 2 * sSlot;
  const bool split = sSlot > 0 && splitTotal < unifiedTotal;
  plan->mode = split ? WorkspaceMode::Split : WorkspaceMode::Unified;
  plan->sliceArenaBytes = layoutArena(&plan->regular, split);
  if (!plan->tail.empty()) plan->sliceArenaBytes = std::max(plan->sliceArenaBytes, layoutArena(&plan->tail, split));
  // offsets of low/high temps were computed against each plan's own arena; redo them against the merged one
  for (std::vector<StagePlan>* v : {&plan->regular, &plan->tail}) {
    bool low = true;
    for (StagePlan& p : *v) {
      if (p.inRawRing || p.tempBytes == 0) continue;
      p.tempOffset = low ? 0 : plan->sliceArenaBytes - p.tempBytes;
      low = !low;
    }
  }
  plan->rawRingSlotBytes = split ? sSlot : 0;
  plan->registeredBytes = plan->sliceArenaBytes * (size_t)depth;
  plan->unregisteredBytes = 2 * plan->rawRingSlotBytes;
  return ncclSuccess;
}

}  // namespace coccl
