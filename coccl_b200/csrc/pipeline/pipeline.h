// Staged pipeline: the generic path for codecs that have no fused kernel (any SDK plugin).
// A collective is a list of stages over "edges" (a buffer of raw or encoded chunks); a planner
// cuts the message into slices, bounds every intermediate buffer and lays out a workspace; an
// executor runs the slices over streams so that encoding, exchange and decoding overlap.
//
// Behavioural model: src/coccl-extend/core/pipeline/coccl_pipeline.h:9-100 (stage kinds, in-place
// and input layouts), coccl_pipeline_plan.cc:24-562 (depth clamp, serial rule, slice shapes,
// output bounds, staging temps, unified vs split workspace, 256-byte alignment),
// coccl_pipeline_stage.cc:83-411 (stage handlers), coccl_pipeline_execute.cc:23-565 (stream/event
// schedule: serial, slice-major overlap, stage-major overlap for framed codecs) and
// coccl_frame_exchange.cc:38-176 (variable-length frame exchange).
#pragma once
#include <stddef.h>
#include <string>
#include <vector>

#include "compression/compressor_runtime.h"
#include "runtime/comm.h"

namespace coccl {

enum class StageKind { Compress = 0, AllToAll, AllGather, DecompReduceComp, DecompressReduce, Decompress, ReduceScatter, Pack, Unpack };
const char* stageName(StageKind k);

enum class InPlaceLayout { None = 0, SameBuffer, InputRankChunk, OutputRankChunk };
enum class InputLayout { Contiguous = 0, HierarchicalSwizzle };

struct Stage {
  StageKind kind;
  Comm* comm = nullptr;             // collective stages: the communicator they run on
  size_t reduceChunks = 0;          // reducing stages: copies summed per output chunk
  CompressorPolicy* codec = nullptr;  // Compress / DecompReduceComp: the encoder of this stage
  static Stage compress(CompressorPolicy* c) { return {StageKind::Compress, nullptr, 0, c}; }
  static Stage allToAll(Comm* c) { return {StageKind::AllToAll, c, 0, nullptr}; }
  static Stage allGather(Comm* c) { return {StageKind::AllGather, c, 0, nullptr}; }
  static Stage decompReduceComp(size_t r, CompressorPolicy* c) { return {StageKind::DecompReduceComp, nullptr, r, c}; }
  static Stage decompressReduce(size_t r) { return {StageKind::DecompressReduce, nullptr, r, nullptr}; }
  static Stage decompress() { return {StageKind::Decompress, nullptr, 0, nullptr}; }
  static Stage reduceScatter(Comm* c) { return {StageKind::ReduceScatter, c, 0, nullptr}; }
};

// rawChunkCount = unsliced elements of one rank chunk; inputChunks = rank chunks entering.
struct PipelineSpec {
  const char* name = "";
  const void* input = nullptr;
  void* output = nullptr;
  size_t rawChunkCount = 0;
  size_t inputChunks = 0;
  ncclDataType_t datatype = ncclFloat32;
  Comm* ownerComm = nullptr;
  cudaStream_t stream = nullptr;
  std::vector<Stage> stages;
  InPlaceLayout inPlace = InPlaceLayout::None;
  InputLayout inputLayout = InputLayout::Contiguous;
};

constexpr size_t kWorkspaceAlign = 256;
constexpr size_t kFrameMetaBytes = 16;

inline size_t alignUpSize(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct SliceShape {
  size_t offsetElems = 0;  // first element of the slice inside every rank chunk
  size_t elems = 0;        // elements per chunk in this slice
};

// What one stage produces for one slice.
struct StagePlan {
  StageKind kind;
  size_t inChunks = 0, outChunks = 0;
  size_t outElemsPerChunk = 0;   // raw stages
  bool outEncoded = false;
  size_t outBoundBytes = 0;      // capacity reserved for the output edge (payload)
  bool framed = false;
  size_t frameStrideBytes = 0;   // bound / chunks for framed edges
  size_t metaOffset = 0;         // 256-aligned offset of the metadata array behind the payload
  size_t tempBytes = 0;          // payload + metadata, aligned; 0 when the stage writes the user buffer
  size_t tempOffset = 0;         // offset inside the slice arena (or raw ring for boundary temps)
  bool inRawRing = false;
  CompressorPolicy* edgeCodec = nullptr;  // codec that describes the (encoded) output edge
};

enum class WorkspaceMode { Unified, Split };

struct PipelinePlan {
  int depth = 1;
  bool serial = false;
  bool framed = false;
  bool stageInput = false;    // Pack into a temp before stage 0
  bool stageOutput = false;   // final stage writes a temp, Unpack scatters it
  bool swizzle = false;       // the Pack applies the hierarchical rank swizzle
  std::vector<SliceShape> slices;
  std::vector<StagePlan> regular;  // plan of a full slice (includes Pack/Unpack entries when staged)
  std::vector<StagePlan> tail;     // plan of the last slice when it differs
  size_t sliceArenaBytes = 0;      // per slice, registered
  size_t rawRingSlotBytes = 0;     // split mode: one slot of the 2-slot unregistered ring
  WorkspaceMode mode = WorkspaceMode::Unified;
  size_t registeredBytes = 0, unregisteredBytes = 0;
  const std::vector<StagePlan>& stagesFor(size_t slice) const {
    return (slice + 1 == slices.size() && !tail.empty()) ? tail : regular;
  }
};

// Requested depth -> effective depth: <=1 -> 1, >16 -> 1 (not clamped), never more than rawChunkCount.
int clampPipelineDepth(int requested, size_t rawChunkCount);
// True when the user buffers overlap in a way that is not exactly the declared in-place layout.
bool userBuffersRequireSerial(const PipelineSpec& spec, size_t outputChunks, int rank);
// Number of chunks / elements the last stage writes to the user buffer.
bool finalShape(const PipelineSpec& spec, size_t* chunks);
ncclResult_t preparePipeline(const PipelineSpec& spec, int requestedDepth, PipelinePlan* plan, std::string* error);

// ---- execution -------------------------------------------------------------------------------
// Buffer source for workspaces (the buffer manager in production, plain allocations in tests).
struct WorkspaceProvider {
  virtual ~WorkspaceProvider() {}
  virtual ncclResult_t acquire(Comm* comm, size_t bytes, bool registered, cudaStream_t stream, void** ptr, void** lease) = 0;
  virtual void release(void* lease, cudaStream_t stream) = 0;
};

struct PipelineRuntime {
  WorkspaceProvider* workspace = nullptr;
  int configuredDepth = 1;
  // test hooks: null = CUDA
  const DeviceAllocator* alloc = nullptr;
};

ncclResult_t runPipeline(const PipelineSpec& spec, const PipelineRuntime& rt);
ncclResult_t runPipelineSerial(const PipelineSpec& spec, const PipelineRuntime& rt);
void destroyPipelineResources();

// ---- frame exchange (variable-length codecs) ---------------------------------------------------
struct FrameTransfer { int peer; size_t sendOffset, sendBytes, recvOffset, recvBytes; };
// Metadata is valid when 0 < payloadBytes <= stride and encoding is Encoded or Raw.
bool frameMetadataValid(const cocclCompressorFrameMetadata& m, size_t strideBytes);
// Build the per-peer transfers of an all-to-all (slot i goes to rank i) or all-gather (every slot of
// mine goes to everyone) exchange from host copies of the metadata.
ncclResult_t buildFrameExchange(bool allGather, int rank, int nRanks, size_t framesPerRank, size_t strideBytes,
                                const cocclCompressorFrameMetadata* sendMeta, const cocclCompressorFrameMetadata* recvMeta,
                                std::vector<FrameTransfer>* sends, std::vector<FrameTransfer>* recvs);

}  // namespace coccl
