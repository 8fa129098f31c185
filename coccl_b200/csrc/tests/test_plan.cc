// Pipeline planner, serial execution with a fake codec/transport, frame exchange, size bound and
// codec glue. Scenario sources: coccl_pipeline_plan_test, coccl_inplace_plan_test,
// coccl_remainder_plan_test, coccl_framed_pipeline_plan_test, coccl_swizzle_plan_test,
// coccl_unified_arena_test / coccl_pipeline_workspace_test, coccl_frame_exchange_test.cc:30-170,
// coccl_size_query_test, coccl_codec_flow_test of the reference.
#include "fakes.h"
#include "host_test.h"
#include "pipeline/pipeline.h"

using namespace coccl;
using fakes::FakeTransport;

namespace {

struct PlanFixture {
  FakeTransport transport;
  Comm comm;
  LoadedPlugin plugin;
  std::unique_ptr<CompressorPolicy> codec;
  std::vector<char> in, out;
  PlanFixture(int nRanks = 8, int nNodes = 1, size_t bytes = 1 << 20) : in(bytes), out(bytes) {
    comm = fakes::makeComm(&transport, 2, nRanks, nNodes);
    plugin.name = "fake";
    plugin.descriptor = fakes::fakePlugin("fake");
    codec.reset(new CompressorPolicy(&plugin, malloc(4), 0, "test"));
  }
  PipelineSpec spec(size_t rawChunkCount, size_t chunks, std::vector<Stage> stages) {
    PipelineSpec s;
    s.name = "test";
    s.input = in.data();
    s.output = out.data();
    s.rawChunkCount = rawChunkCount;
    s.inputChunks = chunks;
    s.datatype = ncclFloat32;
    s.ownerComm = &comm;
    s.stages = std::move(stages);
    return s;
  }
};

}  // namespace

TEST(plan_depth_clamp_rules) {
  EXPECT_EQ(clampPipelineDepth(0, 100), 1);
  EXPECT_EQ(clampPipelineDepth(1, 100), 1);
  EXPECT_EQ(clampPipelineDepth(4, 100), 4);
  EXPECT_EQ(clampPipelineDepth(16, 100), 16);
  EXPECT_EQ(clampPipelineDepth(17, 100), 1);   // beyond the maximum falls back to 1, it is not clamped to 16
  EXPECT_EQ(clampPipelineDepth(8, 3), 3);      // never more slices than elements
}

TEST(plan_slices_remainder_and_staging) {
  fakes::knobs() = fakes::PluginKnobs();
  PlanFixture f;
  PipelineSpec s = f.spec(1003, 8, {Stage::compress(f.codec.get()), Stage::allToAll(&f.comm), Stage::decompressReduce(8)});
  PipelinePlan p;
  std::string err;
  EXPECT(preparePipeline(s, 4, &p, &err) == ncclSuccess);
  EXPECT_EQ(p.depth, 4);
  EXPECT_EQ(p.slices.size(), (size_t)4);
  EXPECT(p.slices[0].elems == 250 && p.slices[3].elems == 253 && p.slices[3].offsetElems == 750);  // remainder to the last slice
  EXPECT(p.stageInput);      // several input chunks and depth > 1: slices are gathered by Pack
  EXPECT(!p.stageOutput);    // one output chunk: the last stage writes the user buffer directly
  EXPECT(!p.tail.empty());   // the tail slice is planned separately
  EXPECT(p.regular.front().kind == StageKind::Pack && p.regular.back().kind == StageKind::DecompressReduce);
  EXPECT_EQ(p.regular.back().tempBytes, (size_t)0);
  // encoded bound = raw / 4 (fake ratio), aligned temps
  const StagePlan& c = p.regular[1];
  EXPECT(c.outEncoded && c.outBoundBytes == 8 * 250 * 4 / 4 && c.tempBytes % kWorkspaceAlign == 0);
  EXPECT(p.registeredBytes == p.sliceArenaBytes * 4);
  // depth 1: nothing is staged
  EXPECT(preparePipeline(s, 1, &p, &err) == ncclSuccess);
  EXPECT(!p.stageInput && !p.stageOutput && p.slices.size() == 1 && p.tail.empty());
  // all-to-all with many output chunks and depth > 1 stages the output too
  PipelineSpec a2a = f.spec(1000, 8, {Stage::compress(f.codec.get()), Stage::allToAll(&f.comm), Stage::decompress()});
  EXPECT(preparePipeline(a2a, 2, &p, &err) == ncclSuccess);
  EXPECT(p.stageInput && p.stageOutput && p.regular.back().kind == StageKind::Unpack);
  // all-gather: one input chunk is never staged
  PipelineSpec ag = f.spec(1000, 1, {Stage::compress(f.codec.get()), Stage::allGather(&f.comm), Stage::decompress()});
  EXPECT(preparePipeline(ag, 2, &p, &err) == ncclSuccess);
  EXPECT(!p.stageInput && p.stageOutput);
  EXPECT(p.regular[1].outChunks == 8 && p.regular[1].outBoundBytes == 8 * p.regular[0].outBoundBytes);
}

TEST(plan_codec_that_expands_is_capped_at_raw) {
  fakes::knobs() = fakes::PluginKnobs();
  fakes::knobs().compressRatio = 0.5;  // "compression" doubles the size
  PlanFixture f;
  PipelineSpec s = f.spec(1024, 8, {Stage::compress(f.codec.get()), Stage::allToAll(&f.comm), Stage::decompress()});
  PipelinePlan p;
  std::string err;
  EXPECT(preparePipeline(s, 1, &p, &err) == ncclSuccess);
  EXPECT_EQ(p.regular[0].outBoundBytes, (size_t)8 * 1024 * 4);
  // a codec without a bound plans raw bytes
  fakes::knobs().sizeBoundUnknown = true;
  EXPECT(preparePipeline(s, 1, &p, &err) == ncclSuccess);
  EXPECT_EQ(p.regular[0].outBoundBytes, (size_t)8 * 1024 * 4);
}

TEST(plan_inplace_layouts_and_serial_rule) {
  fakes::knobs() = fakes::PluginKnobs();
  PlanFixture f;
  const size_t count = 1000, chunkBytes = count * 4;
  auto rs = [&](const void* in, void* out, InPlaceLayout l) {
    PipelineSpec s = f.spec(count, 8, {Stage::compress(f.codec.get()), Stage::allToAll(&f.comm), Stage::decompressReduce(8)});
    s.input = in; s.output = out; s.inPlace = l;
    return s;
  };
  char* base = f.in.data();
  PipelinePlan p;
  std::string err;
  // disjoint buffers never force the serial path
  EXPECT(!userBuffersRequireSerial(rs(base, f.out.data(), InPlaceLayout::None), 1, 2));
  // declared NCCL in-place reduce-scatter: out == in + rank * chunk
  EXPECT(!userBuffersRequireSerial(rs(base, base + 2 * chunkBytes, InPlaceLayout::OutputRankChunk), 1, 2));
  EXPECT(userBuffersRequireSerial(rs(base, base + 3 * chunkBytes, InPlaceLayout::OutputRankChunk), 1, 2));   // wrong chunk
  EXPECT(userBuffersRequireSerial(rs(base, base + 2 * chunkBytes, InPlaceLayout::None), 1, 2));             // overlap not declared
  EXPECT(preparePipeline(rs(base, base + 3 * chunkBytes, InPlaceLayout::OutputRankChunk), 4, &p, &err) == ncclSuccess);
  EXPECT(p.serial && p.depth == 1);
  EXPECT(preparePipeline(rs(base, base + 2 * chunkBytes, InPlaceLayout::OutputRankChunk), 4, &p, &err) == ncclSuccess);
  EXPECT(!p.serial && p.depth == 4);
  // all-gather in place: in == out + rank * chunk, one input chunk
  PipelineSpec ag = f.spec(count, 1, {Stage::compress(f.codec.get()), Stage::allGather(&f.comm), Stage::decompress()});
  ag.output = base; ag.input = base + 2 * chunkBytes; ag.inPlace = InPlaceLayout::InputRankChunk;
  EXPECT(!userBuffersRequireSerial(ag, 8, 2));
  ag.input = base + 2 * chunkBytes + 4;
  EXPECT(userBuffersRequireSerial(ag, 8, 2));
  // same buffer (all-reduce)
  PipelineSpec ar = f.spec(count, 8, {Stage::compress(f.codec.get()), Stage::allToAll(&f.comm), Stage::decompReduceComp(8, f.codec.get()),
                                      Stage::allGather(&f.comm), Stage::decompress()});
  ar.output = base; ar.input = base; ar.inPlace = InPlaceLayout::SameBuffer;
  EXPECT(!userBuffersRequireSerial(ar, 8, 2));
  ar.output = base + 8;
  EXPECT(userBuffersRequireSerial(ar, 8, 2));
}

TEST(plan_framed_edges_carry_metadata) {
  fakes::knobs() = fakes::PluginKnobs();
  fakes::knobs().framed = true;
  PlanFixture f;
  PipelineSpec s = f.spec(4096, 8, {Stage::compress(f.codec.get()), Stage::allToAll(&f.comm), Stage::decompress()});
  PipelinePlan p;
  std::string err;
  EXPECT(preparePipeline(s, 2, &p, &err) == ncclSuccess);
  EXPECT(p.framed);
  const StagePlan& c = p.regular[1];  // [Pack, Compress, AllToAll, Decompress, Unpack]
  EXPECT(c.kind == StageKind::Compress && c.framed);
  EXPECT_EQ(c.frameStrideBytes, c.outBoundBytes / 8);
  EXPECT(c.metaOffset % kWorkspaceAlign == 0 && c.metaOffset >= c.outBoundBytes);
  EXPECT(c.tempBytes >= c.metaOffset + 8 * kFrameMetaBytes);
  EXPECT(p.regular[2].framed && p.regular[2].frameStrideBytes == c.frameStrideBytes);
  EXPECT(!p.regular[3].framed);
}

TEST(plan_swizzle_and_fused_swizzle_codec) {
  fakes::knobs() = fakes::PluginKnobs();
  PlanFixture f(16, 2);
  Comm intra = fakes::makeComm(&f.transport, 2, 8, 1), inter = fakes::makeComm(&f.transport, 0, 2, 2);
  PipelineSpec s = f.spec(1000, 16, {Stage::compress(f.codec.get()), Stage::allToAll(&intra), Stage::decompReduceComp(8, f.codec.get()),
                                     Stage::allToAll(&inter), Stage::decompressReduce(2)});
  s.inputLayout = InputLayout::HierarchicalSwizzle;
  PipelinePlan p;
  std::string err;
  EXPECT(preparePipeline(s, 1, &p, &err) == ncclSuccess);
  EXPECT(p.swizzle && p.stageInput);  // the swizzle needs the Pack even without slicing
  EXPECT(p.regular[0].kind == StageKind::Pack);
  EXPECT(p.regular[3].outChunks == 2 && p.regular[5].outChunks == 1);
  // a codec that swizzles while compressing removes the staging copy
  fakes::knobs().fusedSwizzle = true;
  f.plugin.descriptor = fakes::fakePlugin("fake");
  EXPECT(preparePipeline(s, 1, &p, &err) == ncclSuccess);
  EXPECT(!p.swizzle && !p.stageInput);
}

TEST(plan_workspace_unified_vs_split) {
  fakes::knobs() = fakes::PluginKnobs();
  fakes::knobs().compressRatio = 8.0;
  PlanFixture f(8, 1, 8 << 20);
  // raw boundary temps (pack input, unpack output) dominate: moving them to a 2-slot ring saves memory at depth 8
  PipelineSpec s = f.spec(200000, 8, {Stage::compress(f.codec.get()), Stage::allToAll(&f.comm), Stage::decompress()});
  PipelinePlan p;
  std::string err;
  EXPECT(preparePipeline(s, 8, &p, &err) == ncclSuccess);
  EXPECT(p.mode == WorkspaceMode::Split);
  EXPECT(p.rawRingSlotBytes >= 8 * 25000 * 4);
  EXPECT(p.unregisteredBytes == 2 * p.rawRingSlotBytes);
  EXPECT(p.registeredBytes == 8 * p.sliceArenaBytes);
  EXPECT(p.sliceArenaBytes < p.rawRingSlotBytes);
  // depth 2: the ring (2 slots) cannot beat the arena (2 slices) -> unified
  EXPECT(preparePipeline(s, 2, &p, &err) == ncclSuccess);
  EXPECT(p.mode == WorkspaceMode::Unified && p.unregisteredBytes == 0);
  // adjacent temps never overlap inside the arena
  for (size_t i = 0; i + 1 < p.regular.size(); ++i) {
    const StagePlan &a = p.regular[i], &b = p.regular[i + 1];
    if (!a.tempBytes || !b.tempBytes) continue;
    const bool disjoint = a.tempOffset + a.tempBytes <= b.tempOffset || b.tempOffset + b.tempBytes <= a.tempOffset;
    EXPECT(disjoint);
    EXPECT(a.tempOffset + a.tempBytes <= p.sliceArenaBytes && b.tempOffset + b.tempBytes <= p.sliceArenaBytes);
  }
}

TEST(plan_rejects_malformed_stage_lists) {
  fakes::knobs() = fakes::PluginKnobs();
  PlanFixture f;
  PipelinePlan p;
  std::string err;
  EXPECT(preparePipeline(f.spec(100, 8, {Stage::decompress()}), 1, &p, &err) != ncclSuccess);                      // nothing encoded
  EXPECT(preparePipeline(f.spec(100, 8, {Stage::compress(f.codec.get())}), 1, &p, &err) != ncclSuccess);            // ends encoded
  EXPECT(preparePipeline(f.spec(100, 6, {Stage::compress(f.codec.get()), Stage::allToAll(&f.comm), Stage::decompress()}), 1, &p, &err) != ncclSuccess);
  EXPECT(preparePipeline(f.spec(100, 8, {Stage::compress(f.codec.get()), Stage::allToAll(&f.comm), Stage::decompressReduce(3)}), 1, &p, &err) != ncclSuccess);
  EXPECT(preparePipeline(f.spec(0, 8, {Stage::compress(f.codec.get()), Stage::decompress()}), 1, &p, &err) != ncclSuccess);
}

namespace {
struct HostWorkspace : WorkspaceProvider {
  int acquired = 0, released = 0;
  ncclResult_t acquire(Comm*, size_t bytes, bool, cudaStream_t, void** ptr, void** lease) override {
    *ptr = malloc(bytes ? bytes : 1); *lease = *ptr; ++acquired; return ncclSuccess;
  }
  void release(void* lease, cudaStream_t) override { free(lease); ++released; }
};
}  // namespace

TEST(pipeline_serial_execution_flow_with_fakes) {
  fakes::knobs() = fakes::PluginKnobs();
  PlanFixture f;
  HostWorkspace ws;
  PipelineRuntime rt;
  rt.workspace = &ws;
  rt.alloc = &fakes::hostAllocator();
  rt.configuredDepth = 4;  // one node + fixed-size codec: forced back to depth 1
  // two-shot all-reduce: Compress -> A2A -> DRC -> AllGather -> Decompress
  PipelineSpec s = f.spec(1024, 8, {Stage::compress(f.codec.get()), Stage::allToAll(&f.comm), Stage::decompReduceComp(8, f.codec.get()),
                                    Stage::allGather(&f.comm), Stage::decompress()});
  EXPECT(runPipeline(s, rt) == ncclSuccess);
  fakes::PluginKnobs& k = fakes::knobs();
  EXPECT(k.compressCalls == 1 && k.drcCalls == 1 && k.decompressCalls == 1);
  EXPECT(f.transport.log.size() == 2 && f.transport.log[0] == "allToAll" && f.transport.log[1] == "allGather");
  EXPECT(ws.acquired == 1 && ws.released == 1);
  // codec without the fused ops: generic path = decode all + chunk reduction (+ re-encode)
  k = fakes::PluginKnobs();
  k.hasReduce = false; k.hasDrc = false;
  f.plugin.descriptor = fakes::fakePlugin("fake");
  static int reduceCalls = 0;
  reduceCalls = 0;
  setReduceChunksHook([](const void*, void*, long, int chunks, long, int, cudaStream_t) { ++reduceCalls; return chunks == 8 ? 0 : 1; });
  EXPECT(runPipelineSerial(s, rt) == ncclSuccess);
  EXPECT(k.compressCalls == 2 && k.decompressCalls == 2 && k.drcCalls == 0 && reduceCalls == 1);
  setReduceChunksHook(nullptr);
  // a failing transport surfaces as an error and the workspace is still returned
  f.transport.fail = ncclSystemError;
  const int rel = ws.released;
  EXPECT(runPipelineSerial(s, rt) == ncclSystemError);
  EXPECT(ws.released == rel + 1);
}

TEST(frame_exchange_slots_and_validation) {
  const size_t stride = 1024;
  std::vector<cocclCompressorFrameMetadata> sendMeta(8), recvMeta(8);
  for (int i = 0; i < 8; ++i) { sendMeta[i] = {(uint64_t)(100 + i), cocclCompressorFrameEncoded, 0}; recvMeta[i] = {(uint64_t)(200 + i), (uint32_t)(i % 2), 0}; }
  std::vector<FrameTransfer> sends, recvs;
  // all-to-all, 4 ranks x 2 frames: frames [2p, 2p+1] go to rank p, slots [2p, 2p+1] come from rank p
  EXPECT(buildFrameExchange(false, 1, 4, 2, stride, sendMeta.data(), recvMeta.data(), &sends, &recvs) == ncclSuccess);
  EXPECT(sends.size() == 8 && recvs.size() == 8);
  EXPECT(sends[5].peer == 2 && sends[5].sendOffset == 5 * stride && sends[5].sendBytes == 105);
  EXPECT(recvs[5].peer == 2 && recvs[5].recvOffset == 5 * stride && recvs[5].recvBytes == 205);
  // all-gather, 4 ranks x 2 frames: my 2 frames go to everyone
  EXPECT(buildFrameExchange(true, 1, 4, 2, stride, sendMeta.data(), recvMeta.data(), &sends, &recvs) == ncclSuccess);
  EXPECT(sends[5].peer == 2 && sends[5].sendOffset == 1 * stride && sends[5].sendBytes == 101);
  EXPECT(recvs[5].recvOffset == 5 * stride);
  // invalid metadata: empty payload, payload beyond the slot, unknown encoding
  EXPECT(!frameMetadataValid({0, cocclCompressorFrameEncoded, 0}, stride));
  EXPECT(!frameMetadataValid({stride + 1, cocclCompressorFrameRaw, 0}, stride));
  EXPECT(!frameMetadataValid({10, 7, 0}, stride));
  EXPECT(frameMetadataValid({stride, cocclCompressorFrameRaw, 0}, stride));
  recvMeta[3].payloadBytes = 0;
  EXPECT(buildFrameExchange(false, 1, 4, 2, stride, sendMeta.data(), recvMeta.data(), &sends, &recvs) == ncclInvalidUsage);
}

TEST(size_bound_query_rules) {
  fakes::knobs() = fakes::PluginKnobs();
  PlanFixture f;
  size_t b = 0;
  EXPECT(encodedSizeBound(f.codec.get(), cocclCompressorOperationCompress, 4096, 4, ncclFloat32, &b) == ncclSuccess && b == 4096);
  EXPECT(b % 4 == 0);
  fakes::knobs().sizeBoundUnknown = true;
  EXPECT(encodedSizeBound(f.codec.get(), cocclCompressorOperationCompress, 4096, 4, ncclFloat32, &b) == ncclSuccess && b == 16384);  // raw size
  EXPECT(encodedSizeBound(f.codec.get(), cocclCompressorOperationCompress, 4096, 0, ncclFloat32, &b) == ncclInvalidArgument);
  EXPECT(encodedSizeBound(nullptr, cocclCompressorOperationCompress, 4096, 4, ncclFloat32, &b) == ncclInvalidArgument);
}

TEST(host_api_scratch_persistent_state) {
  fakes::knobs() = fakes::PluginKnobs();
  // a codec that uses all three host services
  struct Probe {
    struct State { int uses = 0; };
    static coccl::Status compress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
      coccl::Buffer s1, s2, p;
      if (ctx.scratch(100, &s1) != ncclSuccess || ctx.scratch(50, &s2) != ncclSuccess) return ncclSystemError;
      if (ctx.persistent(3, 1000, &p) != ncclSuccess || p.bytes() < 1000) return ncclSystemError;
      State* st = nullptr;
      if (ctx.instance(&st) != ncclSuccess) return ncclSystemError;
      ++st->uses;
      return out.commitBytes(in.bytes() / 2 + (size_t)st->uses * 0, in.chunks());
    }
    static coccl::Status decompress(const coccl::Input&, coccl::Output&, coccl::Context&) { return ncclSuccess; }
  };
  LoadedPlugin pl;
  pl.name = "probe";
  pl.descriptor = coccl::PluginAdapter<Probe>::descriptor("probe");
  void* cfg = nullptr;
  char err[64];
  cocclConfigView empty{nullptr, 0};
  cocclCompressorConfigContext cc{cocclCompressorConfigDefault, 1, 8};
  EXPECT(pl.descriptor->parseConfig(&empty, &cc, &cfg, err, sizeof(err)) == ncclSuccess);
  fakes::allocLog() = fakes::AllocLog();
  {
    CompressorPolicy policy(&pl, cfg, 0, "probe");
    ExecEnv env;
    env.alloc = &fakes::hostAllocator();
    char in[256], outb[256];
    cocclCompressorView iv{in, 256, 256, 64, 1, ncclFloat32, nullptr, 0};
    cocclCompressorView ov{outb, 256, 0, 256, 1, ncclInt8, nullptr, 0};
    EXPECT(compress(&policy, iv, &ov, env) == ncclSuccess && ov.bytes == 128);
    EXPECT(compress(&policy, iv, &ov, env) == ncclSuccess);
    fakes::AllocLog& l = fakes::allocLog();
    EXPECT(l.asyncMallocs == 4 && l.asyncFrees == 4);  // scratch is returned after every call
    EXPECT(l.mallocs == 1);                            // persistent slot allocated once
    EXPECT(policy.resources(0).scratchPeak == 150 && policy.resources(0).persistentBytes == 1000);
    EXPECT(policy.resources(0).states.size() == 1);
    policy.releaseResources(fakes::hostAllocator());
    EXPECT(l.frees == 1);
  }
}
