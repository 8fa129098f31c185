// Router acceptance matrix, explicit calls, group batching, hierarchy cache, recipes.
// Scenarios follow tests/coccl-tests/src/coccl_runtime_test.cc:300-525, coccl_group_test.cc,
// coccl_allreduce_recipe_test.cc:56-80 and coccl_reducescatter_recipe_test.cc of the reference.
#include <chrono>

#include "fakes.h"
#include "host_test.h"
#include "runtime/primitives.h"
#include "runtime/runtime.h"
#include "tuning/autotune.h"
#include "tuning/measured.h"

using namespace coccl;
using fakes::FakeTransport;

namespace {

struct CountingExecutor : Executor {
  int executed = 0, batches = 0, batchCalls = 0;
  std::vector<Algorithm> algorithms;
  ncclResult_t execute(Runtime*, const PreparedCall& c) override { ++executed; algorithms.push_back(c.algorithm); return ncclSuccess; }
  ncclResult_t executeSendRecvBatch(Runtime*, const std::vector<PreparedCall>& b) override { ++batches; batchCalls += (int)b.size(); return ncclSuccess; }
};

struct FixedRoles : RoleOracle {
  Role role = Role::Unknown;
  int observed = 0;
  void observe(const CallInfo&, int) override { ++observed; }
  Role roleOf(Comm*) override { return role; }
};

std::string configText(const char* mode, const char* body, size_t threshold = 1024) {
  std::string s = "[runtime]\nmode = \"" + std::string(mode) + "\"\ncompression_threshold_bytes = " + std::to_string(threshold) +
                  "\n[compressor_plugins]\ncompressors = [\"fake\"]\nlibrary_path = \"/nowhere\"\n";
  if (std::string(mode) == "training")
    s += "[training.classifier]\ndata_parallel_size = 4\ntensor_parallel_size = 2\npipeline_parallel_size = 2\n";
  return s + body;
}

struct Fixture {
  Runtime rt;
  FakeTransport transport;
  CountingExecutor exec;
  ModelStore store;
  AutotuneSelector selector{&store};
  Comm comm;
  char send[64], recv[64];
  Fixture(const char* mode, const char* body, int nRanks = 8, int nNodes = 1, size_t threshold = 1024) {
    fakes::knobs() = fakes::PluginKnobs();
    comm = fakes::makeComm(&transport, 1, nRanks, nNodes);
    Config cfg;
    std::string err;
    bool ok = loadConfigText(configText(mode, body, threshold), ".", &cfg, &err);
    if (!ok) fprintf(stderr, "  fixture config error: %s\n", err.c_str());
    rt.compressors().addBuiltin(fakes::fakePlugin("fake"));
    if (rt.enable(cfg, nNodes, nRanks / nNodes, &err) != ncclSuccess) fprintf(stderr, "  fixture enable error: %s\n", err.c_str());
    rt.setExecutor(&exec);
    rt.setSelector(&selector);
  }
  CallInfo coll(Operation op, size_t count, ncclDataType_t t = ncclFloat32, ncclRedOp_t red = ncclSum) {
    CallInfo i;
    i.op = op; i.sendbuff = send; i.recvbuff = recv; i.count = count; i.datatype = t; i.redOp = red; i.comm = &comm;
    return i;
  }
  CallInfo p2p(bool isSend, int peer, size_t count) {
    CallInfo i;
    i.op = Operation::SendRecv; i.func = isSend ? Func::Send : Func::Recv; i.sendbuff = isSend ? send : nullptr;
    i.recvbuff = isSend ? nullptr : recv; i.count = count; i.peer = peer; i.comm = &comm;
    return i;
  }
};

const char* kAllOps =
    "[normal.all_reduce.default]\ncompressor = \"fake\"\n[normal.reduce_scatter.default]\ncompressor = \"fake\"\n"
    "[normal.all_gather.default]\ncompressor = \"fake\"\n[normal.all_to_all.default]\ncompressor = \"fake\"\n"
    "[normal.sendrecv.default]\ncompressor = \"fake\"\n";

}  // namespace

TEST(router_disabled_does_no_lookups) {
  Runtime rt;
  FakeTransport t;
  Comm c = fakes::makeComm(&t, 0, 8, 1);
  CallInfo i;
  char b[8];
  i.op = Operation::AllReduce; i.sendbuff = b; i.recvbuff = b; i.count = 1 << 20; i.comm = &c;
  bool taken = true;
  EXPECT(rt.enqueueCheck(i, &taken) == ncclSuccess && !taken);
  EXPECT_EQ(rt.stats().policyLookups, (uint64_t)0);
  EXPECT(rt.enqueueExplicit(i, Algorithm::ArTwoShot) == ncclInvalidUsage);
}

TEST(router_threshold_sum_divisibility_and_bytes_scaling) {
  Fixture f("normal", kAllOps);
  bool taken = false;
  // 256 floats = 1024 bytes: not larger than the threshold -> native (<= rule)
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 256), &taken) == ncclSuccess && !taken);
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 264), &taken) == ncclSuccess && taken);
  EXPECT_EQ(f.exec.executed, 1);
  // all-gather bytes are scaled by the number of ranks: 40 floats * 8 ranks = 1280 B > 1024
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 40), &taken) == ncclSuccess && taken);
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 32), &taken) == ncclSuccess && !taken);
  // non-sum reductions stay native
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 4096, ncclFloat32, ncclMax), &taken) == ncclSuccess && !taken);
  // all-reduce count not divisible by the ranks: native, and no policy lookup at all
  const uint64_t before = f.rt.stats().policyLookups;
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 4097), &taken) == ncclSuccess && !taken);
  EXPECT_EQ(f.rt.stats().policyLookups, before);
  // null buffers, zero count, single rank
  CallInfo bad = f.coll(Operation::ReduceScatter, 4096);
  bad.recvbuff = nullptr;
  EXPECT(f.rt.enqueueCheck(bad, &taken) == ncclSuccess && !taken);
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::ReduceScatter, 0), &taken) == ncclSuccess && !taken);
  f.comm.nRanks = 1;
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096), &taken) == ncclSuccess && !taken);
}

TEST(router_datatypes_lossy_vs_lossless) {
  {
    Fixture f("normal", kAllOps);
    bool taken = true;
    const uint64_t before = f.rt.stats().policyLookups;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096, ncclInt8), &taken) == ncclSuccess && !taken);
    EXPECT_EQ(f.rt.stats().policyLookups - before, (uint64_t)3);  // the three scopes were consulted
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096, ncclBfloat16), &taken) == ncclSuccess && taken);
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096, ncclFloat64), &taken) == ncclSuccess && !taken);
    // explicit call with an unsupported datatype: replayed natively, success
    const int native = f.transport.nativeCalls;
    EXPECT(f.rt.enqueueExplicit(f.coll(Operation::AllGather, 4096, ncclInt8), Algorithm::None) == ncclSuccess);
    EXPECT_EQ(f.transport.nativeCalls, native + 1);
  }
  {
    Fixture f("normal", kAllOps);
    f.rt.disable();
    fakes::knobs().lossless = true;
    Config cfg;
    std::string err;
    loadConfigText(configText("normal", kAllOps), ".", &cfg, &err);
    f.rt.compressors().addBuiltin(fakes::fakePlugin("fake"));
    f.rt.enable(cfg, 1, 8, &err);
    f.rt.setExecutor(&f.exec);
    f.rt.setSelector(&f.selector);
    bool taken = false;
    for (ncclDataType_t t : {ncclInt8, ncclInt32, ncclInt64}) {
      EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096, t), &taken) == ncclSuccess && taken);
    }
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096, ncclUint8), &taken) == ncclSuccess && !taken);
  }
}

TEST(router_explicit_ignores_threshold_and_needs_policy) {
  Fixture f("normal", "[normal.all_gather.default]\ncompressor = \"fake\"\n", 8, 1, (size_t)-1 >> 1);
  bool taken = true;
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 1 << 20), &taken) == ncclSuccess && !taken);  // huge threshold
  EXPECT(f.rt.enqueueExplicit(f.coll(Operation::AllGather, 16), Algorithm::None) == ncclSuccess);
  EXPECT_EQ(f.exec.executed, 1);
  // no policy for all-to-all: explicit call is a usage error, implicit call stays native
  EXPECT(f.rt.enqueueExplicit(f.coll(Operation::AllToAll, 16), Algorithm::None) == ncclInvalidUsage);
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllToAll, 1 << 20), &taken) == ncclSuccess && !taken);
}

TEST(router_single_node_uses_intra_scope) {
  {
    Fixture f("normal", "[normal.all_gather.inter]\ncompressor = \"fake\"\n");
    bool taken = true;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096), &taken) == ncclSuccess && !taken);  // inter-only policy, one node
  }
  {
    Fixture f("normal", "[normal.all_gather.intra]\ncompressor = \"fake\"\n");
    bool taken = false;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096), &taken) == ncclSuccess && taken);
  }
  {
    Fixture f("normal", "[normal.all_gather.intra]\ncompressor = \"fake\"\n", 16, 2);
    bool taken = true;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096), &taken) == ncclSuccess && !taken);  // two nodes need the default scope
  }
}

TEST(router_sendrecv_scope_by_peer_node_and_direction) {
  Fixture f("normal", "[normal.sendrecv.inter]\ncompressor = \"fake\"\n", 16, 2);  // rank 1 lives on node 0
  bool taken = true;
  EXPECT(f.rt.enqueueCheck(f.p2p(true, 2, 4096), &taken) == ncclSuccess && !taken);   // peer on my node: intra scope, none configured
  EXPECT(f.rt.enqueueCheck(f.p2p(true, 9, 4096), &taken) == ncclSuccess && taken);    // peer on the other node
  // training mode, pipeline role: forward iff rank < peer on send, rank > peer on recv
  Fixture g("training", "[training.pp.sendrecv.forward.default]\ncompressor = \"fake\"\n");
  FixedRoles roles;
  roles.role = Role::PipelineParallel;
  g.rt.setRoleOracle(&roles);
  EXPECT(g.rt.enqueueCheck(g.p2p(true, 5, 4096), &taken) == ncclSuccess && taken);    // rank 1 -> 5: forward
  EXPECT(g.rt.enqueueCheck(g.p2p(true, 0, 4096), &taken) == ncclSuccess && !taken);   // 1 -> 0: backward, no policy
  EXPECT(g.rt.enqueueCheck(g.p2p(false, 0, 4096), &taken) == ncclSuccess && taken);   // recv from 0: forward
  EXPECT(roles.observed >= 3);
}

TEST(router_training_mode_unknown_role_is_native) {
  Fixture f("training", "[training.dp.reduce_scatter.default]\ncompressor = \"fake\"\n");
  FixedRoles roles;
  f.rt.setRoleOracle(&roles);
  bool taken = true;
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::ReduceScatter, 4096), &taken) == ncclSuccess && !taken);
  EXPECT(f.rt.enqueueExplicit(f.coll(Operation::ReduceScatter, 4096), Algorithm::RsOneShot) == ncclInvalidUsage);
  roles.role = Role::DataParallel;
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::ReduceScatter, 4096), &taken) == ncclSuccess && taken);
  roles.role = Role::TensorParallel;  // no TP policy configured
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::ReduceScatter, 4096), &taken) == ncclSuccess && !taken);
}

TEST(router_algorithm_selection_rules) {
  {  // one node: reduce-scatter one-shot, all-reduce two-shot by heuristic
    Fixture f("normal", kAllOps);
    bool taken;
    f.rt.enqueueCheck(f.coll(Operation::ReduceScatter, 4096), &taken);
    f.rt.enqueueCheck(f.coll(Operation::AllReduce, 4096), &taken);
    EXPECT(f.exec.algorithms.size() == 2 && f.exec.algorithms[0] == Algorithm::RsOneShot && f.exec.algorithms[1] == Algorithm::ArTwoShot);
  }
  {  // two nodes, only an intra codec: reduce-scatter still goes two-shot
    Fixture f("normal", "[normal.reduce_scatter.intra]\ncompressor = \"fake\"\n", 16, 2);
    bool taken = false;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::ReduceScatter, 4096), &taken) == ncclSuccess && taken);
    EXPECT(f.exec.algorithms.back() == Algorithm::RsTwoShot);
  }
  {  // two nodes, only an inter codec
    Fixture f("normal", "[normal.reduce_scatter.inter]\ncompressor = \"fake\"\n", 16, 2);
    bool taken = false;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::ReduceScatter, 4096), &taken) == ncclSuccess && taken);
    EXPECT(f.exec.algorithms.back() == Algorithm::RsTwoShot);
  }
  {  // forced triple-shot is honoured with only a default codec
    Fixture f("normal", "[autotune]\nall_reduce_algorithm = \"tripleshot\"\n[normal.all_reduce.default]\ncompressor = \"fake\"\n", 16, 2);
    bool taken = false;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 4096), &taken) == ncclSuccess && taken);
    EXPECT(f.exec.algorithms.back() == Algorithm::ArTripleShot);
  }
  {  // forced two-shot reduce-scatter on one node falls back to one-shot
    Fixture f("normal", "[autotune]\nreduce_scatter_algorithm = \"twoshot\"\n[normal.reduce_scatter.default]\ncompressor = \"fake\"\n");
    bool taken = false;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::ReduceScatter, 4096), &taken) == ncclSuccess && taken);
    EXPECT(f.exec.algorithms.back() == Algorithm::RsOneShot);
  }
}

TEST(group_defers_and_batches) {
  Fixture f("normal", kAllOps);
  bool taken = false;
  f.rt.groupStart();
  f.transport.groupStart();
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096), &taken) == ncclSuccess && taken);
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllToAll, 4096), &taken) == ncclSuccess && taken);
  EXPECT_EQ(f.exec.executed, 0);  // deferred, nothing executed inside the group
  EXPECT(f.rt.groupHasPending());
  EXPECT(f.rt.groupEnd(&f.transport, false) == ncclSuccess);
  EXPECT_EQ(f.exec.executed, 2);  // collectives one by one after the transport group was flushed
  EXPECT(f.transport.log.back() == "groupEnd");
  // send/recv batch runs as ONE unit
  f.rt.groupStart();
  f.transport.groupStart();
  f.rt.enqueueCheck(f.p2p(true, 2, 4096), &taken);
  f.rt.enqueueCheck(f.p2p(false, 0, 4096), &taken);
  EXPECT(f.rt.groupEnd(&f.transport, false) == ncclSuccess);
  EXPECT(f.exec.batches == 1 && f.exec.batchCalls == 2);
}

TEST(group_replays_natively_when_mixed_or_native_pending) {
  Fixture f("normal", kAllOps);
  bool taken = false;
  // a grouped send below the threshold is queued as a native entry -> whole batch native
  f.rt.groupStart();
  f.transport.groupStart();
  EXPECT(f.rt.enqueueCheck(f.p2p(true, 2, 4096), &taken) == ncclSuccess && taken);
  EXPECT(f.rt.enqueueCheck(f.p2p(false, 0, 8), &taken) == ncclSuccess && taken);  // below threshold, still queued
  EXPECT(f.rt.groupEnd(&f.transport, false) == ncclSuccess);
  EXPECT(f.exec.batches == 0 && f.transport.nativeCalls == 2);
  // send/recv mixed with a collective -> native
  f.rt.groupStart();
  f.transport.groupStart();
  f.rt.enqueueCheck(f.p2p(true, 2, 4096), &taken);
  f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096), &taken);
  EXPECT(f.rt.groupEnd(&f.transport, false) == ncclSuccess);
  EXPECT(f.exec.executed == 0 && f.exec.batches == 0 && f.transport.nativeCalls == 4);
  // native work pending in the transport's group -> native
  f.rt.groupStart();
  f.transport.groupStart();
  f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096), &taken);
  EXPECT(f.rt.groupEnd(&f.transport, true) == ncclSuccess);
  EXPECT(f.exec.executed == 0 && f.transport.nativeCalls == 5);
  // abort clears what is pending
  f.rt.groupStart();
  f.rt.enqueueCheck(f.coll(Operation::AllGather, 4096), &taken);
  f.rt.groupAbort();
  EXPECT(!f.rt.groupHasPending());
  f.transport.groupStart();
  f.rt.groupEnd(&f.transport, false);
}

TEST(router_internal_calls_bypass_and_overhead) {
  Fixture f("normal", kAllOps);
  struct Reentrant : Executor {
    Runtime* rt; CallInfo inner; bool innerTaken = true;
    ncclResult_t execute(Runtime* r, const PreparedCall&) override { return r->enqueueCheck(inner, &innerTaken); }
    ncclResult_t executeSendRecvBatch(Runtime*, const std::vector<PreparedCall>&) override { return ncclSuccess; }
  } re;
  re.inner = f.coll(Operation::AllGather, 4096);
  f.rt.setExecutor(&re);
  bool taken = false;
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllToAll, 4096), &taken) == ncclSuccess && taken);
  EXPECT(!re.innerTaken);  // the runtime's own calls are never routed again
  f.rt.setExecutor(&f.exec);
  // overhead of the two cheapest decisions, reported for information
  const int iters = 200000;
  CallInfo small = f.coll(Operation::AllGather, 8);
  auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < iters; ++i) f.rt.enqueueCheck(small, &taken);
  auto t1 = std::chrono::steady_clock::now();
  f.rt.disable();
  for (int i = 0; i < iters; ++i) f.rt.enqueueCheck(small, &taken);
  auto t2 = std::chrono::steady_clock::now();
  printf("  router overhead: below-threshold %.0f ns/call, disabled %.0f ns/call\n",
         std::chrono::duration<double, std::nano>(t1 - t0).count() / iters,
         std::chrono::duration<double, std::nano>(t2 - t1).count() / iters);
}

TEST(hierarchy_cache_and_recipes) {
  Fixture f("normal", "[normal.reduce_scatter.default]\ncompressor = \"fake\"\n[normal.all_reduce.default]\ncompressor = \"fake\"\n"
                      "[normal.all_gather.default]\ncompressor = \"fake\"\n[normal.all_to_all.default]\ncompressor = \"fake\"\n", 16, 2);
  Comm *intra = nullptr, *inter = nullptr;
  EXPECT(f.rt.hierarchy(&f.comm, &intra, &inter) == ncclSuccess);
  EXPECT(intra && inter && intra->nRanks == 8 && inter->nRanks == 2 && intra->isChild && inter->nNodes == 2);
  Comm *i2 = nullptr, *x2 = nullptr;
  EXPECT(f.rt.hierarchy(&f.comm, &i2, &x2) == ncclSuccess && i2 == intra && x2 == inter);
  EXPECT_EQ(f.transport.splits, 2);  // created once
  EXPECT(f.rt.hierarchy(intra, &i2, &x2) == ncclInvalidUsage);  // children own no hierarchy

  auto prepared = [&](Operation op, Algorithm a, size_t count) {
    PreparedCall p;
    p.info = f.coll(op, count);
    p.desc = describe(op);
    p.algorithm = a;
    for (int s = 0; s < 3; ++s) { p.codecs[s] = f.rt.compressors().resolve(Role::Normal, Variant::Default, op, (Scope)s); p.datatypeOk[s] = p.codecs[s] != nullptr; }
    return p;
  };
  PipelineSpec spec;
  EXPECT(buildRecipe(prepared(Operation::AllGather, Algorithm::None, 100), nullptr, nullptr, &spec) == ncclSuccess);
  EXPECT(spec.stages.size() == 3 && spec.stages[0].kind == StageKind::Compress && spec.stages[1].kind == StageKind::AllGather &&
         spec.stages[2].kind == StageKind::Decompress && spec.inputChunks == 1 && spec.inPlace == InPlaceLayout::InputRankChunk);
  EXPECT(buildRecipe(prepared(Operation::AllToAll, Algorithm::None, 100), nullptr, nullptr, &spec) == ncclSuccess);
  EXPECT(spec.stages[1].kind == StageKind::AllToAll && spec.inputChunks == 16 && spec.inPlace == InPlaceLayout::None);
  EXPECT(buildRecipe(prepared(Operation::ReduceScatter, Algorithm::RsOneShot, 100), nullptr, nullptr, &spec) == ncclSuccess);
  EXPECT(spec.stages.size() == 3 && spec.stages[2].kind == StageKind::DecompressReduce && spec.stages[2].reduceChunks == 16 &&
         spec.inPlace == InPlaceLayout::OutputRankChunk);
  EXPECT(buildRecipe(prepared(Operation::ReduceScatter, Algorithm::RsTwoShot, 100), intra, inter, &spec) == ncclSuccess);
  EXPECT(spec.inputLayout == InputLayout::HierarchicalSwizzle && spec.stages.size() == 5);
  EXPECT(spec.stages[1].kind == StageKind::AllToAll && spec.stages[1].comm == intra && spec.stages[2].kind == StageKind::DecompReduceComp &&
         spec.stages[2].reduceChunks == 8 && spec.stages[3].comm == inter && spec.stages[4].kind == StageKind::DecompressReduce &&
         spec.stages[4].reduceChunks == 2);
  EXPECT(buildRecipe(prepared(Operation::AllReduce, Algorithm::ArOneShot, 1600), nullptr, nullptr, &spec) == ncclSuccess);
  EXPECT(spec.rawChunkCount == 100 && spec.stages[1].kind == StageKind::AllGather && spec.stages[2].reduceChunks == 16);
  EXPECT(buildRecipe(prepared(Operation::AllReduce, Algorithm::ArTwoShot, 1600), nullptr, nullptr, &spec) == ncclSuccess);
  EXPECT(spec.stages.size() == 5 && spec.stages[2].kind == StageKind::DecompReduceComp && spec.stages[3].kind == StageKind::AllGather &&
         spec.stages[4].kind == StageKind::Decompress && spec.inPlace == InPlaceLayout::SameBuffer);
  EXPECT(buildRecipe(prepared(Operation::AllReduce, Algorithm::ArTripleShot, 1600), intra, inter, &spec) == ncclSuccess);
  EXPECT(spec.stages.size() == 7 && spec.stages[4].kind == StageKind::DecompReduceComp && spec.stages[5].kind == StageKind::AllGather &&
         spec.stages[5].comm == &f.comm && spec.stages[6].kind == StageKind::Decompress);
  // a hierarchy level without codec reduces natively
  Fixture g("normal", "[normal.reduce_scatter.inter]\ncompressor = \"fake\"\n", 16, 2);
  PreparedCall p;
  p.info = g.coll(Operation::ReduceScatter, 100);
  p.desc = describe(Operation::ReduceScatter);
  p.algorithm = Algorithm::RsTwoShot;
  p.codecs[(int)Scope::Inter] = g.rt.compressors().resolve(Role::Normal, Variant::Default, Operation::ReduceScatter, Scope::Inter);
  EXPECT(buildRecipe(p, intra, inter, &spec) == ncclSuccess);
  EXPECT(spec.stages[0].kind == StageKind::ReduceScatter && spec.stages[1].kind == StageKind::Compress && spec.stages[2].kind == StageKind::AllToAll);
  f.rt.commDestroy(&f.comm);
  EXPECT(f.comm.intra == nullptr && f.comm.inter == nullptr);
}

// ---------------------------------------------------------------------------- measured selection (tuning/measured.h)
namespace {
// One-shot costs a fixed 10 us plus 4 ns per KiB, two-shot 30 us plus 1 ns per KiB: they cross near 6.7 MiB.
struct FakeTimer : AlgorithmTimer {
  int asked = 0, timed = 0;
  bool allow = true, failTwoShot = false;
  bool measurable(Runtime*, const PreparedCall&) override { ++asked; return allow; }
  bool time(Runtime*, const PreparedCall& call, Algorithm a, double* seconds) override {
    ++timed;
    if (failTwoShot && a == Algorithm::ArTwoShot) return false;
    const double kib = (double)(call.info.count * cocclTypeSize(call.info.datatype)) / 1024.0;
    *seconds = a == Algorithm::ArOneShot ? 10e-6 + 4e-9 * kib : 30e-6 + 1e-9 * kib;
    return true;
  }
};
const char* kAutotuneAr = "[autotune]\nenabled = true\n[normal.all_reduce.default]\ncompressor = \"fake\"\n"
                          "[normal.reduce_scatter.default]\ncompressor = \"fake\"\n";
}  // namespace

TEST(measured_selector_times_each_bucket_once_and_picks_the_faster) {
  Fixture f("normal", kAutotuneAr);
  MeasuredTable table;
  FakeTimer timer;
  MeasuredSelector sel(&f.store, &table, &timer);
  f.rt.setSelector(&sel);
  bool taken = false;
  // 1 MiB: one-shot wins (14 us against 31 us); the second call of the bucket is not timed again
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 1 << 18), &taken) == ncclSuccess && taken);
  EXPECT(f.exec.algorithms.back() == Algorithm::ArOneShot && timer.timed == 2 && sel.measuredBuckets() == 1);
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, (1 << 18) + 8), &taken) == ncclSuccess && taken);
  EXPECT(f.exec.algorithms.back() == Algorithm::ArOneShot && timer.timed == 2);
  // 64 MiB: its own bucket, two-shot wins (96 us against 272 us)
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 1 << 24), &taken) == ncclSuccess && taken);
  EXPECT(f.exec.algorithms.back() == Algorithm::ArTwoShot && timer.timed == 4 && table.size() == 2);
  // reduce-scatter on one node has a single flat algorithm: never timed
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::ReduceScatter, 1 << 18), &taken) == ncclSuccess && taken);
  EXPECT(f.exec.algorithms.back() == Algorithm::RsOneShot && timer.timed == 4);
  // inside a group nothing is timed; the nearest measured bucket decides
  f.rt.groupStart();
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 1 << 21), &taken) == ncclSuccess && taken);
  EXPECT(timer.timed == 4);
  EXPECT(f.rt.groupEnd(&f.transport, false) == ncclSuccess);
  EXPECT(f.exec.algorithms.back() == Algorithm::ArOneShot);   // 8 MiB falls back on the 1 MiB bucket below it
}

TEST(measured_selector_times_every_communicator_on_its_own) {
  // A rank belongs to several communicators of the same size (tensor- and data-parallel groups of two, say). Whether a
  // call is timed may depend on that communicator's history only: its other ranks have not seen this rank's calls
  // elsewhere, and would wait in the collective timing for a rank that skipped it.
  Fixture f("normal", kAutotuneAr);
  MeasuredTable table;
  FakeTimer timer;
  MeasuredSelector sel(&f.store, &table, &timer);
  f.rt.setSelector(&sel);
  Comm other = fakes::makeComm(&f.transport, 1, 8, 1);
  other.id = f.comm.id + 1000;
  bool taken = false;
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 1 << 18), &taken) == ncclSuccess && taken);
  EXPECT(timer.timed == 2);
  CallInfo i = f.coll(Operation::AllReduce, 1 << 18);
  i.comm = &other;
  EXPECT(f.rt.enqueueCheck(i, &taken) == ncclSuccess && taken);
  EXPECT(timer.timed == 4 && sel.measuredBuckets() == 2 && table.size() == 2);
  // entries of one communicator do not decide for the other: a bucket only the first one has measured
  EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 1 << 24), &taken) == ncclSuccess && taken);
  EXPECT(f.exec.algorithms.back() == Algorithm::ArTwoShot && timer.timed == 6);
  timer.allow = false;
  i = f.coll(Operation::AllReduce, 1 << 24);
  i.comm = &other;
  EXPECT(f.rt.enqueueCheck(i, &taken) == ncclSuccess && taken);
  EXPECT(f.exec.algorithms.back() == Algorithm::ArOneShot && timer.timed == 6);   // its own 1 MiB entry, the nearest below
}

TEST(measured_selector_failures_forced_algorithms_and_disabled_autotune) {
  {  // a candidate that cannot be timed gets no entry; the other one is chosen; the bucket is not tried again
    Fixture f("normal", kAutotuneAr);
    MeasuredTable table;
    FakeTimer timer;
    timer.failTwoShot = true;
    MeasuredSelector sel(&f.store, &table, &timer);
    f.rt.setSelector(&sel);
    bool taken = false;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 1 << 24), &taken) == ncclSuccess && taken);
    EXPECT(f.exec.algorithms.back() == Algorithm::ArOneShot && timer.timed == 2);
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 1 << 24), &taken) == ncclSuccess && taken);
    EXPECT(timer.timed == 2);
  }
  {  // calls that cannot be timed are asked about once per bucket and fall back on the model / heuristics
    Fixture f("normal", kAutotuneAr);
    MeasuredTable table;
    FakeTimer timer;
    timer.allow = false;
    MeasuredSelector sel(&f.store, &table, &timer);
    f.rt.setSelector(&sel);
    bool taken = false;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 1 << 18), &taken) == ncclSuccess && taken);
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 1 << 18), &taken) == ncclSuccess && taken);
    EXPECT(timer.asked == 1 && timer.timed == 0 && table.empty() && f.exec.algorithms.back() == Algorithm::ArTwoShot);
  }
  {  // a forced algorithm and a disabled autotuner bypass both the table and the timer
    Fixture f("normal", "[autotune]\nenabled = true\nall_reduce_algorithm = \"twoshot\"\n[normal.all_reduce.default]\ncompressor = \"fake\"\n");
    MeasuredTable table;
    table.set((int)Operation::AllReduce, (int)ncclFloat32, 8, 20, (int)Algorithm::ArOneShot, 1e-6);
    FakeTimer timer;
    MeasuredSelector sel(&f.store, &table, &timer);
    f.rt.setSelector(&sel);
    bool taken = false;
    EXPECT(f.rt.enqueueCheck(f.coll(Operation::AllReduce, 1 << 18), &taken) == ncclSuccess && taken);
    EXPECT(f.exec.algorithms.back() == Algorithm::ArTwoShot && timer.asked == 0);
    Fixture g("normal", "[autotune]\nenabled = false\n[normal.all_reduce.default]\ncompressor = \"fake\"\n");
    MeasuredSelector sel2(&g.store, &table, &timer);
    g.rt.setSelector(&sel2);
    EXPECT(g.rt.enqueueCheck(g.coll(Operation::AllReduce, 1 << 18), &taken) == ncclSuccess && taken);
    EXPECT(g.exec.algorithms.back() == Algorithm::ArTwoShot && timer.asked == 0);
  }
}
