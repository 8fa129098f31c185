// Buffer manager (slice + VMM backends with fake CUDA), autotune cost model / selector, training
// classifier and assist. Scenario sources: coccl_buffer_manager_test.cc, coccl_vmm_buffer_test.cc:48-120,
// coccl_autotune_test.cc:63-185, coccl_training_classifier_test.cc:1121-1153 of the reference.
#include <math.h>
#include <algorithm>

#include "fakes.h"
#include "host_test.h"
#include "memory/buffer_manager.h"
#include "training/assist.h"
#include "training/classifier.h"
#include "tuning/autotune.h"

using namespace coccl;

// ------------------------------------------------------------------ memory
TEST(slice_backend_reuse_pending_and_merge) {
  fakes::allocLog() = fakes::AllocLog();
  fakes::liveEvents().clear();
  SliceBackend b(&fakes::hostAllocator(), &fakes::fakeEvents(), 1 << 20);
  cudaStream_t s1 = reinterpret_cast<cudaStream_t>(0x10), s2 = reinterpret_cast<cudaStream_t>(0x20);
  void *p1, *p2, *p3;
  int blk, a, c, d;
  EXPECT(b.acquire(1000, s1, &p1, &blk, &a) == ncclSuccess);
  EXPECT(b.acquire(5000, s1, &p2, &blk, &c) == ncclSuccess);
  EXPECT_EQ(fakes::allocLog().mallocs, 1);  // both from one block
  EXPECT((char*)p2 - (char*)p1 == 1024);    // 256-byte aligned slices
  EXPECT(b.release(0, a, s1) == ncclSuccess);
  // pending slice: same stream takes it without waiting, another stream must wait for the event
  EXPECT(b.acquire(512, s2, &p3, &blk, &d) == ncclSuccess);
  EXPECT(p3 != p1);
  EXPECT(b.release(0, d, s2) == ncclSuccess);
  void* p4;
  int e;
  EXPECT(b.acquire(512, s1, &p4, &blk, &e) == ncclSuccess);
  EXPECT(p4 == p1);
  EXPECT(b.release(0, e, s1) == ncclSuccess);
  EXPECT(b.release(0, c, s1) == ncclSuccess);
  // once the events have completed everything merges back into one slice that serves a big request
  fakes::completeAllEvents();
  void* big;
  int g;
  EXPECT(b.acquire(1 << 20, s2, &big, &blk, &g) == ncclSuccess);
  EXPECT(big == p1 && fakes::allocLog().mallocs == 1);
  EXPECT(b.release(0, 12345, s1) == ncclInvalidArgument);
  // a request larger than the block size gets its own block
  void* huge;
  EXPECT(b.acquire(3 << 20, s1, &huge, &blk, &g) == ncclSuccess);
  EXPECT(blk == 1 && fakes::allocLog().mallocs == 2 && b.reservedBytes() == (1u << 20) + (3u << 20));
}

TEST(vmm_backend_maps_peers_and_grows_in_place) {
  fakes::vmmLog() = fakes::VmmLog();
  {
    VmmBackend v(&fakes::fakeVmm(), 1, 8 << 20);
    void* p;
    int blk, sl;
    EXPECT(v.acquire(10 << 20, nullptr, &p, &blk, &sl) == ncclSuccess);  // 2 chunks of 8 MiB
    EXPECT(v.chunks() == 2 && v.reservedBytes() == (16u << 20));
    auto& log = fakes::vmmLog().calls;
    auto has = [&](const std::string& s) { return std::find(log.begin(), log.end(), s) != log.end(); };
    EXPECT(log[0] == "granularity");
    EXPECT(has("create:8388608") && has("reserve:16777216") && has("map:1:8388608") && has("map:2:8388608"));
    EXPECT(has("setAccess:16777216x4"));  // read/write for every peer-accessible device
    EXPECT(v.acquire(1, nullptr, &p, &blk, &sl) == ncclInvalidUsage);  // one lease at a time
    EXPECT(v.release(0, 0, nullptr) == ncclSuccess);
    // growing: a larger range is reserved, the OLD handles are mapped again, then the new one
    const size_t before = log.size();
    void* q;
    EXPECT(v.acquire(20 << 20, nullptr, &q, &blk, &sl) == ncclSuccess);
    EXPECT(v.chunks() == 3 && q != p);
    std::vector<std::string> tail(log.begin() + before, log.end());
    auto pos = [&](const std::string& s) { return std::find(tail.begin(), tail.end(), s) - tail.begin(); };
    EXPECT(pos("create:8388608") < pos("reserve:25165824"));
    EXPECT(pos("unmap:16777216") < pos("addressFree:16777216"));
    EXPECT(pos("map:1:8388608") < pos("map:3:8388608"));
    EXPECT(pos("setAccess:25165824x4") < (long)tail.size());
    // a smaller request reuses the mapping
    v.release(0, 0, nullptr);
    const size_t n = log.size();
    EXPECT(v.acquire(1 << 20, nullptr, &p, &blk, &sl) == ncclSuccess && log.size() == n && p == q);
  }
  auto& log = fakes::vmmLog().calls;
  EXPECT(std::count(log.begin(), log.end(), "release") == 3);  // destructor returns every chunk
  EXPECT(log.back() == "addressFree:25165824");
}

TEST(buffer_manager_pools_and_backends) {
  fakes::allocLog() = fakes::AllocLog();
  fakes::vmmLog() = fakes::VmmLog();
  fakes::FakeTransport t;
  Comm a = fakes::makeComm(&t, 0, 8, 1), b = fakes::makeComm(&t, 1, 8, 1);
  BufferOptions opt;
  opt.alloc = &fakes::hostAllocator();
  opt.events = &fakes::fakeEvents();
  opt.vmm = &fakes::fakeVmm();
  {
    BufferManager m(opt);
    m.commInit(&a);
    BufferLease l1, l2, l3;
    EXPECT(m.getBuffer(&a, 1 << 20, true, nullptr, &l1) == ncclSuccess && l1.registered);
    EXPECT(std::string(m.backendName(&a, true)) == "vmm" && std::string(m.backendName(&a, false)) == "slices");
    EXPECT(m.getBuffer(&a, 4096, false, nullptr, &l2) == ncclSuccess && !l2.registered);
    // the growing block is leased: a nested registered request falls back to slices
    EXPECT(m.getBuffer(&a, 4096, true, nullptr, &l3) == ncclSuccess && !l3.registered);
    EXPECT(m.releaseBuffer(&l1, nullptr) == ncclSuccess && l1.ptr == nullptr);
    EXPECT(m.releaseBuffer(&l2, nullptr) == ncclSuccess && m.releaseBuffer(&l3, nullptr) == ncclSuccess);
    EXPECT(m.releaseBuffer(&l3, nullptr) == ncclInvalidArgument);  // double release
    // pools are per communicator
    BufferLease lb;
    EXPECT(m.getBuffer(&b, 4096, false, nullptr, &lb) == ncclSuccess);
    EXPECT(m.reservedBytes(&b) > 0 && m.reservedBytes(&a) > 0);
    m.releaseBuffer(&lb, nullptr);
    m.commDestroy(&b);
    EXPECT(m.reservedBytes(&b) == 0);
    // WorkspaceProvider interface
    void *ptr, *lease;
    EXPECT(m.acquire(&a, 8192, false, nullptr, &ptr, &lease) == ncclSuccess && ptr != nullptr);
    m.release(lease, nullptr);
  }
  // devices without VMM support use slices for registered buffers too
  fakes::vmmLog().supported = false;
  BufferManager m2(opt);
  BufferLease l;
  EXPECT(m2.getBuffer(&a, 4096, true, nullptr, &l) == ncclSuccess);
  EXPECT(std::string(m2.backendName(&a, true)) == "slices");
  m2.releaseBuffer(&l, nullptr);
  // allocation failure surfaces
  fakes::allocLog().failNext = true;
  EXPECT(m2.getBuffer(&a, 64 << 20, false, nullptr, &l) == ncclUnhandledCudaError);
}

// ------------------------------------------------------------------ autotune
TEST(autotune_fit_and_cost_model) {
  LinearModel m = fitLinear({{1e6, 1e-3 + 1e-9 * 1e6}, {4e6, 1e-3 + 1e-9 * 4e6}, {16e6, 1e-3 + 1e-9 * 16e6}});
  EXPECT(m.valid && fabs(m.alpha - 1e-3) < 1e-9 && fabs(m.beta - 1e-9) < 1e-15);
  EXPECT(!fitLinear({{1e6, 1e-3}}).valid);                       // needs two points
  EXPECT(!fitLinear({{1e6, 1e-3}, {1e6, 2e-3}}).valid);          // ... with distinct sizes
  LinearModel neg = fitLinear({{1e6, 5e-3}, {2e6, 1e-3}});        // decreasing: clamped, never negative
  EXPECT(neg.valid && neg.beta >= 0 && neg.alpha >= 0);
  CostInputs in;
  in.topo = {2, 8, true};
  in.intra = {1e-5, 1e-11, true};
  in.inter = {5e-5, 1e-10, true};
  CodecModel c;
  c.roundTrip = {2e-5, 2e-12, true};
  c.ratio = 4;
  in.flat = in.intraCodec = in.interCodec = in.defaultCodec = c;
  const double M = 64e6;
  EXPECT(fabs(costPcca(in.intra, c, M, 8) - (c.roundTrip.time(M) + in.intra.time(M / 32))) < 1e-12);
  const double g = costGlobalPcca(in, c, M);
  EXPECT(fabs(g - (c.roundTrip.time(M) + std::max(in.intra.time(M / (16 * 4)), in.inter.time(M * 1 / (2 * 4))))) < 1e-12);
  EXPECT(fabs(costOf(Algorithm::RsOneShot, in, M) - g) < 1e-12);
  EXPECT(fabs(costOf(Algorithm::ArTwoShot, in, M) - 2 * g) < 1e-12);
  EXPECT(fabs(costOf(Algorithm::RsTwoShot, in, M) - (costPcca(in.intra, c, M, 8) + costPcca(in.inter, c, M / 8, 2))) < 1e-12);
  EXPECT(fabs(costOf(Algorithm::ArTripleShot, in, M) - (costOf(Algorithm::RsTwoShot, in, M) + g)) < 1e-12);
  in.inter.valid = false;
  EXPECT(!std::isfinite(costOf(Algorithm::RsOneShot, in, M)));
  std::vector<size_t> sizes = profileSizes(256 << 10, 10 << 20);
  EXPECT(sizes.size() == 4 && sizes[0] == (256u << 10) && sizes[2] == (4u << 20) && sizes.back() == (10u << 20));
}

namespace {
bool allSupported(Algorithm, void*) { return true; }
bool noTwoShotAr(Algorithm a, void*) { return a != Algorithm::ArTwoShot; }
}  // namespace

TEST(autotune_selection_eligibility_model_and_fallback) {
  Selection s;
  Topology one{1, 8, true}, two{2, 8, true}, ragged{2, 8, false};
  // heuristics
  EXPECT(chooseAlgorithm(Operation::ReduceScatter, 1024, 4, 8, one, nullptr, Algorithm::None, allSupported, nullptr, &s) == ncclSuccess);
  EXPECT(s.algorithm == Algorithm::RsOneShot && !s.usedModel);
  EXPECT(chooseAlgorithm(Operation::ReduceScatter, 1024, 4, 16, two, nullptr, Algorithm::None, allSupported, nullptr, &s) == ncclSuccess);
  EXPECT(s.algorithm == Algorithm::RsTwoShot);
  EXPECT(chooseAlgorithm(Operation::ReduceScatter, 1024, 4, 16, ragged, nullptr, Algorithm::None, allSupported, nullptr, &s) == ncclSuccess);
  EXPECT(s.algorithm == Algorithm::RsOneShot);  // hierarchy needs a uniform layout
  EXPECT(chooseAlgorithm(Operation::AllReduce, 1024, 4, 16, two, nullptr, Algorithm::None, allSupported, nullptr, &s) == ncclSuccess);
  EXPECT(s.algorithm == Algorithm::ArTwoShot);
  EXPECT(chooseAlgorithm(Operation::AllReduce, 1024, 4, 16, two, nullptr, Algorithm::None, noTwoShotAr, nullptr, &s) == ncclSuccess);
  EXPECT(s.algorithm == Algorithm::ArOneShot);
  EXPECT(chooseAlgorithm(Operation::AllReduce, 1023, 4, 16, two, nullptr, Algorithm::None, allSupported, nullptr, &s) == ncclInvalidUsage);
  // forced algorithm honoured, or replaced by its fallback
  EXPECT(chooseAlgorithm(Operation::AllReduce, 1024, 4, 16, two, nullptr, Algorithm::ArTripleShot, allSupported, nullptr, &s) == ncclSuccess);
  EXPECT(s.algorithm == Algorithm::ArTripleShot && s.forced && !s.fellBack);
  EXPECT(chooseAlgorithm(Operation::AllReduce, 1024, 4, 8, one, nullptr, Algorithm::ArTripleShot, allSupported, nullptr, &s) == ncclSuccess);
  EXPECT(s.algorithm == Algorithm::ArTwoShot && s.fellBack);
  // cost model: small messages favour the one-shot all-reduce (fewer latency terms), large ones the two-shot
  CostInputs in;
  in.topo = one;
  in.intra = {5e-6, 1.2e-12, true};
  CodecModel c;
  c.roundTrip = {1e-5, 4e-13, true};
  c.ratio = 7.5;
  in.flat = in.intraCodec = in.defaultCodec = in.interCodec = c;
  EXPECT(chooseAlgorithm(Operation::AllReduce, 1024, 4, 8, one, &in, Algorithm::None, allSupported, nullptr, &s) == ncclSuccess);
  EXPECT(s.usedModel && s.algorithm == Algorithm::ArOneShot);
  EXPECT(chooseAlgorithm(Operation::AllReduce, 256 << 20, 4, 8, one, &in, Algorithm::None, allSupported, nullptr, &s) == ncclSuccess);
  EXPECT(s.usedModel && s.algorithm == Algorithm::ArTwoShot);
  // a missing model falls back to the heuristic order
  in.intra.valid = false;
  EXPECT(chooseAlgorithm(Operation::AllReduce, 1024, 4, 8, one, &in, Algorithm::None, allSupported, nullptr, &s) == ncclSuccess);
  EXPECT(!s.usedModel && s.algorithm == Algorithm::ArTwoShot);
}

// ------------------------------------------------------------------ training classifier
namespace {
struct TraceBuilder {
  std::vector<TraceEvent> ev;
  uint64_t t = 0;
  void add(uint64_t comm, TraceOp op, size_t bytes, int peer = -1, uint64_t dt = 1000) {
    TraceEvent e;
    e.sequence = ev.size(); e.commId = comm; e.op = op; e.logicalBytes = bytes; e.peer = peer; t += dt; e.timestampNs = t;
    ev.push_back(e);
  }
};
// One Megatron-like iteration on a TP2/PP2/DP2 rank: pipeline transfers around tensor-parallel bursts,
// gradient reduce-scatter buckets overlapped with the last bursts, parameter all-gather at the end.
void megatronIteration(TraceBuilder& b, bool firstGap) {
  const size_t MB = 1 << 20;
  for (int mb = 0; mb < 4; ++mb) {
    b.add(3, TraceOp::Recv, 31 * MB, 0, mb == 0 && firstGap ? 5000000 : 1000);
    for (int l = 0; l < 4; ++l) { b.add(2, TraceOp::AllGather, 29 * MB); b.add(2, TraceOp::ReduceScatter, 29 * MB); }
    b.add(3, TraceOp::Send, 31 * MB, 0);
  }
  for (int k = 0; k < 3; ++k) {
    b.add(1, TraceOp::ReduceScatter, 92 * MB);
    b.add(2, TraceOp::AllGather, 29 * MB);
    b.add(2, TraceOp::ReduceScatter, 29 * MB);
  }
  for (int k = 0; k < 3; ++k) b.add(1, TraceOp::AllGather, 46 * MB);
}
}  // namespace

TEST(classifier_topology_and_iteration_detection) {
  ClassifierParams p{4, 2, 2, DpStrategy::Sdp, true};
  TraceComm c4{1, 0, 4, 1, 4}, c2{2, 0, 2, 1, 2}, c8{3, 0, 8, 1, 8};
  EXPECT(topologyRole(c4, TraceOp::AllReduce, p) == Role::DataParallel);
  EXPECT(topologyRole(c2, TraceOp::AllGather, p) == Role::TensorParallel);  // size 2 == tp (pp only matters for p2p)
  EXPECT(topologyRole(c2, TraceOp::Send, p) == Role::PipelineParallel);
  EXPECT(topologyRole(c8, TraceOp::AllReduce, p) == Role::Unknown);
  ClassifierParams same{2, 2, 2, DpStrategy::Sdp, true};
  EXPECT(topologyRole(c2, TraceOp::AllReduce, same) == Role::Unknown);  // matches both DP and TP sizes
  TraceBuilder b;
  b.add(9, TraceOp::AllReduce, 7 << 20);  // start-up noise before the loop
  b.add(9, TraceOp::AllGather, 5 << 20);
  for (int i = 0; i < 6; ++i) megatronIteration(b, true);
  std::vector<IterationRange> its;
  EXPECT(detectIterations(b.ev, 5, &its));
  const size_t period = 4 * 10 + 9 + 3;
  EXPECT(its.size() >= 5);
  for (const IterationRange& r : its) EXPECT_EQ(r.end - r.begin, period);
  EXPECT(b.ev[its[0].begin].op == TraceOp::Recv && b.ev[its[0].begin].commId == 3);  // boundaries sit at the long gap
  // too few events, or no repetition
  std::vector<TraceEvent> few(b.ev.begin(), b.ev.begin() + 5);
  EXPECT(!detectIterations(few, 5, &its));
  TraceBuilder noise;
  for (int i = 0; i < 200; ++i) noise.add(1, TraceOp::AllReduce, (size_t)(i * 7919 + 13) << 10);
  EXPECT(!detectIterations(noise.ev, 5, &its));
}

TEST(classifier_roles_from_traffic_when_sizes_collide) {
  // TP = PP = DP = 2: sizes say nothing, the traffic pattern must decide
  ClassifierParams p{2, 2, 2, DpStrategy::Sdp, true};
  std::vector<TraceComm> comms = {{1, 0, 2, 1, 2}, {2, 0, 2, 1, 2}, {3, 0, 2, 1, 2}};
  TraceBuilder b;
  for (int i = 0; i < 6; ++i) megatronIteration(b, true);
  std::vector<IterationRange> its;
  EXPECT(detectIterations(b.ev, 5, &its));
  std::vector<TraceResult> res;
  classifyTrace(comms, b.ev, its, 5, p, &res);
  EXPECT(res.size() == 3);
  for (const TraceResult& r : res) {
    if (r.commId == 1) { EXPECT(r.classification.role == Role::DataParallel); EXPECT(fabs(r.classification.agToRsRatio - 0.5) < 0.01); }
    if (r.commId == 2) { EXPECT(r.classification.role == Role::TensorParallel); EXPECT(r.classification.callsPerIteration >= 2.0); }
    if (r.commId == 3) EXPECT(r.classification.role == Role::PipelineParallel);
    EXPECT(r.classification.committed);
  }
  // with too few iterations the evidence is scaled down and nothing is committed to a role
  std::vector<IterationRange> two(its.begin(), its.begin() + 2);
  classifyTrace(comms, b.ev, two, 5, p, &res);
  for (const TraceResult& r : res)
    if (r.commId == 2) EXPECT(r.classification.role == Role::Unknown);
}

TEST(classifier_ddp_and_tensor_allreduce_patterns) {
  ClassifierParams ddp{4, 4, 1, DpStrategy::Ddp, false};
  std::vector<TraceComm> comms = {{1, 0, 4, 2, 2}, {2, 0, 4, 1, 4}};  // comm 1 spans two nodes
  TraceBuilder b;
  for (int it = 0; it < 6; ++it) {
    for (int l = 0; l < 6; ++l) b.add(2, TraceOp::AllReduce, 23 << 20, -1, l == 0 ? 4000000 : 1000);
    for (int k = 0; k < 3; ++k) b.add(1, TraceOp::AllReduce, 97 << 20);
  }
  std::vector<IterationRange> its;
  EXPECT(detectIterations(b.ev, 5, &its));
  std::vector<TraceResult> res;
  classifyTrace(comms, b.ev, its, 5, ddp, &res);
  for (const TraceResult& r : res) {
    if (r.commId == 1) EXPECT(r.classification.role == Role::DataParallel);     // cross-node all-reduce-only buckets
    if (r.commId == 2) EXPECT(r.classification.role == Role::TensorParallel);   // stable node-local flow before the DP tail
  }
}

namespace {
uint64_t gFakeNow = 0;
uint64_t fakeNow() { return gFakeNow += 1000; }
}  // namespace

TEST(training_assist_commits_and_activates_at_a_common_call) {
  ClassifierParams p{2, 2, 2, DpStrategy::Sdp, true};
  TrainingAssist assist(p, 5);
  assist.setClock(&fakeNow);
  fakes::FakeTransport t;
  Comm dp = fakes::makeComm(&t, 0, 2, 1), tp = fakes::makeComm(&t, 0, 2, 1), pp = fakes::makeComm(&t, 0, 2, 1), big = fakes::makeComm(&t, 0, 8, 1);
  dp.id = 1; tp.id = 2; pp.id = 3; big.id = 4;
  for (Comm* c : {&dp, &tp, &pp, &big}) assist.registerComm(c);
  char buf[8];
  auto call = [&](Comm* c, Operation op, size_t bytes, Func f = Func::Collective, int peer = -1) {
    CallInfo i;
    i.op = op; i.func = f; i.sendbuff = buf; i.recvbuff = buf; i.comm = c; i.peer = peer; i.datatype = ncclUint8;
    i.count = (op == Operation::AllGather || op == Operation::ReduceScatter) ? bytes / (size_t)c->nRanks : bytes;
    assist.observe(i, 0);
  };
  EXPECT(assist.roleOf(&tp) == Role::Unknown);
  const size_t MB = 1 << 20;
  int iterations = 0;
  uint64_t tpCallsAtCommit = 0;
  for (; iterations < 12; ++iterations) {
    gFakeNow += 5000000;
    for (int mb = 0; mb < 4; ++mb) {
      call(&pp, Operation::SendRecv, 31 * MB, Func::Recv, 1);
      for (int l = 0; l < 4; ++l) { call(&tp, Operation::AllGather, 29 * MB); call(&tp, Operation::ReduceScatter, 29 * MB); }
      call(&pp, Operation::SendRecv, 31 * MB, Func::Send, 1);
      call(&tp, Operation::AllReduce, 64);  // tiny calls are not evidence
    }
    for (int k = 0; k < 3; ++k) { call(&dp, Operation::ReduceScatter, 92 * MB); call(&tp, Operation::AllGather, 29 * MB); call(&tp, Operation::ReduceScatter, 29 * MB); }
    for (int k = 0; k < 3; ++k) call(&dp, Operation::AllGather, 46 * MB);
    Classification c;
    uint64_t act = 0;
    if (tpCallsAtCommit == 0 && assist.query(&tp, &c, &act)) {
      tpCallsAtCommit = act;
      EXPECT(c.role == Role::TensorParallel);
      EXPECT(assist.roleOf(&tp) == Role::Unknown || act <= (uint64_t)(iterations + 1) * 42);  // not before its activation call
    }
  }
  EXPECT(tpCallsAtCommit > 0);
  EXPECT(assist.roleOf(&tp) == Role::TensorParallel);
  EXPECT(assist.roleOf(&dp) == Role::DataParallel);
  EXPECT(assist.roleOf(&pp) == Role::PipelineParallel);
  EXPECT(assist.roleOf(&big) == Role::Unknown);  // never seen
  // the activation index is a function of the trace only: a second observer of the same calls agrees
  Classification c1;
  uint64_t a1 = 0;
  EXPECT(assist.query(&dp, &c1, &a1) && a1 >= 2 * 5 * 6 - 6);
  // a communicator whose size matches exactly one configured dimension is decided at its first call
  ClassifierParams q{8, 2, 2, DpStrategy::Sdp, true};
  TrainingAssist bySize(q, 5);
  bySize.registerComm(&big);
  CallInfo i;
  i.op = Operation::AllReduce; i.sendbuff = buf; i.recvbuff = buf; i.comm = &big; i.count = 16; i.datatype = ncclFloat32;
  bySize.observe(i, 0);
  EXPECT(bySize.roleOf(&big) == Role::DataParallel);
  bySize.unregisterComm(&big);
  EXPECT(bySize.roleOf(&big) == Role::Unknown);
}
