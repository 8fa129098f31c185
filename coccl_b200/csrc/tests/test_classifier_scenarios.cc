// Scenario table of the training classifier: one trace per training set-up, each with the role every communicator
// must get. The scenarios restate, in this library's types, the set-ups the reference checks in
// tests/coccl-tests/src/coccl_training_classifier_test.cc:319-1153. The configured sizes are primes (DP 31, TP 29,
// PP 23) that match no communicator, so only traffic evidence can decide, unless a scenario says otherwise.
#include <math.h>

#include <map>

#include "tests/fakes.h"
#include "tests/host_test.h"
#include "training/assist.h"
#include "training/classifier.h"

using namespace coccl;

namespace {

constexpr int kTarget = 10;

struct Scenario {
  std::vector<TraceEvent> events;
  std::vector<IterationRange> iterations;
  size_t open = (size_t)-1;
  void close() {
    if (open != (size_t)-1) iterations.push_back({open, events.size()});
    open = (size_t)-1;
  }
  void next() { close(); open = events.size(); }
  void add(uint64_t comm, TraceOp op, size_t bytes, int peer = -1) {
    TraceEvent e;
    e.sequence = events.size(); e.commId = comm; e.op = op; e.logicalBytes = bytes; e.peer = peer;
    e.timestampNs = events.size() * 1000;
    events.push_back(e);
  }
};

TraceComm comm(uint64_t id, int nRanks, int nNodes) {
  TraceComm c;
  c.id = id; c.nRanks = nRanks; c.nNodes = nNodes; c.localRanks = nRanks / nNodes;
  return c;
}

ClassifierParams primes() { return ClassifierParams{31, 29, 23, DpStrategy::Sdp, true}; }

std::map<uint64_t, Classification> classify(const std::vector<TraceComm>& comms, Scenario& s,
                                            const ClassifierParams& p = primes(), int target = kTarget) {
  s.close();
  std::vector<TraceResult> res;
  classifyTrace(comms, s.events, s.iterations, target, p, &res);
  std::map<uint64_t, Classification> out;
  for (const TraceResult& r : res) out[r.commId] = r.classification;
  return out;
}

constexpr TraceOp AG = TraceOp::AllGather, RS = TraceOp::ReduceScatter, AR = TraceOp::AllReduce;
constexpr size_t MB = 1 << 20;

}  // namespace

TEST(scenario_partial_suffix_does_not_change_calls_per_iteration) {
  Scenario s;
  for (int it = 0; it < 5; ++it) {
    s.next();
    s.add(1, AG, 128); s.add(1, AG, 256); s.add(1, RS, 512); s.add(1, RS, 1024);
  }
  s.close();
  s.add(1, AG, 128); s.add(1, AG, 256);  // the sixth iteration has only begun
  auto r = classify({comm(1, 2, 1)}, s, primes(), 5);
  EXPECT_EQ(r[1].observedCalls, (uint64_t)22);
  EXPECT(r[1].callsPerIteration == 4.0);
}

TEST(scenario_tensor_all_reduce_next_to_sharded_data_parallel) {
  Scenario s;
  for (int it = 0; it < kTarget; ++it) {
    s.next();
    s.add(30, AG, 1 * MB); s.add(31, AR, 2 * MB); s.add(31, AR, 2 * MB); s.add(30, RS, 2 * MB);
  }
  ClassifierParams p = primes();
  p.sequenceParallel = false;
  auto r = classify({comm(30, 8, 2), comm(31, 2, 1)}, s, p);
  EXPECT(r[30].role == Role::DataParallel);    // all-gather / reduce-scatter at ratio 0.5
  EXPECT(r[31].role == Role::TensorParallel);  // node-local all-reduce pairs
}

TEST(scenario_configured_ddp_and_fsdp) {
  Scenario ddp, fsdp;
  for (int it = 0; it < kTarget; ++it) {
    ddp.next(); ddp.add(32, AR, 2 * MB); ddp.add(32, AR, 4 * MB);
    fsdp.next(); fsdp.add(33, AG, 1 * MB); fsdp.add(33, AG, 2 * MB); fsdp.add(33, RS, 3 * MB);
  }
  ClassifierParams p = primes();
  p.dpStrategy = DpStrategy::Ddp;
  EXPECT(classify({comm(32, 8, 2)}, ddp, p)[32].role == Role::DataParallel);
  p.dpStrategy = DpStrategy::Fsdp;
  EXPECT(classify({comm(33, 8, 2)}, fsdp, p)[33].role == Role::DataParallel);
  // the same DDP trace under the default (sharded) strategy carries no evidence
  EXPECT(classify({comm(32, 8, 2)}, ddp)[32].role == Role::Unknown);
}

TEST(scenario_configured_sizes_decide_at_once) {
  Scenario a, b;
  for (int it = 0; it < kTarget; ++it) {
    a.next(); a.add(34, AR, 2 * MB); a.add(35, AR, 2 * MB); a.add(36, TraceOp::Send, 2 * MB, 1); a.add(36, TraceOp::Recv, 2 * MB, 1);
    b.next(); b.add(37, RS, 2 * MB); b.add(38, AR, 2 * MB);
  }
  ClassifierParams p{4, 2, 2, DpStrategy::Sdp, true};
  auto ra = classify({comm(34, 4, 2), comm(35, 2, 1), comm(36, 2, 2)}, a, p);
  EXPECT(ra[34].role == Role::DataParallel);
  EXPECT(ra[35].role == Role::TensorParallel);
  EXPECT(ra[36].role == Role::PipelineParallel);
  ClassifierParams q{2, 4, 2, DpStrategy::Sdp, true};
  auto rb = classify({comm(37, 2, 2), comm(38, 4, 1)}, b, q);
  EXPECT(rb[37].role == Role::DataParallel);
  EXPECT(rb[38].role == Role::TensorParallel);
}

TEST(scenario_cross_node_dp_brackets_a_heavier_tp_flow) {
  Scenario s;
  for (int it = 0; it < kTarget; ++it) {
    s.next();
    s.add(1, AG, 128);
    for (int i = 0; i < 12; ++i) s.add(2, AR, 64);  // more total bytes than DP: bytes must not decide
    s.add(1, RS, 512);
  }
  auto r = classify({comm(1, 16, 2), comm(2, 8, 1)}, s);
  EXPECT(r[1].role == Role::DataParallel);
  EXPECT(r[2].role == Role::TensorParallel);
  EXPECT(r[2].orderSupport >= 0.6);
}

TEST(scenario_pipeline_transfers) {
  Scenario s;
  for (int it = 0; it < kTarget; ++it) {
    s.next();
    for (int mb = 0; mb < 4; ++mb) { s.add(3, TraceOp::Recv, 1024, 0); s.add(3, TraceOp::Send, 1024, 1); }
  }
  EXPECT(classify({comm(3, 4, 2)}, s)[3].role == Role::PipelineParallel);
  // many peers (an all-to-all written as send/recv) is not a pipeline
  Scenario fan;
  for (int it = 0; it < kTarget; ++it) {
    fan.next();
    for (int peer = 0; peer < 8; ++peer) { fan.add(4, TraceOp::Send, 1024, peer); fan.add(4, TraceOp::Recv, 1024, peer); }
  }
  EXPECT(classify({comm(4, 8, 2)}, fan)[4].role == Role::Unknown);
}

TEST(scenario_overlapped_gradient_buckets) {
  Scenario s;
  for (int it = 0; it < kTarget; ++it) { s.next(); s.add(4, RS, 256); s.add(4, RS, 768); s.add(4, RS, 512); }
  auto r = classify({comm(4, 8, 1)}, s);
  EXPECT(r[4].role == Role::DataParallel);
  EXPECT(r[4].overlapPatternSupport == 1.0);
}

TEST(scenario_overlap_needs_eight_of_ten_iterations) {
  Scenario seven, eight;
  for (int it = 0; it < kTarget; ++it) {
    seven.next();
    seven.add(10, RS, it < 7 ? 256 : (size_t)1024 + it); seven.add(10, RS, it < 7 ? 768 : (size_t)2048 + it);
    eight.next();
    eight.add(11, RS, it < 8 ? 256 : (size_t)1024 + it); eight.add(11, RS, it < 8 ? 768 : (size_t)2048 + it);
  }
  EXPECT(classify({comm(10, 8, 1)}, seven)[10].role == Role::Unknown);
  EXPECT(classify({comm(11, 8, 1)}, eight)[11].role == Role::DataParallel);
}

TEST(scenario_gather_scatter_ratio_needs_six_of_ten_iterations) {
  Scenario five, six;
  for (int it = 0; it < kTarget; ++it) {
    five.next(); five.add(12, AG, 100); five.add(12, RS, it < 5 ? 200 : (size_t)301 + it);
    six.next(); six.add(13, AG, 100); six.add(13, RS, it < 6 ? 200 : (size_t)301 + it);
  }
  EXPECT(classify({comm(12, 8, 1)}, five)[12].role == Role::Unknown);
  EXPECT(classify({comm(13, 8, 1)}, six)[13].role == Role::DataParallel);
}

TEST(scenario_half_and_quarter_precision_ratios_are_kept) {
  Scenario half, quarter;
  for (int it = 0; it < kTarget; ++it) {
    half.next(); half.add(5, AG, 100); half.add(5, RS, 200);        // bf16 parameters, fp32 gradients
    quarter.next(); quarter.add(6, AG, 100); quarter.add(6, RS, 400);  // fp8 parameters, fp32 gradients
  }
  auto h = classify({comm(5, 8, 1)}, half);
  auto q = classify({comm(6, 8, 1)}, quarter);
  EXPECT(h[5].role == Role::DataParallel && fabs(h[5].agToRsRatio - 0.5) < 0.01);
  EXPECT(q[6].role == Role::DataParallel && fabs(q[6].agToRsRatio - 0.25) < 0.01);
  // a ratio of 1 (same precision both ways) is not evidence
  Scenario same;
  for (int it = 0; it < kTarget; ++it) { same.next(); same.add(7, AG, 200); same.add(7, RS, 200); }
  EXPECT(classify({comm(7, 8, 1)}, same)[7].role == Role::Unknown);
}

TEST(scenario_node_local_ddp_tail_behind_a_dense_tp_flow) {
  Scenario s;
  for (int it = 0; it < kTarget; ++it) {
    s.next();
    for (int i = 0; i < 4; ++i) s.add(8, AR, 64);
    s.add(7, AR, 256);
  }
  auto r = classify({comm(7, 8, 1), comm(8, 4, 1)}, s);
  EXPECT(r[7].role == Role::DataParallel);
  EXPECT(r[8].role == Role::TensorParallel);
  // the tail must be larger than the dense flow (1.25x): equal sizes decide nothing
  Scenario flat;
  for (int it = 0; it < kTarget; ++it) {
    flat.next();
    for (int i = 0; i < 4; ++i) flat.add(8, AR, 64);
    flat.add(7, AR, 64);
  }
  auto f = classify({comm(7, 8, 1), comm(8, 4, 1)}, flat);
  EXPECT(f[7].role == Role::Unknown);
  EXPECT(f[8].role == Role::Unknown);
}

TEST(scenario_tp2_pp2_language_model_trace) {
  // A TP2 x PP2 x DP2 run with a distributed optimizer, as one rank records it: world-wide control traffic,
  // the embedding all-reduce between first and last stage, two tensor-parallel communicators, pipeline transfers,
  // the optimizer's reduce-scatter / all-gather buckets, tiny cross-node control calls, one start-up call.
  Scenario s;
  s.add(26, AR, 128);
  for (int it = 0; it < kTarget; ++it) {
    s.next();
    s.add(20, AR, 4); s.add(20, AG, 768);
    s.add(21, AR, 311164928);
    s.add(22, AG, 1048576); s.add(22, AR, 129024); s.add(22, RS, 1048576);
    s.add(27, AG, 1048576); s.add(27, AR, 2048); s.add(27, AR, 4096); s.add(27, AG, 1048576); s.add(27, RS, 1048576);
    s.add(27, AR, 133120);
    s.add(23, TraceOp::Send, 524288, 1); s.add(23, TraceOp::Recv, 524288, 1);
    s.add(24, RS, 440530944); s.add(24, RS, 311164928); s.add(24, AG, 220265472); s.add(24, AG, 155582464);
    s.add(25, AR, 4); s.add(25, AR, 4); s.add(25, AR, 4);
  }
  auto r = classify({comm(20, 8, 2), comm(21, 2, 2), comm(22, 2, 1), comm(23, 2, 2), comm(24, 2, 1), comm(25, 4, 2),
                     comm(26, 2, 1), comm(27, 2, 1)}, s);
  EXPECT(r[20].role == Role::Unknown);           // world control
  EXPECT(r[21].role == Role::Unknown);           // embedding collective
  EXPECT(r[22].role == Role::TensorParallel);
  EXPECT(r[23].role == Role::PipelineParallel);
  EXPECT(r[24].role == Role::DataParallel);      // distributed optimizer, ratio 0.5
  EXPECT(r[25].role == Role::Unknown);           // tiny cross-node control
  EXPECT(r[26].role == Role::Unknown);           // start-up only
  EXPECT(r[27].role == Role::TensorParallel);    // multi-size tensor-parallel flow
}

TEST(scenario_one_constant_collective_is_ambiguous) {
  Scenario s;
  for (int it = 0; it < kTarget; ++it) { s.next(); s.add(9, AR, 64); }
  auto r = classify({comm(9, 8, 1)}, s);
  EXPECT(r[9].role == Role::Unknown);
  EXPECT(r[9].committed);
}

TEST(scenario_evidence_scales_with_observed_iterations) {
  // the same clean trace with 5 of 10 target iterations reaches only half the evidence
  Scenario s;
  for (int it = 0; it < 5; ++it) { s.next(); s.add(5, AG, 100); s.add(5, RS, 200); }
  auto r = classify({comm(5, 8, 1)}, s);
  EXPECT(r[5].role == Role::Unknown);
  EXPECT(r[5].candidate == Role::Unknown || r[5].candidate == Role::DataParallel);
  EXPECT(r[5].confidence < 0.6);
}

// ---------------------------------------------------------------- runtime side
namespace {
uint64_t gNow = 0;
uint64_t fakeNow() { return gNow += 1000; }

CallInfo call(Comm* c, Operation op, Func f, size_t bytes, int peer = -1) {
  static char buf[8];
  CallInfo i;
  i.op = op; i.func = f; i.sendbuff = buf; i.recvbuff = buf; i.comm = c; i.peer = peer; i.datatype = ncclUint8;
  i.count = (op == Operation::AllGather || op == Operation::ReduceScatter) ? bytes / (size_t)c->nRanks : bytes;
  return i;
}
}  // namespace

TEST(scenario_runtime_ignores_calls_below_one_mebibyte) {
  TrainingAssist assist(primes(), kTarget);
  assist.setClock(&fakeNow);
  fakes::FakeTransport t;
  Comm c = fakes::makeComm(&t, 0, 2, 1);
  c.id = 0x1005;
  assist.registerComm(&c);
  for (int i = 0; i < 256; ++i) assist.observe(call(&c, Operation::AllReduce, Func::Collective, kTrainingMinEvidenceBytes - 1), 0);
  EXPECT_EQ(assist.traceSize(), (size_t)0);
  for (int it = 0; it < kTarget; ++it) {
    gNow += 5000000;
    assist.observe(call(&c, Operation::AllReduce, Func::Collective, kTrainingMinEvidenceBytes), 0);
    assist.observe(call(&c, Operation::AllReduce, Func::Collective, kTrainingMinEvidenceBytes), 0);
  }
  EXPECT(assist.traceSize() > 0 || [&] { Classification k; return assist.query(&c, &k); }());
  assist.unregisterComm(&c);
}

TEST(scenario_runtime_commits_configured_sizes_on_the_first_call) {
  ClassifierParams p{4, 2, 2, DpStrategy::Sdp, true};
  TrainingAssist assist(p, kTarget);
  assist.setClock(&fakeNow);
  fakes::FakeTransport t;
  Comm dp = fakes::makeComm(&t, 0, 4, 2), tp = fakes::makeComm(&t, 0, 2, 1), pp = fakes::makeComm(&t, 0, 2, 2);
  dp.id = 0x1010; tp.id = 0x1011; pp.id = 0x1012;
  Classification k;
  assist.registerComm(&dp);
  assist.observe(call(&dp, Operation::AllReduce, Func::Collective, 4), 0);  // far below the evidence minimum: size decides
  EXPECT(assist.query(&dp, &k) && k.committed && k.role == Role::DataParallel);
  EXPECT(assist.roleOf(&dp) == Role::DataParallel);
  for (int i = 0; i < 1000; ++i) {  // steady state: still DP, no trace growth
    assist.observe(call(&dp, Operation::AllReduce, Func::Collective, 4), 0);
    EXPECT(assist.roleOf(&dp) == Role::DataParallel);
  }
  EXPECT_EQ(assist.traceSize(), (size_t)0);
  assist.unregisterComm(&dp);
  EXPECT(!assist.query(&dp, &k));

  assist.registerComm(&tp);
  assist.observe(call(&tp, Operation::AllReduce, Func::Collective, 4), 0);
  EXPECT(assist.query(&tp, &k) && k.role == Role::TensorParallel);
  assist.unregisterComm(&tp);

  assist.registerComm(&pp);
  assist.observe(call(&pp, Operation::SendRecv, Func::Send, 4, 1), 0);
  EXPECT(assist.query(&pp, &k) && k.role == Role::PipelineParallel);
  assist.unregisterComm(&pp);
}

TEST(scenario_flat_inner_loop_is_not_an_iteration) {
  // ten identical layer collectives at an even pace repeat, but nothing marks an iteration boundary
  std::vector<TraceEvent> ev(10);
  for (size_t i = 0; i < ev.size(); ++i) { ev[i].sequence = i; ev[i].commId = 2; ev[i].op = AR; ev[i].logicalBytes = 2 * MB; ev[i].timestampNs = i * 10; }
  std::vector<IterationRange> its;
  EXPECT(!detectIterations(ev, 5, &its));
  EXPECT(its.empty());
}
