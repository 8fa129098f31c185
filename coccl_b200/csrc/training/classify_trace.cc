// Evidence scoring of the training classifier (see classifier.h for the rules and their source).
#include <algorithm>
#include <cmath>
#include <map>
#include <set>

#include "training/classifier.h"

namespace coccl {
namespace {

constexpr double kRoleEvidence = 0.60, kOverlapPattern = 0.80, kConflictMargin = 0.15;
constexpr double kPpShare = 0.70, kPeerConcentration = 0.80, kStablePattern = 0.60;

bool isCollective(TraceOp op) { return op == TraceOp::AllGather || op == TraceOp::ReduceScatter || op == TraceOp::AllReduce; }
bool isP2p(TraceOp op) { return op == TraceOp::Send || op == TraceOp::Recv; }

struct CommStats {
  TraceComm comm;
  uint64_t calls = 0, p2p = 0, coll = 0, ag = 0, rs = 0, ar = 0;
  double p2pShare = 0, peerConcentration = 0;
  double callsPerIteration = 0;
  size_t medianBytes = 0;
  double patternSupport = 0;     // share of iterations showing the most common (op, bytes) sequence
  bool stable = false;
  double overlapSupport = 0;     // share of iterations whose reduce-scatters are interleaved with other traffic
  double ratioSupport = 0;       // share of iterations with AG/RS bytes near 0.5 or 0.25
  double agToRs = 0;
};

CommStats buildStats(const TraceComm& comm, const std::vector<TraceEvent>& ev, const std::vector<IterationRange>& its) {
  CommStats s;
  s.comm = comm;
  std::map<int, uint64_t> peers;
  std::vector<size_t> sizes;
  for (const TraceEvent& e : ev) {
    if (e.commId != comm.id) continue;
    ++s.calls;
    sizes.push_back(e.logicalBytes);
    if (isP2p(e.op)) { ++s.p2p; ++peers[e.peer]; }
    if (isCollective(e.op)) ++s.coll;
    if (e.op == TraceOp::AllGather) ++s.ag;
    if (e.op == TraceOp::ReduceScatter) ++s.rs;
    if (e.op == TraceOp::AllReduce) ++s.ar;
  }
  if (s.calls == 0) return s;
  s.p2pShare = (double)s.p2p / (double)s.calls;
  if (s.p2p) {
    std::vector<uint64_t> c;
    for (auto& kv : peers) c.push_back(kv.second);
    std::sort(c.rbegin(), c.rend());
    const uint64_t top2 = c[0] + (c.size() > 1 ? c[1] : 0);
    s.peerConcentration = (double)top2 / (double)s.p2p;
  }
  std::sort(sizes.begin(), sizes.end());
  s.medianBytes = sizes[sizes.size() / 2];
  if (its.empty()) return s;

  std::map<std::vector<uint64_t>, int> signatures;
  int overlapped = 0, ratioHits = 0, withCalls = 0;
  uint64_t inIterations = 0;
  std::vector<double> ratios;
  for (const IterationRange& it : its) {
    std::vector<uint64_t> sig;
    long firstRs = -1, lastRs = -1;
    int rsCount = 0;
    double agBytes = 0, rsBytes = 0;
    for (size_t i = it.begin; i < it.end && i < ev.size(); ++i) {
      const TraceEvent& e = ev[i];
      if (e.commId != comm.id) continue;
      ++inIterations;
      sig.push_back(((uint64_t)e.op << 56) ^ (uint64_t)e.logicalBytes);
      if (e.op == TraceOp::ReduceScatter) { if (firstRs < 0) firstRs = (long)i; lastRs = (long)i; ++rsCount; rsBytes += (double)e.logicalBytes; }
      if (e.op == TraceOp::AllGather) agBytes += (double)e.logicalBytes;
    }
    if (!sig.empty()) ++withCalls;
    ++signatures[sig];
    if (rsCount >= 2) {
      bool foreign = false;
      for (long i = firstRs; i <= lastRs && !foreign; ++i) foreign = ev[(size_t)i].commId != comm.id;
      if (foreign) ++overlapped;
    }
    if (agBytes > 0 && rsBytes > 0) {
      const double r = agBytes / rsBytes;
      ratios.push_back(r);
      if (std::fabs(r - 0.5) <= 0.2 * 0.5 || std::fabs(r - 0.25) <= 0.2 * 0.25) ++ratioHits;
    }
  }
  const double n = (double)its.size();
  s.callsPerIteration = (double)inIterations / n;
  int best = 0;
  for (auto& kv : signatures)
    if (!kv.first.empty()) best = std::max(best, kv.second);
  s.patternSupport = (double)best / n;
  s.stable = s.patternSupport >= kStablePattern && withCalls > 0;
  s.overlapSupport = (double)overlapped / n;
  s.ratioSupport = (double)ratioHits / n;
  if (!ratios.empty()) { std::sort(ratios.begin(), ratios.end()); s.agToRs = ratios[ratios.size() / 2]; }
  return s;
}

// Share of iterations in which the `tp` communicator's burst comes before the `dp` communicator's
// traffic ends: a data-parallel flow trails the tensor-parallel one (gradient buckets drain last).
double orderRelation(uint64_t dp, uint64_t tp, const std::vector<TraceEvent>& ev, const std::vector<IterationRange>& its) {
  if (its.empty()) return 0;
  int ok = 0;
  for (const IterationRange& it : its) {
    long lastDp = -1, lastTp = -1, firstDp = -1, firstTp = -1;
    for (size_t i = it.begin; i < it.end && i < ev.size(); ++i) {
      if (ev[i].commId == dp) { if (firstDp < 0) firstDp = (long)i; lastDp = (long)i; }
      if (ev[i].commId == tp) { if (firstTp < 0) firstTp = (long)i; lastTp = (long)i; }
    }
    if (lastDp >= 0 && lastTp >= 0 && firstTp < firstDp && lastDp > lastTp) ++ok;
  }
  return (double)ok / (double)its.size();
}

// Share of iterations in which the communicator's collectives sit between pipeline transfers.
double ppInterior(uint64_t id, const std::set<uint64_t>& pp, const std::vector<TraceEvent>& ev, const std::vector<IterationRange>& its) {
  if (its.empty() || pp.empty()) return 0;
  int ok = 0;
  for (const IterationRange& it : its) {
    bool seenPp = false, burstAfterPp = false, closed = false;
    for (size_t i = it.begin; i < it.end && i < ev.size(); ++i) {
      if (pp.count(ev[i].commId)) { if (burstAfterPp) closed = true; seenPp = true; }
      else if (ev[i].commId == id && seenPp) burstAfterPp = true;
    }
    if (closed) ++ok;
  }
  return (double)ok / (double)its.size();
}

struct Evidence { double dp = 0, tp = 0, pp = 0, orderAsDp = 0, orderAsTp = 0; };

}  // namespace

void classifyTrace(const std::vector<TraceComm>& comms, const std::vector<TraceEvent>& events,
                   const std::vector<IterationRange>& iterations, int target, const ClassifierParams& p,
                   std::vector<TraceResult>* results) {
  if (results == nullptr) return;
  results->clear();
  std::map<uint64_t, CommStats> stats;
  std::map<uint64_t, Evidence> evidence;
  const double coverage = target <= 0 ? 0.0 : std::min(1.0, (double)iterations.size() / (double)target);

  for (const TraceComm& c : comms) {
    CommStats s = buildStats(c, events, iterations);
    stats[c.id] = s;
    Evidence& e = evidence[c.id];
    Role topo = Role::Unknown;
    if (s.calls != 0 && s.p2p == s.calls) topo = topologyRole(c, TraceOp::Send, p);
    else if (s.coll != 0) topo = topologyRole(c, TraceOp::AllReduce, p);
    if (topo == Role::DataParallel) { e.dp = 1.0; continue; }
    if (topo == Role::TensorParallel) { e.tp = 1.0; continue; }
    if (topo == Role::PipelineParallel) { e.pp = 1.0; continue; }

    if (p.ppSize > 1 && s.p2pShare >= kPpShare && s.peerConcentration >= kPeerConcentration) {
      e.pp = std::min(s.p2pShare, s.peerConcentration);
      continue;
    }
    double overlap = s.overlapSupport * coverage, ratio = s.ratioSupport * coverage;
    const bool rsOnly = s.rs != 0 && s.ag == 0 && s.ar == 0;
    if (p.dpStrategy == DpStrategy::Ddp) {
      if (c.nNodes > 1 && s.ar != 0 && s.ag == 0 && s.rs == 0 && s.stable && s.callsPerIteration >= 2.0)
        e.dp = s.patternSupport * coverage;
    } else if (p.dpStrategy == DpStrategy::Fsdp) {
      if (c.nNodes > 1 && s.ag != 0 && s.rs != 0 && s.stable) e.dp = s.patternSupport * coverage;
    } else {
      if (!rsOnly || overlap < kOverlapPattern) overlap = 0.0;
      if (ratio < kRoleEvidence) ratio = 0.0;
      e.dp = std::max(overlap, ratio);
    }
    if (!p.sequenceParallel && p.dpStrategy != DpStrategy::Ddp && c.nNodes == 1 && s.ar != 0 && s.ag == 0 && s.rs == 0 &&
        s.stable && s.callsPerIteration >= 2.0)
      e.tp = s.patternSupport * coverage;
  }

  std::set<uint64_t> ppComms;
  for (auto& kv : evidence)
    if (kv.second.pp >= kPpShare) ppComms.insert(kv.first);

  // relative order: a communicator with DP evidence (or a sparse, large node-local tail) marks the
  // stable node-local flow that precedes it as TP
  for (auto& d : stats) {
    if (evidence[d.first].pp >= kPpShare) continue;
    for (auto& t : stats) {
      if (d.first == t.first || evidence[t.first].pp >= kPpShare || t.second.comm.nNodes > 1) continue;
      const double rel = orderRelation(d.first, t.first, events, iterations) * coverage;
      if (rel < kRoleEvidence) continue;
      const bool seeded = evidence[d.first].dp >= kRoleEvidence;
      const bool sparseTail = d.second.comm.nNodes == 1 && d.second.stable && t.second.stable &&
                              d.second.callsPerIteration < t.second.callsPerIteration &&
                              (double)d.second.medianBytes >= 1.25 * (double)t.second.medianBytes;
      if (!seeded && !sparseTail) continue;
      if (!seeded) evidence[d.first].dp = rel;
      evidence[d.first].orderAsDp = std::max(evidence[d.first].orderAsDp, rel);
      if (evidence[t.first].dp < kRoleEvidence && t.second.stable && t.second.callsPerIteration >= 2.0) {
        evidence[t.first].tp = std::max(evidence[t.first].tp, rel);
        evidence[t.first].orderAsTp = std::max(evidence[t.first].orderAsTp, rel);
      }
    }
  }
  // a stable node-local burst between pipeline transfers is TP even without a DP communicator
  for (auto& kv : stats) {
    Evidence& e = evidence[kv.first];
    if (kv.second.comm.nNodes > 1 || e.pp >= kPpShare || e.dp >= kRoleEvidence || !kv.second.stable || kv.second.callsPerIteration < 2.0) continue;
    const double in = ppInterior(kv.first, ppComms, events, iterations) * coverage;
    e.tp = std::max(e.tp, in);
    e.orderAsTp = std::max(e.orderAsTp, in);
  }
  // with DP established, any other repeated node-local flow with >= 2 collectives per iteration is a TP candidate
  bool haveDp = false;
  for (auto& kv : evidence) haveDp = haveDp || kv.second.dp >= kRoleEvidence;
  if (haveDp)
    for (auto& kv : stats) {
      Evidence& e = evidence[kv.first];
      if (kv.second.comm.nNodes == 1 && e.dp < kRoleEvidence && e.pp < kPpShare && kv.second.stable && kv.second.callsPerIteration >= 2.0)
        e.tp = std::max(e.tp, kRoleEvidence * coverage);
    }

  for (auto& kv : stats) {
    const CommStats& s = kv.second;
    const Evidence& e = evidence[kv.first];
    Classification c;
    c.observedCalls = s.calls;
    c.cycleSupport = s.patternSupport;
    c.overlapPatternSupport = s.overlapSupport;
    c.orderSupport = std::max(e.orderAsDp, e.orderAsTp);
    c.agToRsRatio = s.agToRs;
    c.callsPerIteration = s.callsPerIteration;
    c.medianBytes = s.medianBytes;
    c.committed = true;
    if (e.pp >= kPpShare) {
      c.role = c.candidate = Role::PipelineParallel;
      c.confidence = e.pp;
    } else {
      const double dp = e.dp, tp = s.comm.nNodes > 1 ? 0.0 : e.tp;
      c.candidate = dp >= tp ? (dp > 0 ? Role::DataParallel : Role::Unknown) : Role::TensorParallel;
      if (dp >= kRoleEvidence && (tp < kRoleEvidence || dp - tp >= kConflictMargin)) { c.role = Role::DataParallel; c.confidence = dp; }
      else if (tp >= kRoleEvidence && (dp < kRoleEvidence || tp - dp >= kConflictMargin)) { c.role = Role::TensorParallel; c.confidence = tp; }
      else { c.role = Role::Unknown; c.confidence = std::max(dp, tp); }
    }
    results->push_back({kv.first, c});
  }
}

}  // namespace coccl
