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
  double overlapSupport = 0;     // share of iterations showing the most common pattern with one op in >= 2 sizes (buckets)
  double ratioSupport = 0;       // share of iterations with AG/RS bytes near 0.5 or 0.25
  double agToRs = 0;
};

// One iteration as one communicator sees it.
struct IterationView {
  std::vector<uint64_t> pattern;         // (op, bytes) of its collectives, in order
  uint64_t calls = 0;                    // collectives and point-to-point
  double agBytes = 0, rsBytes = 0;
  bool multiSize = false;                // some operation appears with two or more distinct sizes (gradient buckets)
};

IterationView viewOf(uint64_t id, const std::vector<TraceEvent>& ev, const IterationRange& it) {
  IterationView v;
  std::set<size_t> sizes[3];
  const size_t end = std::min(it.end, ev.size());
  for (size_t i = it.begin; i < end; ++i) {
    const TraceEvent& e = ev[i];
    if (e.commId != id) continue;
    ++v.calls;
    if (!isCollective(e.op)) continue;
    v.pattern.push_back(((uint64_t)e.op << 56) ^ (uint64_t)e.logicalBytes);
    sizes[(int)e.op].insert(e.logicalBytes);
    if (e.op == TraceOp::AllGather) v.agBytes += (double)e.logicalBytes;
    if (e.op == TraceOp::ReduceScatter) v.rsBytes += (double)e.logicalBytes;
  }
  for (const std::set<size_t>& s : sizes) v.multiSize = v.multiSize || s.size() >= 2;
  return v;
}

bool nearRatio(double r, double target) { return std::fabs(r - target) <= 0.2 * target; }

CommStats buildStats(const TraceComm& comm, const std::vector<TraceEvent>& ev, const std::vector<IterationRange>& its) {
  CommStats s;
  s.comm = comm;
  std::map<int, uint64_t> peers;
  std::vector<size_t> sizes;
  // whole trace (a partial iteration after the last boundary counts as observed calls, nothing else)
  for (const TraceEvent& e : ev) {
    if (e.commId != comm.id) continue;
    ++s.calls;
    if (isP2p(e.op)) { ++s.p2p; ++peers[e.peer]; }
    if (isCollective(e.op)) { ++s.coll; sizes.push_back(e.logicalBytes); }
    if (e.op == TraceOp::AllGather) ++s.ag;
    if (e.op == TraceOp::ReduceScatter) ++s.rs;
    if (e.op == TraceOp::AllReduce) ++s.ar;
  }
  if (s.calls == 0) return s;
  s.p2pShare = (double)s.p2p / (double)s.calls;
  if (s.p2p) {
    uint64_t first = 0, second = 0;
    for (auto& kv : peers) {
      if (kv.second > first) { second = first; first = kv.second; }
      else if (kv.second > second) second = kv.second;
    }
    s.peerConcentration = (double)(first + second) / (double)s.p2p;
  }
  if (!sizes.empty()) { std::sort(sizes.begin(), sizes.end()); s.medianBytes = sizes[sizes.size() / 2]; }
  if (its.empty()) return s;

  std::map<std::vector<uint64_t>, int> all, buckets;
  std::vector<uint64_t> perIteration;
  std::vector<double> ratios;
  for (const IterationRange& it : its) {
    const IterationView v = viewOf(comm.id, ev, it);
    perIteration.push_back(v.calls);
    if (!v.pattern.empty()) {
      ++all[v.pattern];
      if (v.multiSize) ++buckets[v.pattern];
    }
    if (v.agBytes > 0 && v.rsBytes > 0) {
      const double r = v.agBytes / v.rsBytes;
      if (nearRatio(r, 0.5) || nearRatio(r, 0.25)) ratios.push_back(r);
    }
  }
  const double n = (double)its.size();
  std::sort(perIteration.begin(), perIteration.end());
  s.callsPerIteration = (double)perIteration[perIteration.size() / 2];
  int best = 0, bestBuckets = 0;
  for (auto& kv : all) best = std::max(best, kv.second);
  for (auto& kv : buckets) bestBuckets = std::max(bestBuckets, kv.second);
  s.patternSupport = (double)best / n;
  s.stable = s.coll != 0 && s.patternSupport >= kStablePattern;
  s.overlapSupport = (double)bestBuckets / n;
  s.ratioSupport = (double)ratios.size() / n;
  if (!ratios.empty()) { std::sort(ratios.begin(), ratios.end()); s.agToRs = ratios[ratios.size() / 2]; }
  return s;
}

// Share of iterations in which the `tp` flow sits inside or right before the `dp` flow. Two shapes count:
//   bracket: a dp all-gather, then at least two tp collectives, then a dp reduce-scatter (ZeRO / FSDP: parameters
//            gathered before the layers run, gradients scattered after);
//   tail:    at least two of the (up to eight) collectives that precede a dp reduce-scatter or all-reduce
//            belong to tp (gradient buckets drain behind the last layers).
double orderRelation(uint64_t dp, uint64_t tp, const std::vector<TraceEvent>& ev, const std::vector<IterationRange>& its) {
  if (its.empty()) return 0;
  int ok = 0;
  for (const IterationRange& it : its) {
    const size_t end = std::min(it.end, ev.size());
    bool bracket = false, tail = false;
    int sinceGather = -1;  // tp collectives since the last dp all-gather; -1 before any
    for (size_t i = it.begin; i < end && !bracket; ++i) {
      const TraceEvent& e = ev[i];
      if (e.commId == dp && e.op == TraceOp::AllGather) { if (sinceGather < 0) sinceGather = 0; }
      else if (e.commId == tp && isCollective(e.op)) { if (sinceGather >= 0) ++sinceGather; }
      else if (e.commId == dp && e.op == TraceOp::ReduceScatter && sinceGather >= 0) {
        if (sinceGather >= 2) bracket = true;
        else sinceGather = -1;  // this gather's window closed without a burst; a later gather opens a new one
      }
    }
    if (!bracket) {
      std::vector<uint64_t> recent;  // communicator of the last eight collectives
      for (size_t i = it.begin; i < end && !tail; ++i) {
        const TraceEvent& e = ev[i];
        if (!isCollective(e.op)) continue;
        if (e.commId == dp && (e.op == TraceOp::ReduceScatter || e.op == TraceOp::AllReduce))
          tail = std::count(recent.begin(), recent.end(), tp) >= 2;
        recent.push_back(e.commId);
        if (recent.size() > 8) recent.erase(recent.begin());
      }
    }
    if (bracket || tail) ++ok;
  }
  return (double)ok / (double)its.size();
}

// Share of iterations in which at least two of the communicator's collectives sit between two pipeline transfers.
double ppInterior(uint64_t id, const std::set<uint64_t>& pp, const std::vector<TraceEvent>& ev, const std::vector<IterationRange>& its) {
  if (its.empty() || pp.empty()) return 0;
  int ok = 0;
  for (const IterationRange& it : its) {
    const size_t end = std::min(it.end, ev.size());
    int burst = -1;  // collectives of `id` since the last transfer; -1 before the first transfer
    bool found = false;
    for (size_t i = it.begin; i < end && !found; ++i) {
      const TraceEvent& e = ev[i];
      if (pp.count(e.commId) && isP2p(e.op)) { found = burst >= 2; burst = 0; }
      else if (burst >= 0 && e.commId == id && isCollective(e.op)) ++burst;
    }
    if (found) ++ok;
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
