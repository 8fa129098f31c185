// Training-mode traffic classifier (pure CPU, no runtime pointers, deterministic).
//
// Given the calls observed on every communicator it answers "which parallel dimension does this
// communicator serve": data (DP), tensor (TP), pipeline (PP) or unknown. Three stages:
//   1 topology: a communicator whose size equals exactly one of the configured DP/TP sizes (or the
//     PP size for point-to-point traffic) is classified at once;
//   2 iteration detection: the longest periodic suffix of the call trace (>= 90 % token agreement,
//     sampled pre-check at 85 % on <= 16 samples, boundaries chosen where the time gap is >= 2x the
//     median gap);
//   3 evidence scoring per communicator over the detected iterations.
// Thresholds follow src/coccl-extend/core/training/coccl_training_classifier.cc:13-18 and :500-716:
// role evidence >= 0.60, overlap pattern (reduce-scatter buckets of two or more sizes repeating) >= 0.80, conflict margin 0.15, PP when the p2p share is
// >= 0.70 and the two busiest peers carry >= 0.80 of it, all-gather/reduce-scatter byte ratio within
// 20 % of 0.5 or 0.25, stable pattern = best per-iteration signature support >= 0.60, TP needs >= 2
// collectives per iteration on one node, a sparse node-local DP tail needs median bytes >= 1.25x
// the TP flow's. Evidence is scaled by min(1, iterations / target).
#pragma once
#include <stddef.h>
#include <stdint.h>
#include <vector>

#include "config/config.h"

namespace coccl {

enum class TraceOp : uint8_t { AllGather = 0, ReduceScatter, AllReduce, AllToAll, Send, Recv, Other };

struct TraceComm {
  uint64_t id = 0;
  int rank = 0, nRanks = 0, nNodes = 1, localRanks = 1;
};

struct TraceEvent {
  uint64_t sequence = 0;
  uint64_t commId = 0;
  TraceOp op = TraceOp::AllReduce;
  size_t logicalBytes = 0;
  int peer = -1;
  uint64_t timestampNs = 0;
  int groupDepth = 0;
};

struct IterationRange { size_t begin = 0, end = 0; };

struct Classification {
  Role role = Role::Unknown;
  Role candidate = Role::Unknown;
  double confidence = 0.0;
  bool committed = false;
  uint64_t observedCalls = 0;
  double cycleSupport = 0, overlapPatternSupport = 0, orderSupport = 0, agToRsRatio = 0, callsPerIteration = 0;
  size_t medianBytes = 0;
};

struct TraceResult { uint64_t commId = 0; Classification classification; };

struct ClassifierParams {
  int dpSize = 1, tpSize = 1, ppSize = 1;
  DpStrategy dpStrategy = DpStrategy::Sdp;
  bool sequenceParallel = false;
  static ClassifierParams from(const Config& c) {
    return {c.dpSize, c.tpSize, c.ppSize, c.dpStrategy, c.sequenceParallel};
  }
};

Role topologyRole(const TraceComm& comm, TraceOp op, const ClassifierParams& p);
bool detectIterations(const std::vector<TraceEvent>& events, int targetIterations, std::vector<IterationRange>* out);
void classifyTrace(const std::vector<TraceComm>& comms, const std::vector<TraceEvent>& events,
                   const std::vector<IterationRange>& iterations, int targetIterations, const ClassifierParams& p,
                   std::vector<TraceResult>* results);
const char* roleName(Role r);

}  // namespace coccl
