#include "training/assist.h"

#include <time.h>

#include "runtime/log.h"

namespace coccl {

static uint64_t monotonicNs() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

static TraceOp traceOp(const CallInfo& info) {
  switch (info.op) {
    case Operation::AllGather: return TraceOp::AllGather;
    case Operation::ReduceScatter: return TraceOp::ReduceScatter;
    case Operation::AllReduce: return TraceOp::AllReduce;
    case Operation::AllToAll: return TraceOp::AllToAll;
    case Operation::SendRecv: return info.func == Func::Send ? TraceOp::Send : TraceOp::Recv;
    default: return TraceOp::Other;
  }
}

void TrainingAssist::registerComm(Comm* comm) {
  if (comm == nullptr || comm->isChild) return;  // hierarchy children inherit their owner's traffic
  std::lock_guard<std::mutex> lock(mutex_);
  Entry& e = entries_[comm];
  e.comm.id = comm->id ? comm->id : (uint64_t)(uintptr_t)comm;
  e.comm.rank = comm->rank;
  e.comm.nRanks = comm->nRanks;
  e.comm.nNodes = comm->nNodes;
  e.comm.localRanks = comm->localRanks;
}

void TrainingAssist::unregisterComm(Comm* comm) {
  std::lock_guard<std::mutex> lock(mutex_);
  entries_.erase(comm);
}

void TrainingAssist::commitTraceLocked(const std::vector<IterationRange>& iterations, int target) {
  std::vector<TraceComm> comms;
  for (auto& kv : entries_) comms.push_back(kv.second.comm);
  std::vector<TraceResult> results;
  classifyTrace(comms, events_, iterations, target, params_, &results);
  for (auto& kv : entries_) {
    Entry& e = kv.second;
    if (e.classification.committed) continue;  // topology decisions stand
    for (const TraceResult& r : results) {
      if (r.commId != e.comm.id) continue;
      e.classification = r.classification;
      const double perIter = r.classification.callsPerIteration > 0 ? r.classification.callsPerIteration : 1.0;
      e.activationCall = (uint64_t)(2.0 * (double)iterations_ * perIter + 0.5);
      if (e.activationCall < e.observedCalls) {
        // round up to a whole number of iterations beyond what every rank has certainly seen
        const uint64_t step = (uint64_t)(perIter + 0.5) ? (uint64_t)(perIter + 0.5) : 1;
        e.activationCall = (e.observedCalls / step + 1) * step;
      }
      COCCL_INFO(kLogTuning, "training: comm %llu (size %d) -> %s confidence %.2f cycle %.2f overlap %.2f order %.2f ag/rs %.2f "
                 "calls/iter %.1f, routing from call %llu", (unsigned long long)e.comm.id, e.comm.nRanks,
                 roleName(e.classification.role), e.classification.confidence, e.classification.cycleSupport,
                 e.classification.overlapPatternSupport, e.classification.orderSupport, e.classification.agToRsRatio,
                 e.classification.callsPerIteration, (unsigned long long)e.activationCall);
    }
  }
  traceCommitted_ = true;
}

void TrainingAssist::observe(const CallInfo& info, int groupDepth) {
  if (info.comm == nullptr) return;
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = entries_.find(info.comm);
  if (it == entries_.end()) return;
  Entry& e = it->second;
  ++e.observedCalls;
  if (e.classification.committed) return;
  const TraceOp op = traceOp(info);
  const Role topo = topologyRole(e.comm, op, params_);
  if (topo != Role::Unknown) {
    e.classification.role = e.classification.candidate = topo;
    e.classification.confidence = 1.0;
    e.classification.committed = true;
    e.activationCall = e.observedCalls;  // every rank sees the same first call
    COCCL_INFO(kLogTuning, "training: comm %llu (size %d) -> %s by size", (unsigned long long)e.comm.id, e.comm.nRanks, roleName(topo));
    return;
  }
  if (traceCommitted_) return;
  size_t bytes = info.count * cocclTypeSize(info.datatype);
  if (info.op == Operation::AllGather || info.op == Operation::ReduceScatter || info.op == Operation::AllToAll) bytes *= (size_t)info.comm->nRanks;
  if (bytes < kTrainingMinEvidenceBytes) return;
  if (events_.size() < kTrainingMaxEvents) {
    TraceEvent ev;
    ev.sequence = sequence_++;
    ev.commId = e.comm.id;
    ev.op = op;
    ev.logicalBytes = bytes;
    ev.peer = info.peer;
    ev.timestampNs = now_ ? now_() : monotonicNs();
    ev.groupDepth = groupDepth;
    events_.push_back(ev);
  }
  std::vector<IterationRange> its;
  if (events_.size() >= (size_t)iterations_ * 2 && detectIterations(events_, iterations_, &its)) {
    commitTraceLocked(its, iterations_);
  } else if (events_.size() >= kTrainingMaxEvents && !fallbackTried_) {
    fallbackTried_ = true;
    if (detectIterations(events_, 3, &its)) commitTraceLocked(its, iterations_);
    else COCCL_WARN("training: no periodic pattern found in %zu calls; unclassified communicators stay native", events_.size());
  }
}

bool TrainingAssist::query(Comm* comm, Classification* out, uint64_t* activationCall) {
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = entries_.find(comm);
  if (it == entries_.end() || !it->second.classification.committed) return false;
  if (out) { *out = it->second.classification; out->observedCalls = it->second.observedCalls; }  // calls seen so far, not only those in the trace
  if (activationCall) *activationCall = it->second.activationCall;
  return true;
}

Role TrainingAssist::roleOf(Comm* comm) {
  std::lock_guard<std::mutex> lock(mutex_);
  // a hierarchy child is routed like its owner
  auto it = entries_.find(comm);
  if (it == entries_.end()) return Role::Unknown;
  const Entry& e = it->second;
  if (!e.classification.committed || e.observedCalls < e.activationCall) return Role::Unknown;
  return e.classification.role;
}

}  // namespace coccl
