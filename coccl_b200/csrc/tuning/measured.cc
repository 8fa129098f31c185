#include "tuning/measured.h"

#include <vector>

#include "runtime/log.h"

namespace coccl {

void MeasuredSelector::measure(Runtime* rt, PreparedCall* call, int log2Bytes) {
  const int op = (int)call->info.op, dt = (int)call->info.datatype, n = call->info.comm->nRanks;
  const uint64_t scope = call->info.comm->id;
  std::vector<Algorithm> candidates;
  for (const Candidate& c : candidateTable())
    if (c.op == call->info.op && !c.hierarchical && algorithmSupported(*call, c.algorithm) &&
        (!c.divisibleByRanks || call->info.count % (size_t)n == 0))
      candidates.push_back(c.algorithm);
  if (candidates.size() < 2) return;   // nothing to choose between
  ++measuredBuckets_;
  for (Algorithm a : candidates) {
    double seconds = 0.0;
    if (timer_->time(rt, *call, a, &seconds) && seconds > 0.0) table_->set(op, dt, n, log2Bytes, (int)a, seconds, scope);
  }
}

ncclResult_t MeasuredSelector::select(Runtime* rt, PreparedCall* call) {
  const Config& cfg = rt->config();
  const bool forced = call->info.op == Operation::ReduceScatter ? cfg.rsAlgorithm != RsAlgorithmPolicy::Auto
                                                                : cfg.arAlgorithm != ArAlgorithmPolicy::Auto;
  if (cfg.autotune && !forced) {
    const size_t bytes = call->info.count * cocclTypeSize(call->info.datatype);
    const int op = (int)call->info.op, dt = (int)call->info.datatype, n = call->info.comm->nRanks;
    const int lg = MeasuredTable::bucketOf(bytes);
    // First call of a size bucket: time the candidates (once per bucket, also when nothing could be timed). Never
    // inside a group: the grouped calls run later, together.
    // with a timer the table is shared by the communicators of the process: entries carry the communicator's id
    const uint64_t scope = timer_ != nullptr ? call->info.comm->id : 0;
    if (timer_ != nullptr && rt->groupDepth() == 0) {
      bool first;
      {
        std::lock_guard<std::mutex> lock(mutex_);
        first = attempted_.insert(MeasuredTable::Key{scope, op, dt, n, lg}).second;
      }
      // the lock is not held while timing: the ranks of the communicator, threads of this process among them, meet there
      if (first && timer_->measurable(rt, *call)) measure(rt, call, lg);
    }
    MeasuredTable::Times best;
    if (table_->nearest(op, dt, n, bytes, &best, false, scope)) {
      int algo = 0;
      double t = 0.0;
      for (const auto& kv : best) {
        if (!algorithmSupported(*call, (Algorithm)kv.first)) continue;
        if (algo == 0 || kv.second < t) { algo = kv.first; t = kv.second; }
      }
      if (algo != 0) {
        call->algorithm = (Algorithm)algo;
        if (call->info.comm->rank == 0 && logEnabled(kLevelInfo, kLogTuning)) {
          std::string all;
          for (const auto& kv : best) all += std::string(algorithmName((Algorithm)kv.first)) + "=" + std::to_string(kv.second * 1e6) + "us ";
          COCCL_INFO(kLogTuning, "select bytes=%zu measured %s-> %s", bytes, all.c_str(), algorithmName(call->algorithm));
        }
        return ncclSuccess;
      }
    }
  }
  return inner_.select(rt, call);
}

}  // namespace coccl
