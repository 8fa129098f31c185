// Selection from measured times of what really runs.
//
// The cost model of tuning/autotune.cc is fitted to the staged pipeline (codec kernels + transport), but on one
// NVSwitch domain most calls are served by ONE fused kernel whose one-shot and two-shot forms have their own
// crossover. This selector therefore keeps a table of measured times per (operation, datatype, ranks, size bucket)
// and picks the fastest supported entry; without an entry near the call it falls back to the model / heuristics of
// AutotuneSelector. The reference profiles at communicator creation and fits a model
// (src/coccl-extend/core/tuning/coccl_autotune_profiler.cc:62-618, coccl_autotune_selector.cc:12-165); here the table
// holds direct measurements of the kernels that serve the calls.
//
// Both front ends share it. The Python communicator times the candidates itself and writes the table through the
// routing session (cocclRouterSetMeasured). The C API gives the selector an AlgorithmTimer: at the first call of a
// size bucket the candidates are timed in place of the call (tuning/fused_timer.cc), every rank takes the maximum
// over the ranks, and the communicator's entries are identical on all of its ranks, so they select the same algorithm.
#pragma once
#include <atomic>
#include <map>
#include <mutex>
#include <set>
#include <utility>
#include <string>

#include "runtime/runtime.h"
#include "tuning/autotune.h"

namespace coccl {

class MeasuredTable {
 public:
  // `scope` separates communicators that share one table (the C API's process-wide table: the communicator's id,
  // which is never reused); a table that belongs to one communicator (a routing session) uses scope 0.
  struct Key {
    uint64_t scope;
    int op, dtype, nRanks, log2Bytes;
    bool operator<(const Key& o) const {
      if (scope != o.scope) return scope < o.scope;
      if (op != o.op) return op < o.op;
      if (dtype != o.dtype) return dtype < o.dtype;
      if (nRanks != o.nRanks) return nRanks < o.nRanks;
      return log2Bytes < o.log2Bytes;
    }
  };
  typedef std::map<int, double> Times;   // algorithm (or variant) -> seconds

  static int bucketOf(size_t bytes) {
    int lg = 0;
    while ((bytes >> (lg + 1)) != 0) ++lg;
    return lg;
  }
  // Every method takes the table's lock: ranks that live in one process as threads share the table.
  void set(int op, int dtype, int nRanks, int log2Bytes, int algorithm, double seconds, uint64_t scope = 0) {
    std::lock_guard<std::mutex> lock(mutex_);
    table_[Key{scope, op, dtype, nRanks, log2Bytes}][algorithm] = seconds;
  }
  bool empty() const { std::lock_guard<std::mutex> lock(mutex_); return table_.empty(); }
  size_t size() const { std::lock_guard<std::mutex> lock(mutex_); return table_.size(); }
  // Times of exactly this bucket (a copy); false when the bucket holds none.
  bool exact(int op, int dtype, int nRanks, int log2Bytes, Times* out = nullptr, uint64_t scope = 0) const {
    std::lock_guard<std::mutex> lock(mutex_);
    return find(scope, op, dtype, nRanks, log2Bytes, out);
  }
  // The bucket of `bytes`, else the nearest measured bucket below it, else (unless belowOnly) the nearest above.
  bool nearest(int op, int dtype, int nRanks, size_t bytes, Times* out, bool belowOnly = false, uint64_t scope = 0) const {
    std::lock_guard<std::mutex> lock(mutex_);
    const int lg = bucketOf(bytes);
    for (int d = 0; d < 48; ++d)
      if (find(scope, op, dtype, nRanks, lg - d, out)) return true;
    for (int d = 1; d < 48 && !belowOnly; ++d)
      if (find(scope, op, dtype, nRanks, lg + d, out)) return true;
    return false;
  }

 private:
  bool find(uint64_t scope, int op, int dtype, int nRanks, int log2Bytes, Times* out) const {
    auto it = table_.find(Key{scope, op, dtype, nRanks, log2Bytes});
    if (it == table_.end()) return false;
    if (out) *out = it->second;
    return true;
  }
  mutable std::mutex mutex_;
  std::map<Key, Times> table_;
};

// Times one candidate algorithm for a prepared call. Implementations are collective: every rank of the call's
// communicator calls time() for the same candidates in the same order, and all ranks get the same answer.
class AlgorithmTimer {
 public:
  virtual ~AlgorithmTimer() {}
  // Whether this call can be timed at all (depends on the call's sizes, codecs and the communicator only, so every
  // rank answers alike).
  virtual bool measurable(Runtime* rt, const PreparedCall& call) = 0;
  // false: this candidate could not be timed (on any rank); it gets no entry.
  virtual bool time(Runtime* rt, const PreparedCall& call, Algorithm algorithm, double* seconds) = 0;
};

class MeasuredSelector : public AlgorithmSelector {
 public:
  MeasuredSelector(ModelStore* store, MeasuredTable* table, AlgorithmTimer* timer = nullptr)
      : inner_(store), table_(table), timer_(timer) {}
  ncclResult_t select(Runtime* rt, PreparedCall* call) override;
  uint64_t measuredBuckets() const { return measuredBuckets_.load(); }

 private:
  void measure(Runtime* rt, PreparedCall* call, int log2Bytes);
  AutotuneSelector inner_;
  MeasuredTable* table_;
  AlgorithmTimer* timer_;
  std::atomic<uint64_t> measuredBuckets_{0};
  // Buckets (per communicator) whose timing was tried. Whether a call is timed must depend on the communicator's own
  // history only: the ranks of a communicator have seen the same calls on IT, but not on the other communicators each
  // of them belongs to, and a rank that timed alone would wait for peers that never come.
  std::mutex mutex_;
  std::set<MeasuredTable::Key> attempted_;
};

}  // namespace coccl
