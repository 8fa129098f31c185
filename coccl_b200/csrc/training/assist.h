// Runtime side of training mode: records the calls of every communicator, decides their roles
// with the classifier and tells the router which role a communicator has.
//
// A role is reported only from call number 2 * iterations * callsPerIteration of that communicator
// on, so that every rank of the communicator (which sees the same call sequence) switches from the
// native to the compressed protocol at the same call. Only calls of at least 1 MiB are evidence; the
// trace holds at most 65,536 events, after which a 3-iteration fallback is tried once.
// Behavioural model: src/coccl-extend/core/training/coccl_training_assist.cc:24-392 and
// coccl_training_assist.h:11.
#pragma once
#include <map>
#include <mutex>
#include <vector>

#include "runtime/runtime.h"
#include "training/classifier.h"

namespace coccl {

constexpr size_t kTrainingMinEvidenceBytes = 1ull << 20;
constexpr size_t kTrainingMaxEvents = 65536;

class TrainingAssist : public RoleOracle {
 public:
  TrainingAssist(const ClassifierParams& params, int observationIterations)
      : params_(params), iterations_(observationIterations) {}
  void registerComm(Comm* comm);
  void unregisterComm(Comm* comm);
  void observe(const CallInfo& info, int groupDepth) override;
  Role roleOf(Comm* comm) override;
  // The classification of a communicator, whether or not routing has been activated yet.
  bool query(Comm* comm, Classification* out, uint64_t* activationCall = nullptr);
  size_t traceSize() const { return events_.size(); }
  // Clock used for timestamps (tests install a deterministic one).
  void setClock(uint64_t (*now)()) { now_ = now; }

 private:
  struct Entry {
    TraceComm comm;
    uint64_t observedCalls = 0;
    Classification classification;
    uint64_t activationCall = 0;
  };
  void commitTraceLocked(const std::vector<IterationRange>& iterations, int target);
  ClassifierParams params_;
  int iterations_;
  std::mutex mutex_;
  std::map<Comm*, Entry> entries_;
  std::vector<TraceEvent> events_;
  uint64_t sequence_ = 0;
  bool traceCommitted_ = false, fallbackTried_ = false;
  uint64_t (*now_)() = nullptr;
};

}  // namespace coccl
