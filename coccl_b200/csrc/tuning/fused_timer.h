// Times the one-shot and two-shot forms of a fused all-reduce in place of a call's first occurrence, for the
// C API's selector (tuning/measured.h). The candidate runs on the call's own input and stream, with its output sent
// to a scratch buffer so that the user's buffers are untouched; the time is the maximum over the ranks.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include <map>
#include <mutex>

#include "runtime/primitives.h"
#include "tuning/measured.h"

namespace coccl {

class FusedTimer : public AlgorithmTimer {
 public:
  explicit FusedTimer(FusedExecutor* executor) : executor_(executor) {}
  ~FusedTimer() override;
  bool measurable(Runtime* rt, const PreparedCall& call) override;
  bool time(Runtime* rt, const PreparedCall& call, Algorithm algorithm, double* seconds) override;
  // Sizes that are timed; calls outside take the nearest measured bucket (or the model).
  static constexpr size_t kMinBytes = 64u << 10, kMaxBytes = 256u << 20;
  static constexpr int kWarmup = 1, kIterations = 3;
  // Frees the communicator's scratch buffer (communicator destruction).
  void release(Comm* comm);

 private:
  struct Scratch { void* ptr = nullptr; size_t capacity = 0; };
  FusedExecutor* executor_;
  std::mutex mutex_;                    // guards the table; a communicator's entry is used by its own thread only
  std::map<Comm*, Scratch> scratch_;    // per communicator: ranks of one process sit on different devices
};

}  // namespace coccl
