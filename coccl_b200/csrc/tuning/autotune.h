// Algorithm autotuner: linear cost models (time = alpha + beta * bytes) of the point-to-point
// links and of every enabled codec, the PCCA cost formulas of each reduce-scatter / all-reduce
// algorithm, the profiler that fits the models at communicator start-up, and the selector.
//
// Behavioural model: src/coccl-extend/core/tuning/coccl_autotune_cost_model.cc:9-167 (formulas,
// least-squares fit with >= 2 points and non-negative coefficients), coccl_autotune_internal.h:57-100
// (candidate table: hierarchical / divisible requirements, heuristic priority, fallback),
// coccl_autotune_profiler.cc:62-618 (profile sizes min, 4*min, ... plus the maximum; time = max
// over ranks; ratio = median), coccl_autotune_selector.cc:12-165 (eligibility, forced algorithm
// with fallback and warning, decision log on rank 0).
#pragma once
#include <map>
#include <string>
#include <vector>

#include "runtime/runtime.h"

namespace coccl {

struct LinearModel {
  double alpha = 0.0, beta = 0.0;  // seconds, seconds per byte
  bool valid = false;
  double time(double bytes) const { return alpha + beta * bytes; }
};
// Least squares over (bytes, seconds) samples; needs >= 2 finite points with distinct sizes;
// coefficients are clamped to be non-negative.
LinearModel fitLinear(const std::vector<std::pair<double, double>>& samples);

struct CodecModel {
  LinearModel roundTrip;  // compress + decompress of `bytes` raw bytes
  double ratio = 1.0;     // raw bytes / encoded bytes
  bool valid() const { return roundTrip.valid && ratio > 0.0; }
};

struct Topology {
  int nodes = 1, localRanks = 1;
  bool uniform = true;
  bool hierarchical() const { return nodes > 1 && localRanks > 1 && uniform; }
};

struct CostInputs {
  Topology topo;
  LinearModel intra, inter;          // p2p models
  CodecModel flat, intraCodec, interCodec, defaultCodec;  // flat = intra scope on one node, default scope otherwise
};

double costPcca(const LinearModel& p2p, const CodecModel& codec, double bytes, double ranks);
double costGlobalPcca(const CostInputs& in, const CodecModel& codec, double bytes);
// `bytes` = count * size (times nRanks for reduce-scatter). Returns +inf / NaN when a needed model is missing.
double costOf(Algorithm a, const CostInputs& in, double bytes);

struct Candidate {
  Algorithm algorithm;
  Operation op;
  bool hierarchical;       // needs nodes > 1, localRanks > 1 and a uniform layout
  bool divisibleByRanks;   // count must divide by the number of ranks
  int heuristicPriority;   // lower wins when no model is usable
  Algorithm unavailableFallback;
};
const std::vector<Candidate>& candidateTable();

struct Selection {
  Algorithm algorithm = Algorithm::None;
  bool usedModel = false;
  bool forced = false, fellBack = false;
  double scores[6] = {0, 0, 0, 0, 0, 0};  // by Algorithm
};

// Pure selection logic (no logging, no runtime): `supported(algo)` says whether the call's codecs and
// datatype allow the algorithm.
ncclResult_t chooseAlgorithm(Operation op, size_t count, size_t typeSize, int nRanks, const Topology& topo,
                             const CostInputs* models, Algorithm forced, bool (*supported)(Algorithm, void*),
                             void* ctx, Selection* out);

// Measured models shared by all communicators of the process.
class ModelStore {
 public:
  void setP2p(bool inter, const LinearModel& m) { (inter ? inter_ : intra_) = m; }
  const LinearModel& p2p(bool inter) const { return inter ? inter_ : intra_; }
  void setCodec(const CompressorPolicy* c, const CodecModel& m) { codecs_[c] = m; }
  const CodecModel* codec(const CompressorPolicy* c) const {
    auto it = codecs_.find(c);
    return it == codecs_.end() ? nullptr : &it->second;
  }
  void clear() { intra_ = inter_ = LinearModel(); codecs_.clear(); }
 private:
  LinearModel intra_, inter_;
  std::map<const CompressorPolicy*, CodecModel> codecs_;
};

// Production selector: cost model when every needed model is valid, heuristics otherwise; honours
// autotune.reduce_scatter_algorithm / all_reduce_algorithm from the configuration.
class AutotuneSelector : public AlgorithmSelector {
 public:
  explicit AutotuneSelector(ModelStore* store) : store_(store) {}
  ncclResult_t select(Runtime* rt, PreparedCall* call) override;
 private:
  ModelStore* store_;
};

// Profile sizes: min, 4*min, 16*min, ... < max, then max itself.
std::vector<size_t> profileSizes(size_t minBytes, size_t maxBytes);

// Measures the p2p ring and every enabled reduce-scatter / all-reduce codec on `comm` and fills the
// store. Collective: every rank of `comm` must call it. Failures leave the models invalid (the
// selector then uses heuristics).
ncclResult_t profileModels(Runtime* rt, Comm* comm, ModelStore* store, cudaStream_t stream);

}  // namespace coccl
