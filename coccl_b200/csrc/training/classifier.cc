#include "training/classifier.h"

#include <algorithm>
#include <cmath>
#include <map>
#include <set>

namespace coccl {

namespace {

constexpr size_t kMinCycleEvents = 2;
constexpr double kCycleMatch = 0.90;
constexpr double kSampledMatch = 0.85;
constexpr size_t kMaxSamples = 16;
constexpr double kBoundaryGapScore = 2.0;
constexpr double kRoleEvidence = 0.60;
constexpr double kOverlapPattern = 0.80;
constexpr double kConflictMargin = 0.15;
constexpr double kPpShare = 0.70;
constexpr double kPeerConcentration = 0.80;
constexpr double kStablePattern = 0.60;

bool isCollective(TraceOp op) { return op == TraceOp::AllGather || op == TraceOp::ReduceScatter || op == TraceOp::AllReduce; }
bool isP2p(TraceOp op) { return op == TraceOp::Send || op == TraceOp::Recv; }

uint64_t mix(uint64_t v) {
  v ^= v >> 30; v *= 0xbf58476d1ce4e5b9ull;
  v ^= v >> 27; v *= 0x94d049bb133111ebull;
  return v ^ (v >> 31);
}
uint64_t token(const TraceEvent& e) {
  return mix(e.commId) ^ mix((uint64_t)e.op + 0x9e3779b9u) ^ mix((uint64_t)e.logicalBytes + 0x9e3779b97f4a7c15ull);
}

template <typename T>
T medianOf(std::vector<T> v) {
  if (v.empty()) return T{};
  const size_t mid = v.size() / 2;
  std::nth_element(v.begin(), v.begin() + mid, v.end());
  return v[mid];
}

// fraction of positions in the last (cycles-1)*period events that equal the event one period earlier
double periodMatch(const std::vector<uint64_t>& tok, size_t period, size_t cycles, bool sampled) {
  const size_t n = tok.size();
  const size_t span = (cycles - 1) * period;
  if (span == 0 || cycles * period > n) return 0.0;
  const size_t first = n - span;
  if (sampled) {
    const size_t samples = std::min(kMaxSamples, span);
    size_t hit = 0;
    for (size_t s = 0; s < samples; ++s) {
      const size_t i = first + (s * span) / samples;
      if (tok[i] == tok[i - period]) ++hit;
    }
    return (double)hit / (double)samples;
  }
  size_t hit = 0;
  for (size_t i = first; i < n; ++i)
    if (tok[i] == tok[i - period]) ++hit;
  return (double)hit / (double)span;
}

}  // namespace

const char* roleName(Role r) {
  switch (r) {
    case Role::Normal: return "normal";
    case Role::DataParallel: return "dp";
    case Role::TensorParallel: return "tp";
    case Role::PipelineParallel: return "pp";
    default: return "unknown";
  }
}

Role topologyRole(const TraceComm& comm, TraceOp op, const ClassifierParams& p) {
  if (isP2p(op)) return (p.ppSize > 1 && comm.nRanks == p.ppSize) ? Role::PipelineParallel : Role::Unknown;
  if (!isCollective(op)) return Role::Unknown;
  const bool dp = comm.nRanks == p.dpSize, tp = comm.nRanks == p.tpSize;
  if (dp == tp) return Role::Unknown;  // matches both or neither: size alone does not decide
  return dp ? Role::DataParallel : Role::TensorParallel;
}

bool detectIterations(const std::vector<TraceEvent>& events, int target, std::vector<IterationRange>* out) {
  if (out == nullptr) return false;
  out->clear();
  const size_t n = events.size();
  if (target < 2 || n < (size_t)target * kMinCycleEvents) return false;
  std::vector<uint64_t> tok(n);
  for (size_t i = 0; i < n; ++i) tok[i] = token(events[i]);

  bool haveTime = false;
  for (size_t i = 1; i < n && !haveTime; ++i) haveTime = events[i].timestampNs != events[0].timestampNs;

  // Candidate periods in ascending order. A candidate must repeat (>= 90 % agreement over the last
  // `target` cycles) AND, when timestamps are available, show a pause at its boundaries: an inner loop
  // (layers, micro-batches) repeats too, but only a training iteration ends in a gap (optimizer step,
  // data loading) of at least twice the median gap.
  size_t period = 0, cycles = 0, shift = 0;
  for (size_t p = kMinCycleEvents; p * (size_t)target <= n && period == 0; ++p) {
    if (periodMatch(tok, p, (size_t)target, true) < kSampledMatch) continue;
    if (periodMatch(tok, p, (size_t)target, false) < kCycleMatch) continue;
    size_t c = (size_t)target;
    while ((c + 1) * p <= n && periodMatch(tok, p, c + 1, false) >= kCycleMatch) ++c;
    if (!haveTime) { period = p; cycles = c; shift = 0; break; }
    const size_t start = n - c * p;
    std::vector<double> gaps;
    for (size_t i = start + 1; i < n; ++i) gaps.push_back((double)(events[i].timestampNs - events[i - 1].timestampNs));
    const double med = std::max(1.0, medianOf(gaps));
    double bestScore = 0.0;
    size_t bestShift = 0;
    for (size_t r = 0; r < p; ++r) {
      std::vector<double> bnd;
      for (size_t k = 1; k < c; ++k) {
        const size_t idx = start + k * p - r;  // boundary before event idx
        if (idx <= start || idx >= n) continue;
        bnd.push_back((double)(events[idx].timestampNs - events[idx - 1].timestampNs));
      }
      if (bnd.empty()) continue;
      const double score = medianOf(bnd) / med;
      if (score > bestScore) { bestScore = score; bestShift = r; }
    }
    if (bestScore < kBoundaryGapScore) continue;  // repeats, but is not an iteration
    // the rotation costs one cycle; keep at least `target`
    if (bestShift != 0 && c < (size_t)target + 1) continue;
    period = p; cycles = c; shift = bestShift;
  }
  if (period == 0) return false;
  // a rotation by `shift` drops the incomplete iteration at the end
  const size_t usable = shift == 0 ? cycles : cycles - 1;
  if (usable < 2) { shift = 0; }
  const size_t count = shift == 0 ? cycles : cycles - 1;
  const size_t end = n - shift;
  const size_t begin = end - count * period;
  for (size_t c = 0; c < count; ++c) out->push_back({begin + c * period, begin + (c + 1) * period});
  return !out->empty();
}

}  // namespace coccl
