#include "tuning/autotune.h"

#include <math.h>
#include <algorithm>
#include <limits>

#include "runtime/log.h"

namespace coccl {

LinearModel fitLinear(const std::vector<std::pair<double, double>>& samples) {
  LinearModel m;
  std::vector<std::pair<double, double>> pts;
  for (const auto& s : samples)
    if (std::isfinite(s.first) && std::isfinite(s.second) && s.first >= 0 && s.second >= 0) pts.push_back(s);
  if (pts.size() < 2) return m;
  double sx = 0, sy = 0, sxx = 0, sxy = 0;
  for (const auto& p : pts) { sx += p.first; sy += p.second; sxx += p.first * p.first; sxy += p.first * p.second; }
  const double n = (double)pts.size();
  const double den = n * sxx - sx * sx;
  if (!(fabs(den) > 0)) return m;
  double beta = (n * sxy - sx * sy) / den;
  double alpha = (sy - beta * sx) / n;
  if (beta < 0) { beta = 0; alpha = sy / n; }
  if (alpha < 0) {  // refit through the origin
    alpha = 0;
    beta = sxx > 0 ? sxy / sxx : 0;
    if (beta < 0) beta = 0;
  }
  if (!std::isfinite(alpha) || !std::isfinite(beta)) return m;
  m.alpha = alpha;
  m.beta = beta;
  m.valid = true;
  return m;
}

static const double kInf = std::numeric_limits<double>::infinity();

double costPcca(const LinearModel& p2p, const CodecModel& codec, double bytes, double ranks) {
  if (!p2p.valid || !codec.valid() || ranks <= 0) return kInf;
  return codec.roundTrip.time(bytes) + p2p.time(bytes / (codec.ratio * ranks));
}

double costGlobalPcca(const CostInputs& in, const CodecModel& codec, double bytes) {
  if (!codec.valid()) return kInf;
  const double nodes = in.topo.nodes, local = in.topo.localRanks;
  double link = 0;
  if (in.topo.localRanks > 1) {
    if (!in.intra.valid) return kInf;
    link = std::max(link, in.intra.time(bytes / (nodes * local * codec.ratio)));
  }
  if (in.topo.nodes > 1) {
    if (!in.inter.valid) return kInf;
    link = std::max(link, in.inter.time(bytes * (nodes - 1) / (nodes * codec.ratio)));
  }
  return codec.roundTrip.time(bytes) + link;
}

double costOf(Algorithm a, const CostInputs& in, double M) {
  const double nodes = in.topo.nodes, local = in.topo.localRanks;
  switch (a) {
    case Algorithm::RsOneShot: return costGlobalPcca(in, in.flat, M);
    case Algorithm::RsTwoShot:
      return costPcca(in.intra, in.intraCodec, M, local) + costPcca(in.inter, in.interCodec, M / local, nodes);
    case Algorithm::ArOneShot: {
      double c = costPcca(in.intra, in.flat, M * local, local);
      if (in.topo.nodes > 1) c += costPcca(in.inter, in.flat, M * local * (nodes - 1), local * (nodes - 1) + 1);
      return c;
    }
    case Algorithm::ArTwoShot: return 2.0 * costGlobalPcca(in, in.flat, M);
    case Algorithm::ArTripleShot:
      return costOf(Algorithm::RsTwoShot, in, M) + costGlobalPcca(in, in.defaultCodec, M);
    default: return kInf;
  }
}

const std::vector<Candidate>& candidateTable() {
  static const std::vector<Candidate> t = {
      {Algorithm::RsTwoShot, Operation::ReduceScatter, true, false, 0, Algorithm::RsOneShot},
      {Algorithm::RsOneShot, Operation::ReduceScatter, false, false, 1, Algorithm::None},
      {Algorithm::ArTwoShot, Operation::AllReduce, false, true, 0, Algorithm::None},
      {Algorithm::ArOneShot, Operation::AllReduce, false, true, 1, Algorithm::None},
      {Algorithm::ArTripleShot, Operation::AllReduce, true, true, 2, Algorithm::ArTwoShot},
  };
  return t;
}

ncclResult_t chooseAlgorithm(Operation op, size_t count, size_t typeSize, int nRanks, const Topology& topo,
                             const CostInputs* models, Algorithm forced, bool (*supported)(Algorithm, void*),
                             void* ctx, Selection* out) {
  *out = Selection();
  auto eligible = [&](const Candidate& c) {
    if (c.op != op) return false;
    if (c.hierarchical && !topo.hierarchical()) return false;
    if (c.divisibleByRanks && nRanks > 0 && count % (size_t)nRanks != 0) return false;
    return supported == nullptr || supported(c.algorithm, ctx);
  };
  std::vector<const Candidate*> pool;
  for (const Candidate& c : candidateTable())
    if (eligible(c)) pool.push_back(&c);
  if (forced != Algorithm::None) {
    out->forced = true;
    Algorithm want = forced;
    for (int hop = 0; hop < 2 && want != Algorithm::None; ++hop) {
      const Candidate* def = nullptr;
      for (const Candidate& c : candidateTable())
        if (c.algorithm == want) def = &c;
      if (def == nullptr || def->op != op) break;
      if (eligible(*def)) {
        out->algorithm = want;
        return ncclSuccess;
      }
      want = def->unavailableFallback;
      out->fellBack = true;
    }
    // neither the forced algorithm nor its fallback can run: choose among what can
  }
  if (pool.empty()) return ncclInvalidUsage;
  double M = (double)count * (double)typeSize;
  if (op == Operation::ReduceScatter) M *= (double)nRanks;
  bool modelOk = models != nullptr;
  const Candidate* best = nullptr;
  double bestScore = kInf;
  if (modelOk) {
    for (const Candidate* c : pool) {
      const double s = costOf(c->algorithm, *models, M);
      out->scores[(int)c->algorithm] = s;
      if (!std::isfinite(s)) { modelOk = false; break; }
      if (s < bestScore) { bestScore = s; best = c; }
    }
  }
  if (!modelOk || best == nullptr) {
    best = pool[0];
    for (const Candidate* c : pool)
      if (c->heuristicPriority < best->heuristicPriority) best = c;
    out->usedModel = false;
  } else {
    out->usedModel = true;
  }
  out->algorithm = best->algorithm;
  return ncclSuccess;
}

// ------------------------------------------------------------------ production selector
namespace {
struct SupportCtx { const PreparedCall* call; };
bool supportedThunk(Algorithm a, void* p) { return algorithmSupported(*static_cast<SupportCtx*>(p)->call, a); }
}  // namespace

ncclResult_t AutotuneSelector::select(Runtime* rt, PreparedCall* call) {
  const Config& cfg = rt->config();
  const Comm* comm = call->info.comm;
  Topology topo{comm->nNodes, comm->localRanks, comm->uniform};
  Algorithm forced = Algorithm::None;
  if (call->info.op == Operation::ReduceScatter) {
    if (cfg.rsAlgorithm == RsAlgorithmPolicy::OneShot) forced = Algorithm::RsOneShot;
    if (cfg.rsAlgorithm == RsAlgorithmPolicy::TwoShot) forced = Algorithm::RsTwoShot;
  } else {
    if (cfg.arAlgorithm == ArAlgorithmPolicy::OneShot) forced = Algorithm::ArOneShot;
    if (cfg.arAlgorithm == ArAlgorithmPolicy::TwoShot) forced = Algorithm::ArTwoShot;
    if (cfg.arAlgorithm == ArAlgorithmPolicy::TripleShot) forced = Algorithm::ArTripleShot;
  }
  CostInputs in;
  const CostInputs* models = nullptr;
  if (cfg.autotune && store_ != nullptr) {
    in.topo = topo;
    in.intra = store_->p2p(false);
    in.inter = store_->p2p(true);
    auto model = [&](Scope s) {
      const CodecModel* m = call->codec(s) ? store_->codec(call->codec(s)) : nullptr;
      return m ? *m : CodecModel();
    };
    in.intraCodec = model(Scope::Intra);
    in.interCodec = model(Scope::Inter);
    in.defaultCodec = model(Scope::Default);
    in.flat = topo.nodes == 1 ? in.intraCodec : in.defaultCodec;
    models = &in;
  }
  SupportCtx ctx{call};
  Selection sel;
  ncclResult_t r = chooseAlgorithm(call->info.op, call->info.count, cocclTypeSize(call->info.datatype), comm->nRanks,
                                   topo, models, forced, &supportedThunk, &ctx, &sel);
  if (r != ncclSuccess) return r;
  if (sel.forced && sel.fellBack)
    COCCL_WARN("forced algorithm %s is not available for this call; using %s", algorithmName(forced), algorithmName(sel.algorithm));
  call->algorithm = sel.algorithm;
  if (comm->rank == 0)
    COCCL_INFO(kLogTuning, "select bytes=%zu one=%g two=%g triple=%g model=%d -> %s",
               call->info.count * cocclTypeSize(call->info.datatype),
               sel.scores[(int)(call->info.op == Operation::ReduceScatter ? Algorithm::RsOneShot : Algorithm::ArOneShot)],
               sel.scores[(int)(call->info.op == Operation::ReduceScatter ? Algorithm::RsTwoShot : Algorithm::ArTwoShot)],
               sel.scores[(int)Algorithm::ArTripleShot], (int)sel.usedModel, algorithmName(sel.algorithm));
  return ncclSuccess;
}

std::vector<size_t> profileSizes(size_t minBytes, size_t maxBytes) {
  std::vector<size_t> v;
  if (minBytes == 0 || maxBytes < minBytes) return v;
  for (size_t s = minBytes; s < maxBytes; s *= 4) {
    v.push_back(s);
    if (s > std::numeric_limits<size_t>::max() / 4) break;
  }
  v.push_back(maxBytes);
  return v;
}

}  // namespace coccl
