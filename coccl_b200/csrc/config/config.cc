#include "config/config.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <algorithm>
#include <iomanip>
#include <limits>
#include <mutex>
#include <set>
#include <sstream>

#include "config/toml.h"

namespace coccl {

EffectiveScope effectiveScope(const PolicySlot& slot, Scope scope) {
  EffectiveScope e;
  const ScopeEntry& own = slot.configured(scope);
  if (scope != Scope::Default && own.configured) {
    e.entry = &own;
    e.source = scope;
    return e;
  }
  const ScopeEntry& def = slot.configured(Scope::Default);
  if (def.configured) {
    e.entry = &def;
    e.source = Scope::Default;
  }
  return e;
}

static const PolicyInfo kPolicies[kPolicyCount] = {
    {PolicyId::NormalAllGather, "normal.all_gather", Mode::Normal, Role::Normal, {Operation::AllGather, Variant::Default, Scope::Default}},
    {PolicyId::NormalReduceScatter, "normal.reduce_scatter", Mode::Normal, Role::Normal, {Operation::ReduceScatter, Variant::Default, Scope::Default}},
    {PolicyId::NormalAllReduce, "normal.all_reduce", Mode::Normal, Role::Normal, {Operation::AllReduce, Variant::Default, Scope::Default}},
    {PolicyId::NormalAllToAll, "normal.all_to_all", Mode::Normal, Role::Normal, {Operation::AllToAll, Variant::Default, Scope::Default}},
    {PolicyId::NormalSendRecv, "normal.sendrecv", Mode::Normal, Role::Normal, {Operation::SendRecv, Variant::Default, Scope::Default}},
    {PolicyId::DpAllGather, "training.dp.all_gather", Mode::Training, Role::DataParallel, {Operation::AllGather, Variant::Default, Scope::Default}},
    {PolicyId::DpReduceScatter, "training.dp.reduce_scatter", Mode::Training, Role::DataParallel, {Operation::ReduceScatter, Variant::Default, Scope::Default}},
    {PolicyId::DpAllReduce, "training.dp.all_reduce", Mode::Training, Role::DataParallel, {Operation::AllReduce, Variant::Default, Scope::Default}},
    {PolicyId::TpAllGather, "training.tp.all_gather", Mode::Training, Role::TensorParallel, {Operation::AllGather, Variant::Default, Scope::Default}},
    {PolicyId::TpReduceScatter, "training.tp.reduce_scatter", Mode::Training, Role::TensorParallel, {Operation::ReduceScatter, Variant::Default, Scope::Default}},
    {PolicyId::TpAllReduce, "training.tp.all_reduce", Mode::Training, Role::TensorParallel, {Operation::AllReduce, Variant::Default, Scope::Default}},
    {PolicyId::PpSendRecvForward, "training.pp.sendrecv.forward", Mode::Training, Role::PipelineParallel, {Operation::SendRecv, Variant::Forward, Scope::Default}},
    {PolicyId::PpSendRecvBackward, "training.pp.sendrecv.backward", Mode::Training, Role::PipelineParallel, {Operation::SendRecv, Variant::Backward, Scope::Default}},
};

const PolicyInfo& policyInfo(PolicyId id) { return kPolicies[static_cast<size_t>(id)]; }

bool findPolicy(Mode mode, Role role, Operation op, Variant variant, PolicyId* id) {
  for (const PolicyInfo& p : kPolicies) {
    if (p.mode != mode || p.key.op != op) continue;
    if (mode == Mode::Normal) {  // one send/recv policy serves both directions
      *id = p.id;
      return true;
    }
    if (p.role != role) continue;
    if (op == Operation::SendRecv && p.key.variant != variant) continue;
    *id = p.id;
    return true;
  }
  return false;
}

namespace {

struct Ctx {
  std::string* error;
  bool fail(const std::string& m) {
    if (error && error->empty()) *error = m;
    return false;
  }
};

bool onlyKeys(Ctx& c, const TomlValue& t, std::initializer_list<const char*> allowed, const std::string& path) {
  for (const auto& e : t.entries) {
    bool ok = false;
    for (const char* a : allowed) ok = ok || e.first == a;
    if (!ok) return c.fail("unknown key '" + e.first + "' in [" + (path.empty() ? "<root>" : path) + "]");
  }
  return true;
}

// optional child table; wrong kind is an error
bool childTable(Ctx& c, const TomlValue* parent, const char* key, const std::string& path, const TomlValue** out) {
  *out = nullptr;
  if (parent == nullptr) return true;
  const TomlValue* v = parent->find(key);
  if (v == nullptr) return true;
  if (!v->isTable()) return c.fail(path + "." + key + " must be a table");
  *out = v;
  return true;
}

bool readBool(Ctx& c, const TomlValue& t, const char* key, bool* out, const std::string& path) {
  const TomlValue* v = t.find(key);
  if (!v) return true;
  if (v->kind != TomlValue::kBool) return c.fail(path + "." + key + " must be a boolean");
  *out = v->boolean;
  return true;
}
bool readString(Ctx& c, const TomlValue& t, const char* key, std::string* out, bool required, const std::string& path) {
  const TomlValue* v = t.find(key);
  if (!v) return required ? c.fail(path + "." + key + " is required") : true;
  if (v->kind != TomlValue::kString) return c.fail(path + "." + key + " must be a string");
  *out = v->str;
  return true;
}
bool readInt(Ctx& c, const TomlValue& t, const char* key, int* out, int lo, int hi, bool required, const std::string& path) {
  const TomlValue* v = t.find(key);
  if (!v) return required ? c.fail(path + "." + key + " is required") : true;
  if (v->kind != TomlValue::kInteger) return c.fail(path + "." + key + " must be an integer");
  if (v->integer < lo || v->integer > hi)
    return c.fail(path + "." + key + " must be in [" + std::to_string(lo) + ", " + std::to_string(hi) + "]");
  *out = (int)v->integer;
  return true;
}
bool readSize(Ctx& c, const TomlValue& t, const char* key, size_t* out, const std::string& path, bool positive = false) {
  const TomlValue* v = t.find(key);
  if (!v) return true;
  if (v->kind != TomlValue::kInteger || v->integer < 0) return c.fail(path + "." + key + " must be a non-negative integer");
  if (positive && v->integer == 0) return c.fail(path + "." + key + " must be positive");
  *out = (size_t)v->integer;
  return true;
}

bool validName(const std::string& n) {
  if (n.empty()) return false;
  for (unsigned char ch : n)
    if (!(isalnum(ch) || ch == '_' || ch == '-')) return false;
  return true;
}

bool scalarText(const TomlValue& v, std::string* out) {
  switch (v.kind) {
    case TomlValue::kString: *out = v.str; return true;
    case TomlValue::kBool: *out = v.boolean ? "true" : "false"; return true;
    case TomlValue::kInteger: *out = std::to_string(v.integer); return true;
    case TomlValue::kFloat: {
      if (!std::isfinite(v.real)) return false;
      std::ostringstream ss;
      ss << std::setprecision(std::numeric_limits<double>::max_digits10) << v.real;
      *out = ss.str();
      return true;
    }
    default: return false;
  }
}

bool parseScope(Ctx& c, const TomlValue* t, ScopeEntry* s, const std::string& path) {
  *s = ScopeEntry();
  if (t == nullptr) return true;
  s->configured = true;
  s->enabled = true;
  if (!onlyKeys(c, *t, {"enabled", "compressor", "config"}, path)) return false;
  if (!readBool(c, *t, "enabled", &s->enabled, path)) return false;
  if (!readString(c, *t, "compressor", &s->compressor, s->enabled, path)) return false;
  const TomlValue* opts = nullptr;
  if (!childTable(c, t, "config", path, &opts)) return false;
  if (!s->enabled) {
    if (!s->compressor.empty() || opts != nullptr) return c.fail(path + ": a disabled scope cannot configure a compressor");
    return true;
  }
  if (!validName(s->compressor)) return c.fail(path + ".compressor: invalid compressor name '" + s->compressor + "'");
  if (opts != nullptr) {
    for (const auto& e : opts->entries) {
      std::string text;
      if (!scalarText(e.second, &text)) return c.fail(path + ".config." + e.first + " must be a string, integer, float or boolean");
      s->options[e.first] = text;
    }
  }
  return true;
}

bool parseSlot(Ctx& c, const TomlValue* t, PolicySlot* slot, size_t defaultThreshold, const std::string& path) {
  *slot = PolicySlot();
  slot->thresholdBytes = defaultThreshold;
  if (t == nullptr) return true;
  if (!onlyKeys(c, *t, {"threshold_bytes", "default", "intra", "inter"}, path)) return false;
  if (!readSize(c, *t, "threshold_bytes", &slot->thresholdBytes, path)) return false;
  static const char* names[] = {"default", "intra", "inter"};
  for (int i = 0; i < 3; ++i) {
    const TomlValue* st = nullptr;
    if (!childTable(c, t, names[i], path, &st)) return false;
    if (!parseScope(c, st, &slot->scopes[i], path + "." + names[i])) return false;
  }
  return true;
}

// walk "a.b.c" below root; every intermediate must be a table
bool tableAt(Ctx& c, const TomlValue& root, const std::string& path, const TomlValue** out) {
  const TomlValue* cur = &root;
  size_t start = 0;
  std::string walked;
  *out = nullptr;
  while (start <= path.size()) {
    size_t dot = path.find('.', start);
    std::string part = path.substr(start, dot == std::string::npos ? std::string::npos : dot - start);
    const TomlValue* next = nullptr;
    if (!childTable(c, cur, part.c_str(), walked.empty() ? "<root>" : walked, &next)) return false;
    if (next == nullptr) return true;
    walked = walked.empty() ? part : walked + "." + part;
    cur = next;
    if (dot == std::string::npos) break;
    start = dot + 1;
  }
  *out = cur;
  return true;
}

std::string dirOf(const std::string& path) {
  size_t s = path.find_last_of('/');
  return s == std::string::npos ? std::string(".") : path.substr(0, s == 0 ? 1 : s);
}

}  // namespace

bool loadConfigText(const std::string& text, const std::string& baseDir, Config* out, std::string* error) {
  if (error) error->clear();
  Ctx c{error};
  TomlValue root;
  std::string perr;
  if (!parseToml(text, &root, &perr)) return c.fail("TOML: " + perr);
  Config cfg;
  if (!onlyKeys(c, root, {"runtime", "compressor_plugins", "pipeline", "buffer", "autotune", "normal", "training"}, "")) return false;

  // [runtime]
  const TomlValue* rt = nullptr;
  if (!childTable(c, &root, "runtime", "<root>", &rt)) return false;
  if (rt == nullptr) return c.fail("[runtime] is required");
  if (!onlyKeys(c, *rt, {"mode", "compression_threshold_bytes", "fused_kernel_max_ctas"}, "runtime")) return false;
  std::string mode;
  if (!readString(c, *rt, "mode", &mode, true, "runtime")) return false;
  if (mode == "normal") cfg.mode = Mode::Normal;
  else if (mode == "training") cfg.mode = Mode::Training;
  else return c.fail("runtime.mode must be \"normal\" or \"training\"");
  if (!readSize(c, *rt, "compression_threshold_bytes", &cfg.thresholdBytes, "runtime")) return false;
  if (!readInt(c, *rt, "fused_kernel_max_ctas", &cfg.fusedMaxCtas, 0, 4096, false, "runtime")) return false;

  // [compressor_plugins]
  const TomlValue* pl = nullptr;
  if (!childTable(c, &root, "compressor_plugins", "<root>", &pl)) return false;
  if (pl != nullptr) {
    if (!onlyKeys(c, *pl, {"compressors", "library_path"}, "compressor_plugins")) return false;
    if (const TomlValue* arr = pl->find("compressors")) {
      if (arr->kind != TomlValue::kArray) return c.fail("compressor_plugins.compressors must be an array of strings");
      std::set<std::string> seen;
      for (const TomlValue& it : arr->items) {
        if (it.kind != TomlValue::kString) return c.fail("compressor_plugins.compressors must be an array of strings");
        if (!validName(it.str)) return c.fail("compressor_plugins.compressors: invalid compressor name '" + it.str + "'");
        if (!seen.insert(it.str).second) return c.fail("compressor_plugins.compressors: duplicate '" + it.str + "'");
        cfg.compressors.push_back(it.str);
      }
    }
    std::string lp;
    if (!readString(c, *pl, "library_path", &lp, !cfg.compressors.empty(), "compressor_plugins")) return false;
    if (!lp.empty()) cfg.libraryPath = (lp[0] == '/') ? lp : baseDir + "/" + lp;
  }

  // [pipeline]
  const TomlValue* pp = nullptr;
  if (!childTable(c, &root, "pipeline", "<root>", &pp)) return false;
  if (pp != nullptr) {
    if (!onlyKeys(c, *pp, {"depth"}, "pipeline")) return false;
    if (!readInt(c, *pp, "depth", &cfg.pipelineDepth, kMinPipelineDepth, kMaxPipelineDepth, false, "pipeline")) return false;
  }

  // [buffer]
  const TomlValue* bf = nullptr;
  if (!childTable(c, &root, "buffer", "<root>", &bf)) return false;
  if (bf != nullptr) {
    if (!onlyKeys(c, *bf, {"pool_limit_bytes", "legacy_block_bytes", "physical_chunk_bytes"}, "buffer")) return false;
    if (!readSize(c, *bf, "pool_limit_bytes", &cfg.poolLimitBytes, "buffer")) return false;
    if (!readSize(c, *bf, "legacy_block_bytes", &cfg.legacyBlockBytes, "buffer")) return false;
    if (!readSize(c, *bf, "physical_chunk_bytes", &cfg.physicalChunkBytes, "buffer", true)) return false;
  }

  // [autotune]
  const TomlValue* at = nullptr;
  if (!childTable(c, &root, "autotune", "<root>", &at)) return false;
  if (at != nullptr) {
    if (!onlyKeys(c, *at, {"enabled", "profile_min_bytes", "profile_max_bytes", "warmup", "iterations",
                           "reduce_scatter_algorithm", "all_reduce_algorithm"}, "autotune")) return false;
    if (!readBool(c, *at, "enabled", &cfg.autotune, "autotune")) return false;
    if (!readSize(c, *at, "profile_min_bytes", &cfg.profileMinBytes, "autotune", true)) return false;
    if (!readSize(c, *at, "profile_max_bytes", &cfg.profileMaxBytes, "autotune", true)) return false;
    if (cfg.profileMaxBytes < cfg.profileMinBytes) return c.fail("autotune.profile_max_bytes must be >= profile_min_bytes");
    if (!readInt(c, *at, "warmup", &cfg.autotuneWarmup, 0, 100000, false, "autotune")) return false;
    if (!readInt(c, *at, "iterations", &cfg.autotuneIterations, 1, 100000, false, "autotune")) return false;
    std::string a;
    if (!readString(c, *at, "reduce_scatter_algorithm", &a, false, "autotune")) return false;
    if (!a.empty()) {
      if (a == "auto") cfg.rsAlgorithm = RsAlgorithmPolicy::Auto;
      else if (a == "oneshot") cfg.rsAlgorithm = RsAlgorithmPolicy::OneShot;
      else if (a == "twoshot") cfg.rsAlgorithm = RsAlgorithmPolicy::TwoShot;
      else return c.fail("autotune.reduce_scatter_algorithm must be auto|oneshot|twoshot");
    }
    a.clear();
    if (!readString(c, *at, "all_reduce_algorithm", &a, false, "autotune")) return false;
    if (!a.empty()) {
      if (a == "auto") cfg.arAlgorithm = ArAlgorithmPolicy::Auto;
      else if (a == "oneshot") cfg.arAlgorithm = ArAlgorithmPolicy::OneShot;
      else if (a == "twoshot") cfg.arAlgorithm = ArAlgorithmPolicy::TwoShot;
      else if (a == "tripleshot") cfg.arAlgorithm = ArAlgorithmPolicy::TripleShot;
      else return c.fail("autotune.all_reduce_algorithm must be auto|oneshot|twoshot|tripleshot");
    }
  }

  // [normal.*]
  const TomlValue* nm = nullptr;
  if (!childTable(c, &root, "normal", "<root>", &nm)) return false;
  if (nm != nullptr && !onlyKeys(c, *nm, {"all_gather", "reduce_scatter", "all_reduce", "all_to_all", "sendrecv"}, "normal")) return false;

  // [training.*]
  const TomlValue* tr = nullptr;
  if (!childTable(c, &root, "training", "<root>", &tr)) return false;
  if (cfg.mode == Mode::Training && tr == nullptr) return c.fail("[training] is required in training mode");
  if (tr != nullptr) {
    if (!onlyKeys(c, *tr, {"observation_iterations", "classifier", "dp", "tp", "pp"}, "training")) return false;
    if (!readInt(c, *tr, "observation_iterations", &cfg.observationIterations, 2, 100, false, "training")) return false;
    const TomlValue* cl = nullptr;
    if (!childTable(c, tr, "classifier", "training", &cl)) return false;
    const bool need = cfg.mode == Mode::Training;
    if (need && cl == nullptr) return c.fail("[training.classifier] is required in training mode");
    if (cl != nullptr) {
      if (!onlyKeys(c, *cl, {"data_parallel_size", "tensor_parallel_size", "pipeline_parallel_size", "dp_strategy", "sequence_parallel"}, "training.classifier")) return false;
      const int big = 1 << 30;
      if (!readInt(c, *cl, "data_parallel_size", &cfg.dpSize, 1, big, need, "training.classifier")) return false;
      if (!readInt(c, *cl, "tensor_parallel_size", &cfg.tpSize, 1, big, need, "training.classifier")) return false;
      if (!readInt(c, *cl, "pipeline_parallel_size", &cfg.ppSize, 1, big, need, "training.classifier")) return false;
      std::string st;
      if (!readString(c, *cl, "dp_strategy", &st, false, "training.classifier")) return false;
      if (!st.empty()) {
        if (st == "ddp") cfg.dpStrategy = DpStrategy::Ddp;
        else if (st == "sdp") cfg.dpStrategy = DpStrategy::Sdp;
        else if (st == "fsdp") cfg.dpStrategy = DpStrategy::Fsdp;
        else return c.fail("training.classifier.dp_strategy must be ddp|sdp|fsdp");
      }
      if (!readBool(c, *cl, "sequence_parallel", &cfg.sequenceParallel, "training.classifier")) return false;
    }
    for (const char* grp : {"dp", "tp"}) {
      const TomlValue* g = nullptr;
      if (!childTable(c, tr, grp, "training", &g)) return false;
      if (g != nullptr && !onlyKeys(c, *g, {"all_gather", "reduce_scatter", "all_reduce"}, std::string("training.") + grp)) return false;
    }
    const TomlValue* ppt = nullptr;
    if (!childTable(c, tr, "pp", "training", &ppt)) return false;
    if (ppt != nullptr) {
      if (!onlyKeys(c, *ppt, {"sendrecv"}, "training.pp")) return false;
      const TomlValue* sr = nullptr;
      if (!childTable(c, ppt, "sendrecv", "training.pp", &sr)) return false;
      if (sr != nullptr && !onlyKeys(c, *sr, {"forward", "backward"}, "training.pp.sendrecv")) return false;
    }
  }

  // policy slots
  for (size_t i = 0; i < kPolicyCount; ++i) {
    const PolicyInfo& info = kPolicies[i];
    const TomlValue* t = nullptr;
    if (!tableAt(c, root, info.path, &t)) return false;
    if (!parseSlot(c, t, &cfg.slots[i], cfg.thresholdBytes, info.path)) return false;
    for (int s = 0; s < 3; ++s) {
      const ScopeEntry& e = cfg.slots[i].scopes[s];
      if (e.enabled && std::find(cfg.compressors.begin(), cfg.compressors.end(), e.compressor) == cfg.compressors.end())
        return c.fail(std::string(info.path) + "." + scopeName((Scope)s) + ".compressor '" + e.compressor +
                      "' is not listed in compressor_plugins.compressors");
    }
  }
  *out = cfg;
  return true;
}

bool loadConfigFile(const std::string& path, Config* out, std::string* error) {
  TomlValue dummy;
  std::string text;
  {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) {
      if (error) *error = "cannot open config file '" + path + "'";
      return false;
    }
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
    fclose(f);
  }
  return loadConfigText(text, dirOf(path), out, error);
}

std::string formatConfig(const Config& cfg) {
  std::ostringstream o;
  o << "runtime.mode = " << (cfg.mode == Mode::Normal ? "normal" : "training") << "\n";
  o << "runtime.compression_threshold_bytes = " << cfg.thresholdBytes << "\n";
  o << "runtime.fused_kernel_max_ctas = " << cfg.fusedMaxCtas << "\n";
  o << "compressor_plugins.compressors = [";
  for (size_t i = 0; i < cfg.compressors.size(); ++i) o << (i ? ", " : "") << cfg.compressors[i];
  o << "]\n";
  o << "compressor_plugins.library_path = " << cfg.libraryPath << "\n";
  o << "pipeline.depth = " << cfg.pipelineDepth << "\n";
  o << "buffer.pool_limit_bytes = " << cfg.poolLimitBytes << "\n";
  o << "buffer.legacy_block_bytes = " << cfg.legacyBlockBytes << "\n";
  o << "buffer.physical_chunk_bytes = " << cfg.physicalChunkBytes << "\n";
  o << "autotune.enabled = " << (cfg.autotune ? "true" : "false") << "\n";
  o << "autotune.profile_min_bytes = " << cfg.profileMinBytes << "\n";
  o << "autotune.profile_max_bytes = " << cfg.profileMaxBytes << "\n";
  o << "autotune.warmup = " << cfg.autotuneWarmup << "\n";
  o << "autotune.iterations = " << cfg.autotuneIterations << "\n";
  static const char* rs[] = {"auto", "oneshot", "twoshot"};
  static const char* ar[] = {"auto", "oneshot", "twoshot", "tripleshot"};
  o << "autotune.reduce_scatter_algorithm = " << rs[(int)cfg.rsAlgorithm] << "\n";
  o << "autotune.all_reduce_algorithm = " << ar[(int)cfg.arAlgorithm] << "\n";
  if (cfg.mode == Mode::Training) {
    static const char* st[] = {"ddp", "sdp", "fsdp"};
    o << "training.observation_iterations = " << cfg.observationIterations << "\n";
    o << "training.classifier.data_parallel_size = " << cfg.dpSize << "\n";
    o << "training.classifier.tensor_parallel_size = " << cfg.tpSize << "\n";
    o << "training.classifier.pipeline_parallel_size = " << cfg.ppSize << "\n";
    o << "training.classifier.dp_strategy = " << st[(int)cfg.dpStrategy] << "\n";
    o << "training.classifier.sequence_parallel = " << (cfg.sequenceParallel ? "true" : "false") << "\n";
  }
  for (size_t i = 0; i < kPolicyCount; ++i) {
    const PolicyInfo& info = kPolicies[i];
    if (info.mode != cfg.mode) continue;
    const PolicySlot& slot = cfg.slots[i];
    o << info.path << ".threshold_bytes = " << slot.thresholdBytes << "\n";
    for (int s = 0; s < 3; ++s) {
      EffectiveScope e = effectiveScope(slot, (Scope)s);
      const std::string p = std::string(info.path) + "." + scopeName((Scope)s);
      if (e.entry == nullptr) {
        o << p << ".enabled = false\n";
        continue;
      }
      o << "# " << p << " source=" << scopeName(e.source) << "\n";
      o << p << ".enabled = " << (e.entry->enabled ? "true" : "false") << "\n";
      if (!e.entry->enabled) continue;
      o << p << ".compressor = " << e.entry->compressor << "\n";
      for (const auto& kv : e.entry->options) o << p << ".config." << kv.first << " = " << kv.second << "\n";
    }
  }
  return o.str();
}

// ---------------------------------------------------------------------------
static std::mutex gProcMutex;
static ProcessConfig* gProc = nullptr;

static ProcessConfig* evaluateEnvironment() {
  ProcessConfig* p = new ProcessConfig();
  const char* en = getenv("COCCL_ENABLE");
  if (en == nullptr || *en == '\0' || std::string(en) == "0") return p;
  if (std::string(en) != "1") {
    p->valid = false;
    p->error = std::string("COCCL_ENABLE must be 0 or 1 (got '") + en + "'); compression stays disabled";
    return p;
  }
  const char* file = getenv("COCCL_CONFIG_FILE");
  if (file == nullptr || *file == '\0') {
    p->valid = false;
    p->error = "COCCL_ENABLE=1 requires COCCL_CONFIG_FILE; compression stays disabled";
    return p;
  }
  std::string err;
  if (!loadConfigFile(file, &p->config, &err)) {
    p->valid = false;
    p->error = "invalid COCCL_CONFIG_FILE '" + std::string(file) + "': " + err + "; compression stays disabled";
    return p;
  }
  p->enabled = true;
  return p;
}

const ProcessConfig& processConfig() {
  std::lock_guard<std::mutex> lock(gProcMutex);
  if (gProc == nullptr) {
    gProc = evaluateEnvironment();
    if (!gProc->valid) fprintf(stderr, "COCCL WARN %s\n", gProc->error.c_str());
  }
  return *gProc;
}

void resetProcessConfigForTesting() {
  std::lock_guard<std::mutex> lock(gProcMutex);
  delete gProc;
  gProc = nullptr;
}

}  // namespace coccl
