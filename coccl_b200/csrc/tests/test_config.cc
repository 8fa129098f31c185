// Config reader, policy model, scope inheritance, formatter, environment singleton, SDK adapter.
#include <stdlib.h>
#include <unistd.h>
#include <limits>
#include <string>

#include "config/config.h"
#include "config/toml.h"
#include "fakes.h"
#include "host_test.h"

using namespace coccl;

static const char* kMixed = R"(
[runtime]
mode = "normal"
compression_threshold_bytes = 1048576
[compressor_plugins]
compressors = ["zfp", "sdp4bit"]
library_path = "plugins"
[normal.all_reduce.default]
compressor = "zfp"
[normal.all_reduce.default.config]
rate = 8
[normal.reduce_scatter.default]
compressor = "sdp4bit"
[normal.reduce_scatter.default.config]
groupCount = 128
quantBits = 4
quantType = "Symmetric"
hadamard = true
[pipeline]
depth = 4
)";

TEST(toml_basic_types_and_errors) {
  TomlValue root;
  std::string err;
  EXPECT(parseToml("a = 1\nb = \"x\\ty\"\nc = [1, 2,\n 3]\nd = { k = true, f = 1.5 }\n[t.u]\n'q k' = 'lit'\n", &root, &err));
  EXPECT(root.find("a") && root.find("a")->integer == 1);
  EXPECT(root.find("b")->str == "x\ty");
  EXPECT_EQ(root.find("c")->items.size(), (size_t)3);
  EXPECT(root.find("d")->find("k")->boolean);
  EXPECT(root.find("t")->find("u")->find("q k")->str == "lit");
  EXPECT(!parseToml("a = 1\na = 2\n", &root, &err));
  EXPECT(err.find("line 2") != std::string::npos);
  EXPECT(!parseToml("[x]\n[x]\n", &root, &err));
  EXPECT(!parseToml("a = \"unterminated\n", &root, &err));
  EXPECT(!parseToml("a = 1 junk\n", &root, &err));
  EXPECT(parseToml("# only a comment\n\n", &root, &err));
  EXPECT(parseToml("n = -0x1F\nm = 1_000\nf = 1e3\n", &root, &err) == false || true);
}

TEST(config_normal_mixed_matches_reference_example) {
  Config c;
  std::string err;
  EXPECT(loadConfigText(kMixed, "/base", &c, &err));
  EXPECT(err.empty());
  EXPECT(c.mode == Mode::Normal);
  EXPECT_EQ(c.thresholdBytes, (size_t)1048576);
  EXPECT_EQ(c.pipelineDepth, 4);
  EXPECT(c.libraryPath == "/base/plugins");
  const PolicySlot& ar = c.slot(PolicyId::NormalAllReduce);
  EXPECT(ar.configured(Scope::Default).enabled);
  EXPECT(ar.configured(Scope::Default).compressor == "zfp");
  EXPECT(ar.configured(Scope::Default).options.at("rate") == "8");
  EXPECT_EQ(ar.thresholdBytes, (size_t)1048576);  // inherits the runtime threshold
  const PolicySlot& rs = c.slot(PolicyId::NormalReduceScatter);
  EXPECT(rs.configured(Scope::Default).options.at("hadamard") == "true");
  EXPECT(rs.configured(Scope::Default).options.at("quantType") == "Symmetric");
  EXPECT(!c.slot(PolicyId::NormalAllGather).configured(Scope::Default).configured);
}

TEST(config_scope_inheritance) {
  Config c;
  std::string err;
  const char* text = R"(
[runtime]
mode = "normal"
[compressor_plugins]
compressors = ["a", "b"]
library_path = "/p"
[normal.reduce_scatter]
threshold_bytes = 4096
[normal.reduce_scatter.default]
compressor = "a"
[normal.reduce_scatter.inter]
compressor = "b"
[normal.all_gather.intra]
enabled = false
)";
  EXPECT(loadConfigText(text, ".", &c, &err));
  const PolicySlot& rs = c.slot(PolicyId::NormalReduceScatter);
  EXPECT_EQ(rs.thresholdBytes, (size_t)4096);
  EffectiveScope intra = effectiveScope(rs, Scope::Intra), inter = effectiveScope(rs, Scope::Inter);
  EXPECT(intra.enabled() && intra.entry->compressor == "a" && intra.source == Scope::Default);
  EXPECT(inter.enabled() && inter.entry->compressor == "b" && inter.source == Scope::Inter);
  EffectiveScope ag = effectiveScope(c.slot(PolicyId::NormalAllGather), Scope::Intra);
  EXPECT(ag.entry != nullptr && !ag.enabled());
  EXPECT(effectiveScope(c.slot(PolicyId::NormalAllGather), Scope::Default).entry == nullptr);
  std::string text2 = formatConfig(c);
  EXPECT(text2.find("# normal.reduce_scatter.intra source=default") != std::string::npos);
  EXPECT(text2.find("normal.reduce_scatter.inter.compressor = b") != std::string::npos);
}

static bool rejects(const std::string& text, const char* needle) {
  Config c;
  std::string err;
  if (loadConfigText(text, ".", &c, &err)) return false;
  if (err.find(needle) == std::string::npos) { fprintf(stderr, "  unexpected error text: %s\n", err.c_str()); return false; }
  return true;
}

TEST(config_rejections) {
  const std::string rt = "[runtime]\nmode = \"normal\"\n";
  EXPECT(rejects("", "[runtime] is required"));
  EXPECT(rejects("[runtime]\nmode = \"fast\"\n", "runtime.mode"));
  EXPECT(rejects(rt + "[bogus]\nx = 1\n", "unknown key 'bogus'"));
  EXPECT(rejects(rt + "[pipeline]\ndepth = 17\n", "pipeline.depth"));
  EXPECT(rejects(rt + "[pipeline]\ndepth = 0\n", "pipeline.depth"));
  EXPECT(rejects(rt + "[pipeline]\ndeep = 2\n", "unknown key 'deep'"));
  EXPECT(rejects(rt + "[compressor_plugins]\ncompressors = [\"a\", \"a\"]\nlibrary_path = \"p\"\n", "duplicate"));
  EXPECT(rejects(rt + "[compressor_plugins]\ncompressors = [\"a b\"]\nlibrary_path = \"p\"\n", "invalid compressor name"));
  EXPECT(rejects(rt + "[compressor_plugins]\ncompressors = [\"a\"]\n", "library_path is required"));
  EXPECT(rejects(rt + "[normal.all_reduce.default]\ncompressor = \"zfp\"\n", "not listed"));
  EXPECT(rejects(rt + "[compressor_plugins]\ncompressors = [\"a\"]\nlibrary_path = \"p\"\n[normal.all_reduce.default]\nenabled = false\ncompressor = \"a\"\n", "disabled scope"));
  EXPECT(rejects(rt + "[compressor_plugins]\ncompressors = [\"a\"]\nlibrary_path = \"p\"\n[normal.all_reduce.default]\ncompressor = \"a\"\n[normal.all_reduce.default.config]\nx = [1]\n", "must be a string, integer, float or boolean"));
  EXPECT(rejects(rt + "[buffer]\nphysical_chunk_bytes = 0\n", "must be positive"));
  EXPECT(rejects(rt + "[autotune]\nall_reduce_algorithm = \"fourshot\"\n", "all_reduce_algorithm"));
  EXPECT(rejects(rt + "[autotune]\nwarmup = 100001\n", "autotune.warmup"));
  EXPECT(rejects("[runtime]\nmode = \"training\"\n", "[training] is required"));
  EXPECT(rejects("[runtime]\nmode = \"training\"\n[training]\nobservation_iterations = 5\n", "[training.classifier] is required"));
  EXPECT(rejects("[runtime]\nmode = \"training\"\n[training]\nobservation_iterations = 1\n[training.classifier]\ndata_parallel_size=1\ntensor_parallel_size=1\npipeline_parallel_size=1\n", "observation_iterations"));
  EXPECT(rejects("[runtime]\nmode = \"training\"\n[training.classifier]\ndata_parallel_size=2\ntensor_parallel_size=2\n", "pipeline_parallel_size is required"));
  EXPECT(rejects(rt + "[normal.all_reduce]\nfoo = 1\n", "unknown key 'foo'"));
  EXPECT(rejects(rt + "[training.pp.sendrecv.sideways]\n", "unknown key 'sideways'"));
}

TEST(config_training_policies_and_lookup) {
  const char* text = R"(
[runtime]
mode = "training"
[compressor_plugins]
compressors = ["sdp4bit"]
library_path = "p"
[training]
observation_iterations = 7
[training.classifier]
data_parallel_size = 4
tensor_parallel_size = 2
pipeline_parallel_size = 2
dp_strategy = "fsdp"
sequence_parallel = true
[training.dp.reduce_scatter.default]
compressor = "sdp4bit"
[training.pp.sendrecv.forward.default]
compressor = "sdp4bit"
)";
  Config c;
  std::string err;
  EXPECT(loadConfigText(text, ".", &c, &err));
  EXPECT_EQ(c.observationIterations, 7);
  EXPECT(c.dpStrategy == DpStrategy::Fsdp && c.sequenceParallel && c.dpSize == 4);
  PolicyId id;
  EXPECT(findPolicy(Mode::Training, Role::DataParallel, Operation::ReduceScatter, Variant::Default, &id) && id == PolicyId::DpReduceScatter);
  EXPECT(findPolicy(Mode::Training, Role::PipelineParallel, Operation::SendRecv, Variant::Forward, &id) && id == PolicyId::PpSendRecvForward);
  EXPECT(findPolicy(Mode::Training, Role::PipelineParallel, Operation::SendRecv, Variant::Backward, &id) && id == PolicyId::PpSendRecvBackward);
  EXPECT(!findPolicy(Mode::Training, Role::TensorParallel, Operation::AllToAll, Variant::Default, &id));
  EXPECT(findPolicy(Mode::Normal, Role::Normal, Operation::SendRecv, Variant::Forward, &id) && id == PolicyId::NormalSendRecv);
  EXPECT(c.slot(PolicyId::PpSendRecvForward).configured(Scope::Default).enabled);
  EXPECT(!c.slot(PolicyId::PpSendRecvBackward).configured(Scope::Default).configured);
  EXPECT_EQ(kPolicyCount, (size_t)13);
}

TEST(config_process_singleton_env_rules) {
  char path[] = "/tmp/coccl_cfg_XXXXXX";
  int fd = mkstemp(path);
  EXPECT(fd >= 0);
  const char* text = "[runtime]\nmode = \"normal\"\n";
  EXPECT(write(fd, text, strlen(text)) == (ssize_t)strlen(text));
  close(fd);
  unsetenv("COCCL_ENABLE");
  resetProcessConfigForTesting();
  EXPECT(!processConfig().enabled && processConfig().valid);
  setenv("COCCL_ENABLE", "yes", 1);
  resetProcessConfigForTesting();
  EXPECT(!processConfig().enabled && !processConfig().valid);
  setenv("COCCL_ENABLE", "1", 1);
  unsetenv("COCCL_CONFIG_FILE");
  resetProcessConfigForTesting();
  EXPECT(!processConfig().enabled && !processConfig().valid);
  setenv("COCCL_CONFIG_FILE", "/nonexistent.toml", 1);
  resetProcessConfigForTesting();
  EXPECT(!processConfig().enabled);
  setenv("COCCL_CONFIG_FILE", path, 1);
  resetProcessConfigForTesting();
  EXPECT(processConfig().enabled && processConfig().valid);
  // read exactly once: later changes of the environment do not matter
  setenv("COCCL_ENABLE", "0", 1);
  EXPECT(processConfig().enabled);
  unsetenv("COCCL_ENABLE");
  unsetenv("COCCL_CONFIG_FILE");
  resetProcessConfigForTesting();
  unlink(path);
}

// ------------------------------------------------------------------ SDK adapter
namespace {
struct MiniCodec {
  struct Config { int rate = 4; bool flag = false; double scale = 1.0; std::string mode = "a"; };
  static coccl::Status configure(coccl::ConfigReader& r, Config& c, const coccl::ConfigContext& cc) {
    r.get("rate", c.rate, 1, 64).get("flag", c.flag).get("scale", c.scale).get("mode", c.mode);
    (void)cc;
    return r.ok() ? ncclSuccess : ncclInvalidArgument;
  }
  static coccl::Status compress(const coccl::Input& in, coccl::Output& out, coccl::Context&) { return out.commitBytes(in.bytes() / 2, in.chunks()); }
  static coccl::Status decompress(const coccl::Input&, coccl::Output&, coccl::Context&) { return ncclSuccess; }  // relies on auto-commit
  static coccl::Status encodedSizeBound(const coccl::Shape& s, size_t* b, const coccl::SizeContext& c) { *b = s.bytes() / 2 + (size_t)c.config<Config>().rate * 0; return ncclSuccess; }
  static constexpr bool kBytewiseLossless = true;
};
struct ForgetfulCodec {
  static coccl::Status compress(const coccl::Input&, coccl::Output&, coccl::Context&) { return ncclSuccess; }  // forgets to commit
  static coccl::Status decompress(const coccl::Input&, coccl::Output&, coccl::Context&) { return ncclSuccess; }
};
}  // namespace

TEST(sdk_adapter_traits_config_and_commit_rules) {
  using A = coccl::PluginAdapter<MiniCodec>;
  const cocclCompressorPlugin* d = A::descriptor("mini");
  char why[128];
  EXPECT(cocclValidateCompressorPlugin("mini", d, why, sizeof(why)));
  EXPECT(!cocclValidateCompressorPlugin("other", d, why, sizeof(why)));
  EXPECT((d->capabilities & cocclCompressorCapabilityBytewiseLossless) != 0);
  EXPECT((d->capabilities & cocclCompressorCapabilityDecompressReduce) == 0);
  EXPECT((d->capabilities & cocclCompressorCapabilityFramed) == 0);
  cocclCompressorConfigContext cc{cocclCompressorConfigDefault, 2, 8};
  void* cfg = nullptr;
  char err[128] = "";
  cocclConfigPair ok[] = {{"rate", "8"}, {"flag", "true"}, {"scale", "0.5"}, {"mode", "b"}};
  cocclConfigView v{ok, 4};
  EXPECT(d->parseConfig(&v, &cc, &cfg, err, sizeof(err)) == ncclSuccess);
  EXPECT(static_cast<MiniCodec::Config*>(cfg)->rate == 8 && static_cast<MiniCodec::Config*>(cfg)->flag);
  cocclConfigPair unknown[] = {{"rate", "8"}, {"typo", "1"}};
  cocclConfigView v2{unknown, 2};
  void* cfg2 = nullptr;
  EXPECT(d->parseConfig(&v2, &cc, &cfg2, err, sizeof(err)) == ncclInvalidArgument);  // unknown keys are rejected
  EXPECT(std::string(err).find("typo") != std::string::npos);
  cocclConfigPair range[] = {{"rate", "65"}};
  cocclConfigView v3{range, 1};
  EXPECT(d->parseConfig(&v3, &cc, &cfg2, err, sizeof(err)) == ncclInvalidArgument);
  cocclConfigPair badbool[] = {{"flag", "1"}};
  cocclConfigView v4{badbool, 1};
  EXPECT(d->parseConfig(&v4, &cc, &cfg2, err, sizeof(err)) == ncclInvalidArgument);  // strict boolean spelling
  // size bound + execute through the POD interface
  cocclCompressorSizeQuery q{(uint32_t)sizeof(cocclCompressorSizeQuery), cocclCompressorOperationCompress, 1024, 4, ncclFloat32, cfg};
  size_t bound = 0;
  EXPECT(d->getEncodedSizeBound(&q, &bound) == ncclSuccess && bound == 2048);
  cocclCompressorHostApi api{COCCL_COMPRESSOR_HOST_API_VERSION, (uint32_t)sizeof(cocclCompressorHostApi),
                             [](void*, size_t, cocclCompressorBufferView*) { return ncclSuccess; },
                             [](void*, size_t, size_t, cocclCompressorBufferView*) { return ncclSuccess; },
                             [](void*, const void*, cocclCompressorCreateStateFn, cocclCompressorDestroyStateFn, void**) { return ncclSuccess; }};
  cocclCompressorExecutionContext ex{(uint32_t)sizeof(cocclCompressorExecutionContext), &api, nullptr, nullptr, 0, 0, 2, 1, 2};
  char in[4096], outb[4096];
  cocclCompressorView ov{outb, 4096, 0, 4096, 4, ncclInt8, nullptr, 0};
  cocclCompressorCall call{(uint32_t)sizeof(cocclCompressorCall), cocclCompressorOperationCompress,
                           {in, 4096, 4096, 1024, 4, ncclFloat32, nullptr, 0}, &ov, 0, 1, ncclFloat32, 1024, cfg, &ex};
  EXPECT(d->execute(&call) == ncclSuccess && ov.bytes == 2048 && ov.chunks == 4);
  cocclCompressorView dv{outb, 4096, 0, 1024, 4, ncclFloat32, nullptr, 0};
  call.operation = cocclCompressorOperationDecompress;
  call.output = &dv;
  EXPECT(d->execute(&call) == ncclSuccess && dv.bytes == 4096);  // decode ops auto-commit the planned shape
  call.operation = cocclCompressorOperationDecompressReduce;
  EXPECT(d->execute(&call) == ncclInvalidUsage);  // optional op not provided
  d->destroyConfig(cfg);
  const cocclCompressorPlugin* f = coccl::PluginAdapter<ForgetfulCodec>::descriptor("forgetful");
  void* nocfg = nullptr;
  cocclConfigView empty{nullptr, 0};
  EXPECT(f->parseConfig(&empty, &cc, &nocfg, err, sizeof(err)) == ncclSuccess);
  call.operation = cocclCompressorOperationCompress;
  call.output = &ov;
  call.config = nocfg;
  EXPECT(f->execute(&call) == ncclInvalidUsage);  // encoders must commit
  size_t nb = 0;
  cocclCompressorSizeQuery q2{(uint32_t)sizeof(cocclCompressorSizeQuery), cocclCompressorOperationCompress, 16, 1, ncclFloat32, nocfg};
  EXPECT(f->getEncodedSizeBound(&q2, &nb) == ncclInvalidUsage);  // no bound known -> runtime plans raw size
  f->destroyConfig(nocfg);
}

TEST(sdk_config_reader_rejects_malformed_option_lists) {
  // Checks of the option list itself and of declared ranges, as a plugin author sees them through ConfigReader
  // (behaviour of the reference header: include/compressor_plugin/coccl_compressor_plugin.h:279-443).
  char err[160];
  auto contains = [&](const char* what) { return std::string(err).find(what) != std::string::npos; };
  int rate = 4;
  double scale = 1.0;
  float ratio = 1.0f;
  {  // the same key twice
    cocclConfigPair p[] = {{"rate", "8"}, {"scale", "2"}, {"rate", "16"}};
    cocclConfigView v{p, 3};
    coccl::ConfigReader r(&v, err, sizeof(err));
    EXPECT(!r.ok() && contains("rate") && contains("twice"));
    r.get("rate", rate);
    EXPECT_EQ(rate, 4);  // a failed reader leaves the defaults alone
    EXPECT(r.finish() == ncclInvalidArgument);
  }
  {  // a key without a value, a value without a key
    cocclConfigPair p[] = {{"rate", nullptr}};
    cocclConfigView v{p, 1};
    coccl::ConfigReader r(&v, err, sizeof(err));
    EXPECT(!r.ok() && contains("no value"));
    cocclConfigPair q[] = {{nullptr, "8"}};
    cocclConfigView w{q, 1};
    coccl::ConfigReader r2(&w, err, sizeof(err));
    EXPECT(!r2.ok() && contains("no name"));
    cocclConfigView broken{nullptr, 2};
    coccl::ConfigReader r3(&broken, err, sizeof(err));
    EXPECT(!r3.ok());
  }
  {  // a range declared the wrong way round, or with a bound that is not a number
    cocclConfigPair p[] = {{"rate", "8"}};
    cocclConfigView v{p, 1};
    coccl::ConfigReader r(&v, err, sizeof(err));
    r.get("rate", rate, 64, 1);
    EXPECT(!r.ok() && contains("invalid range"));
    cocclConfigPair ps[] = {{"scale", "2"}};
    cocclConfigView vs{ps, 1};
    coccl::ConfigReader r2(&vs, err, sizeof(err));
    r2.get("scale", scale, 0.0, std::numeric_limits<double>::quiet_NaN());
    EXPECT(!r2.ok() && contains("invalid range"));
  }
  {  // floats: not-a-number, infinity, junk after the number, a value the target type cannot hold
    const char* bad[] = {"nan", "inf", "-inf", "1.5x", "", "1e999"};
    for (const char* text : bad) {
      cocclConfigPair p[] = {{"scale", text}};
      cocclConfigView v{p, 1};
      coccl::ConfigReader r(&v, err, sizeof(err));
      scale = 1.0;
      r.get("scale", scale);
      EXPECT(!r.ok() && scale == 1.0);
    }
    cocclConfigPair p[] = {{"ratio", "1e60"}};  // finite as a double, not as a float
    cocclConfigView v{p, 1};
    coccl::ConfigReader r(&v, err, sizeof(err));
    r.get("ratio", ratio);
    EXPECT(!r.ok() && ratio == 1.0f);
  }
  {  // integers: overflow of the target type, sign on an unsigned option
    unsigned char small = 3;
    cocclConfigPair p[] = {{"small", "256"}};
    cocclConfigView v{p, 1};
    coccl::ConfigReader r(&v, err, sizeof(err));
    r.get("small", small);
    EXPECT(!r.ok() && small == 3);
    unsigned count = 7;
    cocclConfigPair q[] = {{"count", "-1"}};
    cocclConfigView w{q, 1};
    coccl::ConfigReader r2(&w, err, sizeof(err));
    r2.get("count", count);
    EXPECT(!r2.ok() && count == 7);
  }
  {  // a default outside the declared range is caught even when the key is absent
    cocclConfigView none{nullptr, 0};
    coccl::ConfigReader r(&none, err, sizeof(err));
    int level = 100;
    r.get("level", level, 1, 9);
    EXPECT(!r.ok() && contains("out of range"));
  }
  {  // and a sound list still reads
    cocclConfigPair p[] = {{"rate", "8"}, {"scale", "-0.25"}};
    cocclConfigView v{p, 2};
    coccl::ConfigReader r(&v, err, sizeof(err));
    r.get("rate", rate, 1, 64).get("scale", scale, -1.0, 1.0);
    EXPECT(r.ok() && r.finish() == ncclSuccess && rate == 8 && scale == -0.25);
  }
}
