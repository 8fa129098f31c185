// coccl-config-check [--nodes N] [--devices-per-node N] <config.toml>
// Parses a policy file, prints the effective configuration, loads every catalogued compressor
// plugin, validates its descriptor, and lets it parse (a) an empty option set and (b) the options of
// every configured policy scope, for a topology of nodes x devices-per-node (default 2 x 8).
// Exit status: 0 valid, 1 invalid, 2 usage.
// Same contract as src/coccl-extend/tools/coccl_config_check/coccl_config_check.cc:46-254.
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <map>
#include <string>
#include <vector>

#include "compressor_plugin/detail/coccl_compressor_abi.h"
#include "config/config.h"

using namespace coccl;

static int usage() {
  fprintf(stderr, "usage: coccl-config-check [--nodes N] [--devices-per-node N] <config.toml>\n");
  return 2;
}

static bool parseWith(const cocclCompressorPlugin* d, const OptionMap& opts, bool hierarchical, int nodes, int devs, std::string* why) {
  std::vector<cocclConfigPair> pairs;
  for (const auto& kv : opts) pairs.push_back({kv.first.c_str(), kv.second.c_str()});
  cocclConfigView view{pairs.data(), pairs.size()};
  cocclCompressorConfigContext cc{hierarchical ? cocclCompressorConfigHierarchical : cocclCompressorConfigDefault, nodes, devs};
  void* parsed = nullptr;
  char err[256] = "";
  ncclResult_t r = d->parseConfig(&view, &cc, &parsed, err, sizeof(err));
  if (r != ncclSuccess) {
    *why = err[0] ? err : "invalid configuration";
    return false;
  }
  if (parsed) d->destroyConfig(parsed);
  return true;
}

int main(int argc, char** argv) {
  int nodes = 2, devs = 8;
  const char* path = nullptr;
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--nodes") || !strcmp(argv[i], "--devices-per-node")) {
      if (i + 1 >= argc) return usage();
      const int v = atoi(argv[i + 1]);
      if (v <= 0) return usage();
      (argv[i][2] == 'n' ? nodes : devs) = v;
      ++i;
    } else if (argv[i][0] == '-') {
      return usage();
    } else if (path == nullptr) {
      path = argv[i];
    } else {
      return usage();
    }
  }
  if (path == nullptr) return usage();

  Config cfg;
  std::string err;
  if (!loadConfigFile(path, &cfg, &err)) {
    fprintf(stderr, "INVALID: %s\n", err.c_str());
    return 1;
  }
  fputs(formatConfig(cfg).c_str(), stdout);

  std::map<std::string, const cocclCompressorPlugin*> plugins;
  for (const std::string& name : cfg.compressors) {
    const std::string lib = cfg.libraryPath + "/lib" + name + ".so";
    void* h = dlopen(lib.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) {
      fprintf(stderr, "INVALID: cannot load %s: %s\n", lib.c_str(), dlerror());
      return 1;
    }
    auto entry = reinterpret_cast<cocclGetCompressorPluginFn>(dlsym(h, COCCL_COMPRESSOR_ENTRY_SYMBOL));
    if (!entry) {
      fprintf(stderr, "INVALID: %s does not export %s\n", lib.c_str(), COCCL_COMPRESSOR_ENTRY_SYMBOL);
      return 1;
    }
    const cocclCompressorPlugin* d = entry();
    char why[256] = "";
    if (!cocclValidateCompressorPlugin(name.c_str(), d, why, sizeof(why))) {
      fprintf(stderr, "INVALID: compressor '%s': %s\n", name.c_str(), why);
      return 1;
    }
    std::string perr;
    if (!parseWith(d, OptionMap(), false, nodes, devs, &perr)) {
      fprintf(stderr, "INVALID: compressor '%s' rejects its default options: %s\n", name.c_str(), perr.c_str());
      return 1;
    }
    printf("# plugin %s: ABI v%u, capabilities 0x%llx, %s\n", name.c_str(), d->abiVersion, (unsigned long long)d->capabilities, lib.c_str());
    plugins[name] = d;
  }
  for (size_t i = 0; i < kPolicyCount; ++i) {
    const PolicyInfo& info = policyInfo((PolicyId)i);
    if (info.mode != cfg.mode) continue;
    for (int s = 0; s < 3; ++s) {
      EffectiveScope e = effectiveScope(cfg.slots[i], (Scope)s);
      if (!e.enabled()) continue;
      auto it = plugins.find(e.entry->compressor);
      if (it == plugins.end()) {
        fprintf(stderr, "INVALID: %s.%s uses unknown compressor '%s'\n", info.path, scopeName((Scope)s), e.entry->compressor.c_str());
        return 1;
      }
      std::string perr;
      if (!parseWith(it->second, e.entry->options, (Scope)s != Scope::Default, nodes, devs, &perr)) {
        fprintf(stderr, "INVALID: %s.%s: compressor '%s' rejects its options: %s\n", info.path, scopeName((Scope)s),
                e.entry->compressor.c_str(), perr.c_str());
        return 1;
      }
    }
  }
  printf("# OK (%d nodes x %d devices)\n", nodes, devs);
  return 0;
}
