#include "compression/compressor_runtime.h"

#include <dlfcn.h>
#include <stdio.h>

#include "kernels/kernels_api.h"
#include "runtime/log.h"

namespace coccl {

// ------------------------------------------------------------------ allocator
static cudaError_t cudaMallocAsyncFn(void** p, size_t n, cudaStream_t s) { return cudaMallocAsync(p, n, s); }
static cudaError_t cudaFreeAsyncFn(void* p, cudaStream_t s) { return cudaFreeAsync(p, s); }
static cudaError_t cudaMallocFn(void** p, size_t n) { return cudaMalloc(p, n); }
static cudaError_t cudaFreeFn(void* p) { return cudaFree(p); }

const DeviceAllocator& cudaDeviceAllocator() {
  static const DeviceAllocator a = {&cudaMallocAsyncFn, &cudaFreeAsyncFn, &cudaMallocFn, &cudaFreeFn};
  return a;
}

static ReduceChunksFn gReduce = &cocclkReduceChunks;
void setReduceChunksHook(ReduceChunksFn fn) { gReduce = fn ? fn : &cocclkReduceChunks; }

// ------------------------------------------------------------------ policy
CompressorPolicy::CompressorPolicy(const LoadedPlugin* plugin, void* config, size_t thresholdBytes, std::string where)
    : plugin_(plugin), config_(config), thresholdBytes_(thresholdBytes), where_(std::move(where)) {}

CompressorPolicy::~CompressorPolicy() {
  releaseResources(cudaDeviceAllocator());
  if (config_ != nullptr && plugin_ != nullptr && plugin_->descriptor->destroyConfig != nullptr)
    plugin_->descriptor->destroyConfig(config_);
}

CompressorPolicy::DeviceResources& CompressorPolicy::resources(int device) { return perDevice_[device]; }

void CompressorPolicy::releaseResources(const DeviceAllocator& alloc) {
  std::lock_guard<std::mutex> lock(mutex_);
  for (auto& dev : perDevice_) {
    for (auto& p : dev.second.persistent)
      if (p.second.ptr) alloc.freeSync(p.second.ptr);
    for (auto& s : dev.second.states)
      if (s.second.ptr && s.second.destroy) s.second.destroy(s.second.ptr);
    if (dev.second.scratchPeak || dev.second.persistentBytes)
      COCCL_INFO(kLogCompress, "%s dev %d: scratch peak %zu B, persistent %zu B", where_.c_str(), dev.first,
                 dev.second.scratchPeak, dev.second.persistentBytes);
  }
  perDevice_.clear();
}

// ------------------------------------------------------------------ host API given to plugins
namespace {

struct CallContext {
  CompressorPolicy* policy;
  const ExecEnv* env;
  const DeviceAllocator* alloc;
  std::vector<void*> scratch;  // released (stream-ordered) when the call returns
  size_t scratchBytes = 0;
};

ncclResult_t hostAllocateScratch(void* context, size_t bytes, cocclCompressorBufferView* out) {
  CallContext* c = static_cast<CallContext*>(context);
  if (c == nullptr || out == nullptr) return ncclInvalidArgument;
  out->data = nullptr;
  out->bytes = 0;
  if (bytes == 0) return ncclSuccess;
  void* p = nullptr;
  if (c->alloc->mallocAsync(&p, bytes, c->env->stream) != cudaSuccess) return ncclUnhandledCudaError;
  c->scratch.push_back(p);
  c->scratchBytes += bytes;
  out->data = p;
  out->bytes = bytes;
  return ncclSuccess;
}

ncclResult_t hostAcquirePersistent(void* context, size_t slot, size_t bytes, cocclCompressorBufferView* out) {
  CallContext* c = static_cast<CallContext*>(context);
  if (c == nullptr || out == nullptr) return ncclInvalidArgument;
  std::lock_guard<std::mutex> lock(c->policy->mutex());
  auto& res = c->policy->resources(c->env->cudaDev);
  auto& slotRef = res.persistent[slot];
  if (slotRef.bytes < bytes) {  // grow: contents are not preserved, stateful codecs re-seed
    void* p = nullptr;
    if (c->alloc->mallocSync(&p, bytes) != cudaSuccess) return ncclUnhandledCudaError;
    if (slotRef.ptr) c->alloc->freeSync(slotRef.ptr);
    res.persistentBytes += bytes - slotRef.bytes;
    slotRef.ptr = p;
    slotRef.bytes = bytes;
  }
  out->data = slotRef.ptr;
  out->bytes = slotRef.bytes;
  return ncclSuccess;
}

ncclResult_t hostGetOrCreateState(void* context, const void* typeKey, cocclCompressorCreateStateFn create,
                                  cocclCompressorDestroyStateFn destroy, void** state) {
  CallContext* c = static_cast<CallContext*>(context);
  if (c == nullptr || typeKey == nullptr || create == nullptr || destroy == nullptr || state == nullptr)
    return ncclInvalidArgument;
  std::lock_guard<std::mutex> lock(c->policy->mutex());
  auto& st = c->policy->resources(c->env->cudaDev).states[typeKey];
  if (st.ptr == nullptr) {
    ncclResult_t r = create(&st.ptr);
    if (r != ncclSuccess) return r;
    st.destroy = destroy;
  }
  *state = st.ptr;
  return ncclSuccess;
}

const cocclCompressorHostApi kHostApi = {COCCL_COMPRESSOR_HOST_API_VERSION, (uint32_t)sizeof(cocclCompressorHostApi),
                                         &hostAllocateScratch, &hostAcquirePersistent, &hostGetOrCreateState};

// After an encoding operation the plugin's commit is checked before anything is put on the wire.
ncclResult_t validateEncoded(const CompressorPolicy* p, const cocclCompressorView& out) {
  const bool raw = out.datatype == COCCL_COMPRESSOR_RAW_PASSTHROUGH;
  if (out.datatype != ncclInt8 && !raw) return ncclInvalidUsage;
  if (out.chunks == 0 || out.bytes > out.capacityBytes || out.bytes == 0) return ncclInvalidUsage;
  if (!p->has(cocclCompressorCapabilityFramed) && out.bytes % out.chunks != 0) return ncclInvalidUsage;
  return ncclSuccess;
}

ncclResult_t runPlugin(CompressorPolicy* policy, cocclCompressorOperation op, const cocclCompressorView& input,
                       cocclCompressorView* output, size_t reduceChunks, ncclDataType_t originalDatatype,
                       size_t originalElements, const ExecEnv& env) {
  if (policy == nullptr || output == nullptr) return ncclInvalidArgument;
  CallContext ctx{policy, &env, env.alloc ? env.alloc : &cudaDeviceAllocator(), {}, 0};
  cocclCompressorExecutionContext ex;
  ex.structSize = sizeof(ex);
  ex.hostApi = &kHostApi;
  ex.hostContext = &ctx;
  ex.stream = env.stream;
  ex.cudaDev = env.cudaDev;
  ex.rank = env.rank;
  ex.nRanks = env.nRanks;
  ex.nodes = env.nodes;
  ex.devicesPerNode = env.devicesPerNode;
  cocclCompressorCall call;
  call.structSize = sizeof(call);
  call.operation = op;
  call.input = input;
  call.output = output;
  call.rank = env.rank;
  call.reduceChunks = reduceChunks;
  call.originalDatatype = originalDatatype;
  call.originalElements = originalElements;
  call.config = policy->config();
  call.execution = &ex;
  ncclResult_t r = policy->plugin()->descriptor->execute(&call);
  for (void* p : ctx.scratch) ctx.alloc->freeAsync(p, env.stream);
  {
    std::lock_guard<std::mutex> lock(policy->mutex());
    auto& res = policy->resources(env.cudaDev);
    if (ctx.scratchBytes > res.scratchPeak) res.scratchPeak = ctx.scratchBytes;
  }
  if (r != ncclSuccess) return r;
  const bool encodes = op == cocclCompressorOperationCompress || op == cocclCompressorOperationDecompressReduceCompress;
  return encodes ? validateEncoded(policy, *output) : ncclSuccess;
}

}  // namespace

// ------------------------------------------------------------------ runtime
CompressorRuntime::CompressorRuntime() {}
CompressorRuntime::~CompressorRuntime() { shutdown(); }

void CompressorRuntime::shutdown() {
  policies_.clear();
  for (auto& row : table_)
    for (auto& e : row) e = nullptr;
  for (auto& p : plugins_)
    if (p->handle) dlclose(p->handle);
  plugins_.clear();
  initialized_ = false;
}

void CompressorRuntime::addBuiltin(const cocclCompressorPlugin* d) {
  auto p = std::make_unique<LoadedPlugin>();
  p->name = d->name ? d->name : "";
  p->path = "<builtin>";
  p->descriptor = d;
  plugins_.push_back(std::move(p));
}

const LoadedPlugin* CompressorRuntime::findPlugin(const std::string& name) const {
  for (const auto& p : plugins_)
    if (p->name == name) return p.get();
  return nullptr;
}

bool CompressorRuntime::loadPlugin(const std::string& name, const std::string& dir, std::string* error) {
  if (findPlugin(name) != nullptr) return true;
  const std::string path = dir + "/lib" + name + ".so";
  void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (h == nullptr) {
    const char* why = dlerror();
    *error = "cannot load compressor '" + name + "' from " + path + ": " + (why ? why : "unknown error");
    return false;
  }
  auto entry = reinterpret_cast<cocclGetCompressorPluginFn>(dlsym(h, COCCL_COMPRESSOR_ENTRY_SYMBOL));
  if (entry == nullptr) {
    *error = path + " does not export " + COCCL_COMPRESSOR_ENTRY_SYMBOL;
    dlclose(h);
    return false;
  }
  const cocclCompressorPlugin* d = entry();
  char why[256] = "";
  if (!cocclValidateCompressorPlugin(name.c_str(), d, why, sizeof(why))) {
    *error = "compressor '" + name + "' rejected: " + why;
    dlclose(h);
    return false;
  }
  auto p = std::make_unique<LoadedPlugin>();
  p->name = name;
  p->path = path;
  p->handle = h;
  p->descriptor = d;
  p->fusedQuery = reinterpret_cast<int (*)(const void*, int, void*)>(dlsym(h, "cocclFusedCodecQuery"));
  p->deltaQuery = reinterpret_cast<int (*)(const void*, int, void*)>(dlsym(h, "cocclFusedCodecDeltaQuery"));
  plugins_.push_back(std::move(p));
  COCCL_INFO(kLogInit, "loaded compressor %s (capabilities 0x%llx) from %s", name.c_str(),
             (unsigned long long)d->capabilities, path.c_str());
  return true;
}

bool CompressorRuntime::initialize(const Config& cfg, int nodes, int devicesPerNode, std::string* error) {
  std::string err;
  cfg_ = cfg;
  for (const std::string& name : cfg.compressors)
    if (!loadPlugin(name, cfg.libraryPath, &err)) {
      if (error) *error = err;
      return false;
    }
  for (size_t i = 0; i < kPolicyCount; ++i) {
    const PolicyInfo& info = policyInfo((PolicyId)i);
    if (info.mode != cfg.mode) continue;
    const PolicySlot& slot = cfg.slots[i];
    CompressorPolicy* bySource[3] = {nullptr, nullptr, nullptr};
    for (int s = 0; s < 3; ++s) {
      EffectiveScope eff = effectiveScope(slot, (Scope)s);
      if (!eff.enabled()) continue;
      CompressorPolicy*& made = bySource[(int)eff.source];
      // intra/inter scopes get the hierarchical config variant even when they inherit the default
      // options, so an inherited scope is parsed separately from the default one
      const bool hierarchical = (Scope)s != Scope::Default;
      if (made == nullptr || hierarchical) {
        const LoadedPlugin* pl = findPlugin(eff.entry->compressor);
        if (pl == nullptr) {
          if (error) *error = std::string(info.path) + ": compressor '" + eff.entry->compressor + "' is not loaded";
          return false;
        }
        std::vector<cocclConfigPair> pairs;
        for (const auto& kv : eff.entry->options) pairs.push_back({kv.first.c_str(), kv.second.c_str()});
        cocclConfigView view{pairs.data(), pairs.size()};
        cocclCompressorConfigContext cc{hierarchical ? cocclCompressorConfigHierarchical : cocclCompressorConfigDefault,
                                        nodes, devicesPerNode};
        void* parsed = nullptr;
        char why[256] = "";
        ncclResult_t r = pl->descriptor->parseConfig(&view, &cc, &parsed, why, sizeof(why));
        if (r != ncclSuccess) {
          if (error)
            *error = std::string(info.path) + "." + scopeName((Scope)s) + ": compressor '" + pl->name +
                     "' rejected its options: " + (why[0] ? why : "invalid configuration");
          return false;
        }
        policies_.push_back(std::make_unique<CompressorPolicy>(pl, parsed, slot.thresholdBytes,
                                                               std::string(info.path) + "." + scopeName((Scope)s)));
        CompressorPolicy* np = policies_.back().get();
        if (!hierarchical) made = np;
        table_[i][s] = np;
      } else {
        table_[i][s] = made;
      }
    }
  }
  initialized_ = true;
  return true;
}

CompressorPolicy* CompressorRuntime::resolve(Role role, Variant variant, Operation op, Scope scope) const {
  PolicyId id;
  if (!initialized_ || !findPolicy(cfg_.mode, role, op, variant, &id)) return nullptr;
  return table_[(size_t)id][(size_t)scope];
}

size_t CompressorRuntime::thresholdFor(Role role, Variant variant, Operation op) const {
  PolicyId id;
  if (!findPolicy(cfg_.mode, role, op, variant, &id)) return cfg_.thresholdBytes;
  return cfg_.slots[(size_t)id].thresholdBytes;
}

// ------------------------------------------------------------------ size bound
ncclResult_t encodedSizeBound(const CompressorPolicy* policy, cocclCompressorOperation op, size_t elements,
                              size_t chunks, ncclDataType_t datatype, size_t* bytes) {
  if (policy == nullptr || bytes == nullptr || chunks == 0) return ncclInvalidArgument;
  const size_t width = cocclTypeSize(datatype);
  if (width == 0 || (elements != 0 && width > SIZE_MAX / elements)) return ncclInvalidArgument;
  const size_t raw = elements * width;
  const cocclCompressorPlugin* d = policy->plugin()->descriptor;
  if (d->getEncodedSizeBound == nullptr) {
    *bytes = raw;
    return ncclSuccess;
  }
  cocclCompressorSizeQuery q{(uint32_t)sizeof(cocclCompressorSizeQuery), op, elements, chunks, datatype, policy->config()};
  size_t b = 0;
  ncclResult_t r = d->getEncodedSizeBound(&q, &b);
  if (r == ncclInvalidUsage) {  // the codec has no bound for this shape: plan for raw bytes
    *bytes = raw;
    return ncclSuccess;
  }
  if (r != ncclSuccess) return r;
  if (b == 0 || b % chunks != 0) return ncclInvalidUsage;
  *bytes = b;
  return ncclSuccess;
}

// ------------------------------------------------------------------ operations
ncclResult_t compress(CompressorPolicy* policy, const cocclCompressorView& input, cocclCompressorView* output,
                      const ExecEnv& env) {
  return runPlugin(policy, cocclCompressorOperationCompress, input, output, 1, input.datatype, input.elements, env);
}

static ncclResult_t copyRaw(const cocclCompressorView& input, cocclCompressorView* output, const ExecEnv& env) {
  const size_t want = output->elements * cocclTypeSize(output->datatype);
  if (input.bytes != want || want > output->capacityBytes) return ncclInvalidUsage;
  if (input.data != output->data &&
      cudaMemcpyAsync(output->data, input.data, want, cudaMemcpyDeviceToDevice, env.stream) != cudaSuccess)
    return ncclUnhandledCudaError;
  output->bytes = want;
  return ncclSuccess;
}

ncclResult_t decompress(CompressorPolicy* policy, const cocclCompressorView& input, cocclCompressorView* output,
                        const ExecEnv& env) {
  // Raw pass-through is a plain copy, except for codecs that ask to see it (stateful ones seed from it).
  if (policy == nullptr || output == nullptr) return ncclInvalidArgument;
  if (input.datatype == COCCL_COMPRESSOR_RAW_PASSTHROUGH && !policy->has(cocclCompressorCapabilitySeesPassthrough))
    return copyRaw(input, output, env);
  return runPlugin(policy, cocclCompressorOperationDecompress, input, output, 1, output->datatype, output->elements, env);
}

ncclResult_t decompressReduce(CompressorPolicy* policy, const cocclCompressorView& input,
                              cocclCompressorView* output, size_t reduceChunks, const ExecEnv& env) {
  if (policy == nullptr || output == nullptr || reduceChunks == 0 || input.chunks % reduceChunks != 0)
    return ncclInvalidArgument;
  const bool raw = input.datatype == COCCL_COMPRESSOR_RAW_PASSTHROUGH;
  if (!raw && policy->has(cocclCompressorCapabilityDecompressReduce) && !policy->has(cocclCompressorCapabilityFramed)) {
    const ncclResult_t fusedResult = runPlugin(policy, cocclCompressorOperationDecompressReduce, input, output, reduceChunks,
                                               output->datatype, output->elements, env);
    // a codec may have the fused form for some of its configurations only (ZFP: the rates with a tile codec) and
    // answers "invalid usage" for the others before it touches anything: those take the generic path below
    if (fusedResult != ncclInvalidUsage) return fusedResult;
  }
  // generic path: decode all copies into scratch, then sum the chunks
  const DeviceAllocator* alloc = env.alloc ? env.alloc : &cudaDeviceAllocator();
  const size_t width = cocclTypeSize(output->datatype);
  const size_t outElems = output->elements;
  size_t allElems = 0, allBytes = 0;
  if (width == 0 || outElems == 0 || outElems > SIZE_MAX / reduceChunks) return ncclInvalidArgument;
  allElems = outElems * reduceChunks;
  if (allElems > SIZE_MAX / width) return ncclInvalidArgument;
  allBytes = allElems * width;
  void* tmp = nullptr;
  if (alloc->mallocAsync(&tmp, allBytes, env.stream) != cudaSuccess) return ncclUnhandledCudaError;
  cocclCompressorView decoded{tmp, allBytes, 0, allElems, input.chunks, output->datatype, nullptr, 0};
  ncclResult_t r = raw ? copyRaw(input, &decoded, env)
                       : runPlugin(policy, cocclCompressorOperationDecompress, input, &decoded, 1, output->datatype,
                                   allElems, env);
  if (r == ncclSuccess) {
    int rc = gReduce(tmp, output->data, (long)outElems, (int)reduceChunks, (long)outElems, (int)output->datatype, env.stream);
    r = rc == 0 ? ncclSuccess : (rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError);
  }
  alloc->freeAsync(tmp, env.stream);
  if (r == ncclSuccess) output->bytes = outElems * width;
  return r;
}

ncclResult_t decompressReduceCompress(CompressorPolicy* decoder, CompressorPolicy* encoder,
                                      const cocclCompressorView& input, cocclCompressorView* output,
                                      size_t reduceChunks, ncclDataType_t originalDatatype, size_t originalElements,
                                      const ExecEnv& env) {
  if (decoder == nullptr || encoder == nullptr || output == nullptr || reduceChunks == 0 ||
      input.chunks % reduceChunks != 0)
    return ncclInvalidArgument;
  const bool raw = input.datatype == COCCL_COMPRESSOR_RAW_PASSTHROUGH;
  if (!raw && decoder == encoder && decoder->has(cocclCompressorCapabilityDecompressReduceCompress) &&
      !decoder->has(cocclCompressorCapabilityFramed)) {
    const ncclResult_t fusedResult = runPlugin(decoder, cocclCompressorOperationDecompressReduceCompress, input, output,
                                               reduceChunks, originalDatatype, originalElements, env);
    if (fusedResult != ncclInvalidUsage) return fusedResult;   // see decompressReduce
  }
  const DeviceAllocator* alloc = env.alloc ? env.alloc : &cudaDeviceAllocator();
  const size_t width = cocclTypeSize(originalDatatype);
  if (width == 0 || originalElements == 0 || originalElements > SIZE_MAX / width) return ncclInvalidArgument;
  const size_t bytes = originalElements * width;
  void* tmp = nullptr;
  if (alloc->mallocAsync(&tmp, bytes, env.stream) != cudaSuccess) return ncclUnhandledCudaError;
  cocclCompressorView reduced{tmp, bytes, 0, originalElements, input.chunks / reduceChunks, originalDatatype, nullptr, 0};
  ncclResult_t r = decompressReduce(decoder, input, &reduced, reduceChunks, env);
  if (r == ncclSuccess) {
    reduced.bytes = bytes;
    r = compress(encoder, reduced, output, env);
  }
  alloc->freeAsync(tmp, env.stream);
  return r;
}

}  // namespace coccl
