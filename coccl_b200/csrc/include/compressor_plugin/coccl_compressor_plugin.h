// C++17 compressor-plugin SDK: what a codec author includes.
//
//   struct MyCodec {
//     struct Config { int rate = 4; };                                   // optional
//     static coccl::Status configure(coccl::ConfigReader& r, Config& c, const coccl::ConfigContext&);
//     static coccl::Status compress(const coccl::Input&, coccl::Output&, coccl::Context&);      // required
//     static coccl::Status decompress(const coccl::Input&, coccl::Output&, coccl::Context&);    // required
//     static coccl::Status decompressReduce(...);            // optional fused reduction
//     static coccl::Status decompressReduceCompress(...);    // optional fused reduce + re-encode
//     static coccl::Status encodedSizeBound(const coccl::Shape&, size_t* bytes, const coccl::SizeContext&);
//     static constexpr bool kFramed = false;                 // optional trait flags
//   };
//   COCCL_REGISTER_COMPRESSOR("mycodec", MyCodec)
//
// Four codec families are expressible: fixed-size (size bound is exact), framed
// variable-length (kFramed + commitFrames), stateful (Context::instance / persistent) and
// fused-reduction (the two optional operations). Rules a codec must follow: never call the
// collective library, never allocate (use Context::scratch / persistent), never synchronise
// the host, and commit the output of every encoding operation.
//
// Interface parity: src/coccl-extend/include/compressor_plugin/coccl_compressor_plugin.h
// (Input :88, Shape :116, SizeContext :136, Output :152-245, ConfigReader :279-443,
// Context :445-510, adapter :626-799, registration macro :810-815).
#ifndef COCCL_COMPRESSOR_PLUGIN_SDK_H_
#define COCCL_COMPRESSOR_PLUGIN_SDK_H_

#include <errno.h>
#include <stdlib.h>
#include <limits>
#include <new>
#include <string>
#include <type_traits>

#include "detail/coccl_compressor_abi.h"

namespace coccl {

using Status = ncclResult_t;

inline size_t dataTypeSize(ncclDataType_t t) { return cocclTypeSize(t); }
inline Status fromCuda(cudaError_t e) { return e == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError; }
inline bool checkedMultiply(size_t a, size_t b, size_t* out) {
  if (a != 0 && b > std::numeric_limits<size_t>::max() / a) return false;
  *out = a * b;
  return true;
}
inline bool checkedAdd(size_t a, size_t b, size_t* out) {
  if (b > std::numeric_limits<size_t>::max() - a) return false;
  *out = a + b;
  return true;
}

class Buffer {
 public:
  Buffer() : view_{nullptr, 0} {}
  explicit Buffer(cocclCompressorBufferView v) : view_(v) {}
  void* data() const { return view_.data; }
  size_t bytes() const { return view_.bytes; }
  template <typename T> T* dataAs() const { return static_cast<T*>(view_.data); }
  explicit operator bool() const { return view_.data != nullptr; }
  cocclCompressorBufferView* raw() { return &view_; }
 private:
  cocclCompressorBufferView view_;
};

// Read-only view of what the runtime hands to an operation.
class Input {
 public:
  explicit Input(const cocclCompressorView& v) : view_(&v) {}
  const void* data() const { return view_->data; }
  size_t bytes() const { return view_->bytes; }
  size_t elements() const { return view_->elements; }
  size_t chunks() const { return view_->chunks; }
  ncclDataType_t datatype() const { return view_->datatype; }
  bool framed() const { return view_->frameMetadata != nullptr; }
  const cocclCompressorFrameMetadata* frameMetadata() const { return view_->frameMetadata; }
  size_t frameStrideBytes() const { return view_->frameStrideBytes; }
  size_t elementsPerChunk() const { return view_->chunks == 0 ? 0 : view_->elements / view_->chunks; }
  template <typename T> const T* dataAs() const { return static_cast<const T*>(view_->data); }
 private:
  const cocclCompressorView* view_;
};

// Raw shape of a size-bound question.
class Shape {
 public:
  explicit Shape(const cocclCompressorSizeQuery& q) : q_(&q) {}
  size_t elements() const { return q_->elements; }
  size_t chunks() const { return q_->chunks; }
  ncclDataType_t datatype() const { return q_->datatype; }
  size_t bytes() const {
    size_t b = 0;
    return checkedMultiply(q_->elements, dataTypeSize(q_->datatype), &b) ? b : 0;
  }
  size_t elementsPerChunk() const { return q_->chunks == 0 ? 0 : q_->elements / q_->chunks; }
 private:
  const cocclCompressorSizeQuery* q_;
};

class SizeContext {
 public:
  explicit SizeContext(const cocclCompressorSizeQuery& q) : q_(&q) {}
  cocclCompressorOperation operation() const { return q_->operation; }
  template <typename Config> const Config& config() const { return *static_cast<const Config*>(q_->config); }
 private:
  const cocclCompressorSizeQuery* q_;
};

// Writable destination. A decode operation's planned shape (elements, chunks, datatype) is
// what the runtime expects back; an encode operation must commit what it produced.
class Output {
 public:
  explicit Output(cocclCompressorView* v) : view_(v) {
    if (v != nullptr) { plannedElements_ = v->elements; plannedChunks_ = v->chunks; plannedDatatype_ = v->datatype; }
  }
  void* data() const { return view_ ? view_->data : nullptr; }
  size_t capacityBytes() const { return view_ ? view_->capacityBytes : 0; }
  size_t elements() const { return plannedElements_; }
  size_t chunks() const { return plannedChunks_; }
  ncclDataType_t datatype() const { return plannedDatatype_; }
  bool framed() const { return view_ != nullptr && view_->frameMetadata != nullptr; }
  cocclCompressorFrameMetadata* frameMetadata() const { return view_ ? view_->frameMetadata : nullptr; }
  size_t frameStrideBytes() const { return view_ ? view_->frameStrideBytes : 0; }
  template <typename T> T* dataAs() const { return static_cast<T*>(data()); }

  Status commit(size_t elements, ncclDataType_t datatype, size_t chunks) {
    const size_t width = dataTypeSize(datatype);
    size_t bytes = 0;
    if (view_ == nullptr || view_->data == nullptr || chunks == 0 || width == 0 || elements % chunks != 0 ||
        !checkedMultiply(elements, width, &bytes) || bytes > view_->capacityBytes)
      return ncclInvalidArgument;
    view_->bytes = bytes;
    view_->elements = elements;
    view_->chunks = chunks;
    view_->datatype = datatype;
    committed_ = true;
    return ncclSuccess;
  }
  Status commitBytes(size_t bytes, size_t chunks) { return commit(bytes, ncclInt8, chunks); }
  Status commitFrames() {
    size_t bytes = 0;
    if (!framed() || view_->frameStrideBytes == 0 || plannedChunks_ == 0 ||
        !checkedMultiply(view_->frameStrideBytes, plannedChunks_, &bytes) || bytes > view_->capacityBytes)
      return ncclInvalidArgument;
    return commit(bytes, ncclInt8, plannedChunks_);
  }
  Status commitPlanned() { return commit(plannedElements_, plannedDatatype_, plannedChunks_); }
  // Declare that the input bytes were (or already are) in the output unchanged.
  Status commitPassthrough(const Input& in) { return commit(in.bytes(), COCCL_COMPRESSOR_RAW_PASSTHROUGH, in.chunks()); }
  // Copy the input through and mark it raw.
  Status passthrough(const Input& in, cudaStream_t stream) {
    if (view_ == nullptr || view_->data == nullptr || in.data() == nullptr || in.bytes() > view_->capacityBytes)
      return ncclInvalidArgument;
    if (view_->data != in.data()) {
      cudaError_t e = cudaMemcpyAsync(view_->data, in.data(), in.bytes(), cudaMemcpyDeviceToDevice, stream);
      if (e != cudaSuccess) return fromCuda(e);
    }
    return commitPassthrough(in);
  }
  bool committed() const { return committed_; }

 private:
  cocclCompressorView* view_ = nullptr;
  size_t plannedElements_ = 0, plannedChunks_ = 0;
  ncclDataType_t plannedDatatype_ = ncclInt8;
  bool committed_ = false;
};

// Encoding would expand the data: send it raw instead.
inline bool shouldPassthrough(const Input& in, size_t encodedBytes) { return encodedBytes > in.bytes(); }
inline bool isPassthrough(const Input& in) { return in.datatype() == COCCL_COMPRESSOR_RAW_PASSTHROUGH; }

template <typename Enum> struct EnumEntry { const char* name; Enum value; };

class ConfigContext {
 public:
  explicit ConfigContext(const cocclCompressorConfigContext* c) : c_(c) {}
  bool hierarchical() const { return c_ != nullptr && c_->variant == cocclCompressorConfigHierarchical; }
  int nodes() const { return c_ ? c_->nodes : 0; }
  int devicesPerNode() const { return c_ ? c_->devicesPerNode : 0; }
 private:
  const cocclCompressorConfigContext* c_;
};

// Typed access to the string options of a policy scope. Every key must be consumed:
// finish() fails on keys nobody asked for, so typos are rejected at load time.
class ConfigReader {
 public:
  ConfigReader(const cocclConfigView* values, char* error, size_t errorCapacity)
      : values_(values), error_(error), errorCapacity_(errorCapacity) {
    if (error_ && errorCapacity_) error_[0] = '\0';
    const size_t n = values_ ? values_->count : 0;
    if (n != 0 && values_->pairs == nullptr) { fail("?", "list is missing although its count is not zero"); return; }
    used_ = n ? new (std::nothrow) bool[n]() : nullptr;
    if (n && used_ == nullptr) { fail("?", "list could not be indexed (out of memory)"); return; }
    // The list itself must be sound before any key is read: every entry names a key and carries a value, and
    // no key appears twice (the second one would silently lose against the first).
    for (size_t i = 0; i < n && !failed_; ++i) {
      const char* key = values_->pairs[i].key;
      if (key == nullptr || key[0] == '\0') { fail("?", "has no name"); break; }
      if (values_->pairs[i].value == nullptr) { fail(key, "has no value"); break; }
      for (size_t j = 0; j < i; ++j)
        if (strcmp(values_->pairs[j].key, key) == 0) { fail(key, "is given twice"); break; }
    }
  }
  ~ConfigReader() { delete[] used_; }
  ConfigReader(const ConfigReader&) = delete;
  ConfigReader& operator=(const ConfigReader&) = delete;

  template <typename Value> ConfigReader& get(const char* key, Value& out) {
    bool found = false;
    const char* text = consume(key, &found);
    if (found && !failed_ && !parse(text, &out)) fail(key, "has an invalid value");
    return *this;
  }
  // Range-checked read. The default the caller put into `out` is checked too, so a plugin cannot ship a default
  // outside its own range; bounds given the wrong way round or (for floats) not finite are a plugin bug and fail.
  template <typename Value> ConfigReader& get(const char* key, Value& out, Value lo, Value hi) {
    if (!failed_ && (!finite(lo) || !finite(hi) || hi < lo)) { fail(key, "was declared with an invalid range"); return *this; }
    get(key, out);
    if (!failed_ && !(out >= lo && out <= hi)) fail(key, "is out of range");
    return *this;
  }
  template <typename Enum, size_t N> ConfigReader& getEnum(const char* key, Enum& out, const EnumEntry<Enum> (&table)[N]) {
    bool found = false;
    const char* text = consume(key, &found);
    if (!found || failed_) return *this;
    for (size_t i = 0; i < N; ++i)
      if (strcmp(table[i].name, text) == 0) { out = table[i].value; return *this; }
    fail(key, "has an unknown enumerator");
    return *this;
  }
  Status finish() {
    if (failed_) return ncclInvalidArgument;
    const size_t n = values_ ? values_->count : 0;
    for (size_t i = 0; i < n; ++i)
      if (!used_[i]) { fail(values_->pairs[i].key, "is not a recognised option"); return ncclInvalidArgument; }
    return ncclSuccess;
  }
  bool ok() const { return !failed_; }
  void fail(const char* key, const char* reason) {
    if (!failed_ && error_ && errorCapacity_) snprintf(error_, errorCapacity_, "option '%s' %s", key ? key : "?", reason);
    failed_ = true;
  }

 private:
  const char* consume(const char* key, bool* found) {
    *found = false;
    const size_t n = values_ ? values_->count : 0;
    for (size_t i = 0; i < n; ++i) {
      if (values_->pairs[i].key && strcmp(values_->pairs[i].key, key) == 0) {
        used_[i] = true;
        *found = true;
        return values_->pairs[i].value ? values_->pairs[i].value : "";
      }
    }
    return nullptr;
  }
  template <typename V, typename std::enable_if<std::is_integral<V>::value && !std::is_same<V, bool>::value, int>::type = 0>
  static bool parse(const char* text, V* out) {
    if (*text == '\0') return false;
    errno = 0;
    char* end = nullptr;
    if (std::is_signed<V>::value) {
      long long v = strtoll(text, &end, 10);
      if (errno || *end || v < (long long)std::numeric_limits<V>::min() || v > (long long)std::numeric_limits<V>::max()) return false;
      *out = (V)v;
    } else {
      if (*text == '-') return false;
      unsigned long long v = strtoull(text, &end, 10);
      if (errno || *end || v > (unsigned long long)std::numeric_limits<V>::max()) return false;
      *out = (V)v;
    }
    return true;
  }
  template <typename V, typename std::enable_if<std::is_floating_point<V>::value, int>::type = 0>
  static bool parse(const char* text, V* out) {
    if (*text == '\0') return false;
    errno = 0;
    char* end = nullptr;
    double v = strtod(text, &end);
    if (errno || end == text || *end) return false;
    // "nan", "inf" and values the target type cannot hold are not options a codec can work with
    if (!(v == v) || v > (double)std::numeric_limits<V>::max() || v < -(double)std::numeric_limits<V>::max()) return false;
    *out = (V)v;
    return true;
  }
  template <typename V> static bool finite(V v) {
    return !std::is_floating_point<V>::value || (v == v && v <= std::numeric_limits<V>::max() && v >= std::numeric_limits<V>::lowest());
  }
  static bool parse(const char* text, bool* out) {
    if (strcmp(text, "true") == 0) { *out = true; return true; }
    if (strcmp(text, "false") == 0) { *out = false; return true; }
    return false;
  }
  static bool parse(const char* text, std::string* out) { *out = text; return true; }

  const cocclConfigView* values_;
  bool* used_ = nullptr;
  bool failed_ = false;
  char* error_;
  size_t errorCapacity_;
};

// Execution-time services.
class Context {
 public:
  explicit Context(cocclCompressorCall* call) : call_(call) {}
  cudaStream_t stream() const { return call_->execution->stream; }
  int cudaDevice() const { return call_->execution->cudaDev; }
  int rank() const { return call_->execution->rank; }
  int ranks() const { return call_->execution->nRanks; }
  int nodes() const { return call_->execution->nodes; }
  int devicesPerNode() const { return call_->execution->devicesPerNode; }
  size_t reduceChunks() const { return call_->reduceChunks; }
  ncclDataType_t originalDatatype() const { return call_->originalDatatype; }
  size_t originalElements() const { return call_->originalElements; }
  template <typename Config> const Config& config() const { return *static_cast<const Config*>(call_->config); }

  // Stream-ordered temporary memory, released by the runtime after the call.
  Status scratch(size_t bytes, Buffer* out) {
    return call_->execution->hostApi->allocateScratch(call_->execution->hostContext, bytes, out->raw());
  }
  // Memory that survives across calls, addressed by a small slot number; grows on demand.
  Status persistent(size_t slot, size_t bytes, Buffer* out) {
    return call_->execution->hostApi->acquirePersistent(call_->execution->hostContext, slot, bytes, out->raw());
  }
  // One host-side State object per (policy, device), created on first use.
  template <typename State> Status instance(State** out) {
    static const char key = 0;  // address identifies the State type
    void* p = nullptr;
    Status s = call_->execution->hostApi->getOrCreateState(call_->execution->hostContext, &key, &createState<State>,
                                                           &destroyState<State>, &p);
    if (s == ncclSuccess) *out = static_cast<State*>(p);
    return s;
  }

 private:
  template <typename State> static Status createState(void** p) {
    State* s = new (std::nothrow) State();
    if (!s) return ncclSystemError;
    *p = s;
    return ncclSuccess;
  }
  template <typename State> static void destroyState(void* p) { delete static_cast<State*>(p); }
  cocclCompressorCall* call_;
};

struct EmptyConfig {};

namespace detail {
template <typename...> using VoidT = void;

template <typename C, typename = void> struct ConfigOf { using type = EmptyConfig; static constexpr bool present = false; };
template <typename C> struct ConfigOf<C, VoidT<typename C::Config>> { using type = typename C::Config; static constexpr bool present = true; };

#define COCCL_SDK_DETECT(Name, expr)                                                   \
  template <typename C, typename = void> struct Name : std::false_type {};             \
  template <typename C> struct Name<C, VoidT<decltype(expr)>> : std::true_type {};
COCCL_SDK_DETECT(HasConfigure, C::configure(std::declval<ConfigReader&>(), std::declval<typename ConfigOf<C>::type&>(), std::declval<const ConfigContext&>()))
COCCL_SDK_DETECT(HasCompress, C::compress(std::declval<const Input&>(), std::declval<Output&>(), std::declval<Context&>()))
COCCL_SDK_DETECT(HasDecompress, C::decompress(std::declval<const Input&>(), std::declval<Output&>(), std::declval<Context&>()))
COCCL_SDK_DETECT(HasDecompressReduce, C::decompressReduce(std::declval<const Input&>(), std::declval<Output&>(), std::declval<Context&>()))
COCCL_SDK_DETECT(HasDecompressReduceCompress, C::decompressReduceCompress(std::declval<const Input&>(), std::declval<Output&>(), std::declval<Context&>()))
COCCL_SDK_DETECT(HasEncodedSizeBound, C::encodedSizeBound(std::declval<const Shape&>(), std::declval<size_t*>(), std::declval<const SizeContext&>()))
#undef COCCL_SDK_DETECT

#define COCCL_SDK_FLAG(Name, member)                                                   \
  template <typename C, typename = void> struct Name { static constexpr bool value = false; }; \
  template <typename C> struct Name<C, VoidT<decltype(C::member)>> { static constexpr bool value = C::member; };
COCCL_SDK_FLAG(IsFramed, kFramed)
COCCL_SDK_FLAG(HasFusedSwizzle, kFusedHierarchicalSwizzle)
COCCL_SDK_FLAG(IsBytewiseLossless, kBytewiseLossless)
COCCL_SDK_FLAG(SeesPassthrough, kSeesPassthrough)
#undef COCCL_SDK_FLAG
}  // namespace detail

// Turns a codec class into the POD descriptor, detecting optional members at compile time.
template <typename C>
struct PluginAdapter {
  using Config = typename detail::ConfigOf<C>::type;
  static_assert(detail::HasCompress<C>::value, "a compressor must define static Status compress(const Input&, Output&, Context&)");
  static_assert(detail::HasDecompress<C>::value, "a compressor must define static Status decompress(const Input&, Output&, Context&)");
  static_assert(!detail::HasConfigure<C>::value || detail::ConfigOf<C>::present, "configure() needs a nested Config type");

  static constexpr uint64_t capabilities() {
    return cocclCompressorCapabilityCompress | cocclCompressorCapabilityDecompress |
           (detail::HasDecompressReduce<C>::value ? cocclCompressorCapabilityDecompressReduce : 0) |
           (detail::HasDecompressReduceCompress<C>::value ? cocclCompressorCapabilityDecompressReduceCompress : 0) |
           (detail::IsFramed<C>::value ? cocclCompressorCapabilityFramed : 0) |
           (detail::HasFusedSwizzle<C>::value ? cocclCompressorCapabilityFusedHierarchicalSwizzle : 0) |
           (detail::IsBytewiseLossless<C>::value ? cocclCompressorCapabilityBytewiseLossless : 0) |
           (detail::SeesPassthrough<C>::value ? cocclCompressorCapabilitySeesPassthrough : 0);
  }

  static Status execute(cocclCompressorCall* call) {
    if (call == nullptr || call->structSize != sizeof(*call) || call->execution == nullptr ||
        call->execution->structSize != sizeof(*call->execution) || call->output == nullptr)
      return ncclInvalidArgument;
    const cocclCompressorHostApi* api = call->execution->hostApi;
    if (api == nullptr || api->abiVersion != COCCL_COMPRESSOR_HOST_API_VERSION || api->structSize != sizeof(*api) ||
        api->allocateScratch == nullptr || api->acquirePersistent == nullptr || api->getOrCreateState == nullptr)
      return ncclInvalidArgument;
    Input in(call->input);
    Output out(call->output);
    Context ctx(call);
    Status s = ncclInvalidUsage;
    bool encodes = false;
    switch (call->operation) {
      case cocclCompressorOperationCompress: encodes = true; s = C::compress(in, out, ctx); break;
      case cocclCompressorOperationDecompress: s = C::decompress(in, out, ctx); break;
      case cocclCompressorOperationDecompressReduce: s = callDecompressReduce(in, out, ctx); break;
      case cocclCompressorOperationDecompressReduceCompress: encodes = true; s = callDrc(in, out, ctx); break;
      default: return ncclInvalidArgument;
    }
    if (s != ncclSuccess) return s;
    if (encodes) return out.committed() ? ncclSuccess : ncclInvalidUsage;  // encoders must say what they wrote
    return out.committed() ? ncclSuccess : out.commitPlanned();
  }

  static Status parseConfig(const cocclConfigView* values, const cocclCompressorConfigContext* context, void** parsed,
                            char* error, size_t errorCapacity) {
    if (parsed == nullptr || context == nullptr) return ncclInvalidArgument;
    *parsed = nullptr;
    Config* cfg = new (std::nothrow) Config();
    if (cfg == nullptr) return ncclSystemError;
    ConfigReader reader(values, error, errorCapacity);
    Status s = configureIfPresent(reader, *cfg, ConfigContext(context));
    if (s == ncclSuccess) s = reader.finish();
    if (s != ncclSuccess) { delete cfg; return s; }
    *parsed = cfg;
    return ncclSuccess;
  }
  static void destroyConfig(void* cfg) { delete static_cast<Config*>(cfg); }

  static Status getEncodedSizeBound(const cocclCompressorSizeQuery* q, size_t* bytes) {
    if (q == nullptr || bytes == nullptr || q->structSize != sizeof(*q)) return ncclInvalidArgument;
    return callSizeBound(Shape(*q), bytes, SizeContext(*q));
  }

  static const cocclCompressorPlugin* descriptor(const char* name) {
    static const cocclCompressorPlugin d = {COCCL_COMPRESSOR_ABI_VERSION, (uint32_t)sizeof(cocclCompressorPlugin), name,
                                            capabilities(), &execute, &parseConfig, &destroyConfig, &getEncodedSizeBound};
    return &d;
  }

 private:
  template <typename T = C> static typename std::enable_if<detail::HasConfigure<T>::value, Status>::type
  configureIfPresent(ConfigReader& r, Config& c, const ConfigContext& cc) { return T::configure(r, c, cc); }
  template <typename T = C> static typename std::enable_if<!detail::HasConfigure<T>::value, Status>::type
  configureIfPresent(ConfigReader&, Config&, const ConfigContext&) { return ncclSuccess; }

  template <typename T = C> static typename std::enable_if<detail::HasEncodedSizeBound<T>::value, Status>::type
  callSizeBound(const Shape& s, size_t* b, const SizeContext& c) { return T::encodedSizeBound(s, b, c); }
  template <typename T = C> static typename std::enable_if<!detail::HasEncodedSizeBound<T>::value, Status>::type
  callSizeBound(const Shape&, size_t*, const SizeContext&) { return ncclInvalidUsage; }  // runtime falls back to raw size

  template <typename T = C> static typename std::enable_if<detail::HasDecompressReduce<T>::value, Status>::type
  callDecompressReduce(const Input& i, Output& o, Context& c) { return T::decompressReduce(i, o, c); }
  template <typename T = C> static typename std::enable_if<!detail::HasDecompressReduce<T>::value, Status>::type
  callDecompressReduce(const Input&, Output&, Context&) { return ncclInvalidUsage; }

  template <typename T = C> static typename std::enable_if<detail::HasDecompressReduceCompress<T>::value, Status>::type
  callDrc(const Input& i, Output& o, Context& c) { return T::decompressReduceCompress(i, o, c); }
  template <typename T = C> static typename std::enable_if<!detail::HasDecompressReduceCompress<T>::value, Status>::type
  callDrc(const Input&, Output&, Context&) { return ncclInvalidUsage; }
};

}  // namespace coccl

#if defined(__GNUC__)
#define COCCL_PLUGIN_EXPORT __attribute__((visibility("default")))
#else
#define COCCL_PLUGIN_EXPORT
#endif

#define COCCL_REGISTER_COMPRESSOR(pluginName, CompressorType)                                  \
  extern "C" COCCL_PLUGIN_EXPORT const cocclCompressorPlugin* cocclGetCompressorPlugin() {     \
    return ::coccl::PluginAdapter<CompressorType>::descriptor(pluginName);                     \
  }

#endif  // COCCL_COMPRESSOR_PLUGIN_SDK_H_
