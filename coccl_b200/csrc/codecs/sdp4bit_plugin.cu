// libsdp4bit.so: SDP4Bit group quantisation as a compressor plugin.
//
// Options (defaults) follow the reference plugin
// (src/coccl-extend/extensions/compressor_plugin/sdp4bit/sdp4bit_quan.cu:14-61,229-246):
//   groupCount (2048), quantBits 4|8 (8), quantType Symmetric|Asymmetric (Symmetric),
//   hadamard (false; caps the group at 128), subAdd (false; not with hadamard),
//   pipelineSize (1; number of delta-state slots).
// Extra options of this implementation: rounding = "stochastic"|"nearest" (stochastic),
// seed (0).
//
// Families shown: fixed-size (exact encodedSizeBound), fused-reduction (decompressReduce,
// decompressReduceCompress) and stateful (subAdd keeps the previously decoded values per
// slot in persistent memory: the first round of a slot goes through raw and seeds the
// state, later rounds encode x - prev and decode prev + dq; sdp4bit_quan.cu:286-426).
// The kernels live in libcoccl.so (kernels/codec_kernels.cu).
#include "compressor_plugin/coccl_compressor_plugin.h"
#include "kernels/kernels_api.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace {

using coccl::Status;

enum class QuantType { Symmetric, Asymmetric };
enum class Rounding { Stochastic, Nearest };

struct Sdp4Config {
  int groupCount = 2048;
  int quantBits = 8;
  QuantType quantType = QuantType::Symmetric;
  bool hadamard = false;
  bool subAdd = false;
  int pipelineSize = 1;
  Rounding rounding = Rounding::Stochastic;
  uint32_t seed = 0;
};

int dtypeCode(ncclDataType_t t) {
  switch (t) {
    case ncclFloat32: return 0;
    case ncclFloat16: return 1;
    case ncclBfloat16: return 2;
    default: return -1;
  }
}

cocclkCodec toCodec(const Sdp4Config& c, ncclDataType_t dt) {
  cocclkCodec k = {};
  k.kind = 0;
  k.bits = c.quantBits;
  k.group = c.hadamard && c.groupCount > 128 ? 128 : c.groupCount;
  k.asym = c.quantType == QuantType::Asymmetric;
  k.hadamard = c.hadamard;
  k.stochastic = c.rounding == Rounding::Stochastic;
  k.paramBytes = (dt == ncclFloat32 && !k.asym) ? 4 : 8;
  k.seed = c.seed;
  return k;
}

// Per-policy host state of the delta codec.
struct SubAddState {
  static constexpr int kMaxSlots = 16;
  unsigned long long calls = 0;       // compress calls seen (selects the slot)
  unsigned long long decodes = 0;     // decompress calls seen
  bool seeded[kMaxSlots] = {};
  size_t seededBytes[kMaxSlots] = {};
};

template <typename T>
__global__ void subKernel(const T* x, const T* prev, T* out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = (T)((float)x[i] - (float)prev[i]);
}
template <typename T>
__global__ void addUpdateKernel(T* out, T* prev, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    T v = (T)((float)out[i] + (float)prev[i]);
    out[i] = v;
    prev[i] = v;
  }
}
template <typename F>
Status byType(ncclDataType_t dt, F&& f) {
  switch (dt) {
    case ncclFloat32: f(float{}); return ncclSuccess;
    case ncclFloat16: f(__half{}); return ncclSuccess;
    case ncclBfloat16: f(__nv_bfloat16{}); return ncclSuccess;
    default: return ncclInvalidArgument;
  }
}
int gridFor(size_t n) { size_t b = (n + 255) / 256; return (int)(b > 148 * 16 ? 148 * 16 : (b ? b : 1)); }

struct Sdp4Bit {
  using Config = Sdp4Config;
  static constexpr bool kSeesPassthrough = true;  // the delta state is seeded from the raw first round

  static Status configure(coccl::ConfigReader& r, Config& c, const coccl::ConfigContext&) {
    static const coccl::EnumEntry<QuantType> qt[] = {{"Symmetric", QuantType::Symmetric}, {"Asymmetric", QuantType::Asymmetric}};
    static const coccl::EnumEntry<Rounding> rd[] = {{"stochastic", Rounding::Stochastic}, {"nearest", Rounding::Nearest}};
    r.get("groupCount", c.groupCount).get("quantBits", c.quantBits).getEnum("quantType", c.quantType, qt)
        .get("hadamard", c.hadamard).get("subAdd", c.subAdd).get("pipelineSize", c.pipelineSize)
        .getEnum("rounding", c.rounding, rd).get("seed", c.seed);
    if (!r.ok()) return ncclInvalidArgument;
    if (c.quantBits != 4 && c.quantBits != 8) { r.fail("quantBits", "must be 4 or 8"); return ncclInvalidArgument; }
    if (c.groupCount <= 0 || c.groupCount % (8 / c.quantBits) != 0) { r.fail("groupCount", "must be a positive multiple of 8/quantBits"); return ncclInvalidArgument; }
    if (c.subAdd && c.hadamard) { r.fail("subAdd", "cannot be combined with hadamard"); return ncclInvalidArgument; }
    if (c.pipelineSize < 1 || c.pipelineSize > SubAddState::kMaxSlots) { r.fail("pipelineSize", "must be in [1, 16]"); return ncclInvalidArgument; }
    cocclkCodec k = toCodec(c, ncclFloat32);
    if (!cocclkTileCodecSupported(&k)) { r.fail("groupCount", "must be a power of two in [8, 2048] (>= 32 with hadamard)"); return ncclInvalidArgument; }
    return ncclSuccess;
  }

  static Status encodedSizeBound(const coccl::Shape& s, size_t* bytes, const coccl::SizeContext& sc) {
    if (s.chunks() == 0 || s.elements() % s.chunks() != 0 || dtypeCode(s.datatype()) < 0) return ncclInvalidUsage;
    cocclkCodec k = toCodec(sc.config<Config>(), s.datatype());
    *bytes = (size_t)cocclkEncodedChunkBytes(&k, (long)s.elementsPerChunk()) * s.chunks();
    // the delta codec sends its seeding round raw: reserve room for it
    if (sc.config<Config>().subAdd && *bytes < s.bytes()) *bytes = s.bytes();
    return ncclSuccess;
  }

  static Status compress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    const Config& c = ctx.config<Config>();
    const int dt = dtypeCode(in.datatype());
    if (dt < 0 || in.chunks() == 0 || in.elements() % in.chunks() != 0) return ncclInvalidArgument;
    cocclkCodec k = toCodec(c, in.datatype());
    const long count = (long)in.elementsPerChunk();
    const long stride = cocclkEncodedChunkBytes(&k, count);
    const size_t total = (size_t)stride * in.chunks();
    if (coccl::shouldPassthrough(in, total)) return out.passthrough(in, ctx.stream());
    if (total > out.capacityBytes()) return ncclInvalidArgument;
    const void* src = in.data();
    coccl::Buffer tmp;
    if (c.subAdd) {
      SubAddState* st = nullptr;
      Status s = ctx.instance(&st);
      if (s != ncclSuccess) return s;
      const int slot = (int)(st->calls++ % (unsigned long long)c.pipelineSize);
      const size_t fullBytes = in.bytes() * (size_t)ctx.ranks();
      if (!st->seeded[slot] || st->seededBytes[slot] != fullBytes) return out.passthrough(in, ctx.stream());  // seeding round
      coccl::Buffer prev;
      if ((s = ctx.persistent(slot, fullBytes, &prev)) != ncclSuccess) return s;
      if ((s = ctx.scratch(in.bytes(), &tmp)) != ncclSuccess) return s;
      const char* mine = prev.dataAs<char>() + in.bytes() * (size_t)ctx.rank();
      s = byType(in.datatype(), [&](auto t) {
        using T = decltype(t);
        subKernel<T><<<gridFor(in.elements()), 256, 0, ctx.stream()>>>(in.dataAs<T>(), (const T*)mine, tmp.dataAs<T>(), in.elements());
      });
      if (s != ncclSuccess) return s;
      src = tmp.data();
    }
    int rc = cocclkEncode(src, out.data(), count, (long)in.chunks(), count, stride, dt, &k, ctx.stream());
    if (rc != 0) return rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError;
    return out.commitBytes(total, in.chunks());
  }

  static Status decodeInto(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx, size_t reduce) {
    const Config& c = ctx.config<Config>();
    const int dt = dtypeCode(out.datatype());
    if (dt < 0 || out.chunks() == 0 || out.elements() % out.chunks() != 0 || in.chunks() != out.chunks() * reduce)
      return ncclInvalidArgument;
    cocclkCodec k = toCodec(c, out.datatype());
    const long count = (long)(out.elements() / out.chunks());
    const long stride = cocclkEncodedChunkBytes(&k, count);
    if ((size_t)stride * in.chunks() > in.bytes()) return ncclInvalidArgument;
    int rc = cocclkDecodeReduce(in.data(), out.data(), count, (long)out.chunks(), (long)reduce, count, stride, dt, &k, ctx.stream());
    return rc == 0 ? ncclSuccess : (rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError);
  }

  static Status decompress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    const Config& c = ctx.config<Config>();
    const size_t outBytes = out.elements() * coccl::dataTypeSize(out.datatype());
    SubAddState* st = nullptr;
    int slot = 0;
    if (c.subAdd) {
      Status s = ctx.instance(&st);
      if (s != ncclSuccess) return s;
      slot = (int)(st->decodes++ % (unsigned long long)c.pipelineSize);
    }
    if (coccl::isPassthrough(in)) {
      if (in.bytes() != outBytes) return ncclInvalidArgument;
      if (in.data() != out.data()) {
        cudaError_t e = cudaMemcpyAsync(out.data(), in.data(), outBytes, cudaMemcpyDeviceToDevice, ctx.stream());
        if (e != cudaSuccess) return ncclUnhandledCudaError;
      }
      if (c.subAdd) {  // seed the slot with what every rank now holds
        coccl::Buffer prev;
        Status s = ctx.persistent(slot, outBytes, &prev);
        if (s != ncclSuccess) return s;
        cudaError_t e = cudaMemcpyAsync(prev.data(), out.data(), outBytes, cudaMemcpyDeviceToDevice, ctx.stream());
        if (e != cudaSuccess) return ncclUnhandledCudaError;
        st->seeded[slot] = true;
        st->seededBytes[slot] = outBytes;
      }
      return out.commitPlanned();
    }
    Status s = decodeInto(in, out, ctx, 1);
    if (s != ncclSuccess) return s;
    if (c.subAdd) {
      if (!st->seeded[slot] || st->seededBytes[slot] != outBytes) return ncclInvalidUsage;
      coccl::Buffer prev;
      if ((s = ctx.persistent(slot, outBytes, &prev)) != ncclSuccess) return s;
      s = byType(out.datatype(), [&](auto t) {
        using T = decltype(t);
        addUpdateKernel<T><<<gridFor(out.elements()), 256, 0, ctx.stream()>>>(out.dataAs<T>(), prev.dataAs<T>(), out.elements());
      });
      if (s != ncclSuccess) return s;
    }
    return out.commitPlanned();
  }

  static Status decompressReduce(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    if (ctx.config<Config>().subAdd || coccl::isPassthrough(in)) return ncclInvalidUsage;
    Status s = decodeInto(in, out, ctx, ctx.reduceChunks());
    return s == ncclSuccess ? out.commitPlanned() : s;
  }

  static Status decompressReduceCompress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    const Config& c = ctx.config<Config>();
    if (c.subAdd || coccl::isPassthrough(in)) return ncclInvalidUsage;
    const size_t reduce = ctx.reduceChunks();
    if (reduce == 0 || in.chunks() % reduce != 0 || dtypeCode(ctx.originalDatatype()) < 0) return ncclInvalidArgument;
    const size_t outChunks = in.chunks() / reduce;
    cocclkCodec k = toCodec(c, ctx.originalDatatype());
    // originalElements = raw elements of the reduced result
    const long count = (long)(ctx.originalElements() / outChunks);
    const long stride = cocclkEncodedChunkBytes(&k, count);
    if ((size_t)stride * outChunks > out.capacityBytes()) return ncclInvalidArgument;
    int rc = cocclkDecodeReduceEncode(in.data(), out.data(), count, (long)outChunks, (long)reduce, stride, stride, &k, ctx.stream());
    if (rc != 0) return rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError;
    return out.commitBytes((size_t)stride * outChunks, outChunks);
  }
};

}  // namespace

COCCL_REGISTER_COMPRESSOR("sdp4bit", Sdp4Bit)

// Fused-collective hook: every stateless configuration maps onto the library's tile codec.
extern "C" COCCL_PLUGIN_EXPORT int cocclFusedCodecQuery(const void* config, int ncclDatatype, void* out) {
  const Sdp4Config* c = static_cast<const Sdp4Config*>(config);
  if (c == nullptr || out == nullptr || c->subAdd || dtypeCode((ncclDataType_t)ncclDatatype) < 0) return 0;
  *static_cast<cocclkCodec*>(out) = toCodec(*c, (ncclDataType_t)ncclDatatype);
  return 1;
}

// The stateful delta configuration (subAdd) maps onto the fused all-gather of deltas (kernels/collective_kernels.cuh,
// kOpAllGatherDelta): same tile codec, the output buffer is the state.
extern "C" COCCL_PLUGIN_EXPORT int cocclFusedCodecDeltaQuery(const void* config, int ncclDatatype, void* out) {
  const Sdp4Config* c = static_cast<const Sdp4Config*>(config);
  if (c == nullptr || out == nullptr || !c->subAdd || dtypeCode((ncclDataType_t)ncclDatatype) < 0) return 0;
  *static_cast<cocclkCodec*>(out) = toCodec(*c, (ncclDataType_t)ncclDatatype);
  return 1;
}
