// libfp8block.so: block-scaled FP8 (MX-FP8) as a compressor plugin: E4M3 payload, one UE8M0
// power-of-two scale per 32 elements. The reference ships no such codec (TACO, taco/taco.cu,
// is its only FP8 codec); the option set is therefore this implementation's own:
//   blockSize (32, the only supported value), format "E4M3" (the only supported value).
// Fixed-size codec with fused decode-reduce and decode-reduce-encode.
#include "compressor_plugin/coccl_compressor_plugin.h"
#include "kernels/kernels_api.h"

namespace {
using coccl::Status;

struct Fp8Config {
  int blockSize = 32;
  std::string format = "E4M3";
};

int dtypeCode(ncclDataType_t t) { return t == ncclFloat32 ? 0 : t == ncclFloat16 ? 1 : t == ncclBfloat16 ? 2 : -1; }
cocclkCodec codec() { return cocclkCodec{1, 8, 32, 0, 0, 0, 1, 0, 0, 0.f, 0.f, 0.f}; }
Status rcToStatus(int rc) { return rc == 0 ? ncclSuccess : (rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError); }

struct Fp8Block {
  using Config = Fp8Config;

  static Status configure(coccl::ConfigReader& r, Config& c, const coccl::ConfigContext&) {
    r.get("blockSize", c.blockSize).get("format", c.format);
    if (!r.ok()) return ncclInvalidArgument;
    if (c.blockSize != 32) { r.fail("blockSize", "must be 32"); return ncclInvalidArgument; }
    if (c.format != "E4M3") { r.fail("format", "must be E4M3"); return ncclInvalidArgument; }
    return ncclSuccess;
  }

  static Status encodedSizeBound(const coccl::Shape& s, size_t* bytes, const coccl::SizeContext&) {
    if (s.chunks() == 0 || s.elements() % s.chunks() != 0 || dtypeCode(s.datatype()) < 0) return ncclInvalidUsage;
    cocclkCodec k = codec();
    *bytes = (size_t)cocclkEncodedChunkBytes(&k, (long)s.elementsPerChunk()) * s.chunks();
    return ncclSuccess;
  }

  static Status compress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    const int dt = dtypeCode(in.datatype());
    if (dt < 0 || in.chunks() == 0 || in.elements() % in.chunks() != 0) return ncclInvalidArgument;
    cocclkCodec k = codec();
    const long count = (long)in.elementsPerChunk();
    const long stride = cocclkEncodedChunkBytes(&k, count);
    const size_t total = (size_t)stride * in.chunks();
    if (coccl::shouldPassthrough(in, total)) return out.passthrough(in, ctx.stream());
    if (total > out.capacityBytes()) return ncclInvalidArgument;
    Status s = rcToStatus(cocclkEncode(in.data(), out.data(), count, (long)in.chunks(), count, stride, dt, &k, ctx.stream()));
    return s == ncclSuccess ? out.commitBytes(total, in.chunks()) : s;
  }

  static Status decode(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx, size_t reduce) {
    const int dt = dtypeCode(out.datatype());
    if (dt < 0 || out.chunks() == 0 || out.elements() % out.chunks() != 0 || in.chunks() != out.chunks() * reduce)
      return ncclInvalidArgument;
    cocclkCodec k = codec();
    const long count = (long)(out.elements() / out.chunks());
    const long stride = cocclkEncodedChunkBytes(&k, count);
    if ((size_t)stride * in.chunks() > in.bytes()) return ncclInvalidArgument;
    return rcToStatus(cocclkDecodeReduce(in.data(), out.data(), count, (long)out.chunks(), (long)reduce, count, stride, dt, &k, ctx.stream()));
  }

  static Status decompress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    if (coccl::isPassthrough(in)) {
      if (in.bytes() != out.elements() * coccl::dataTypeSize(out.datatype())) return ncclInvalidArgument;
      if (in.data() != out.data() &&
          cudaMemcpyAsync(out.data(), in.data(), in.bytes(), cudaMemcpyDeviceToDevice, ctx.stream()) != cudaSuccess)
        return ncclUnhandledCudaError;
      return out.commitPlanned();
    }
    Status s = decode(in, out, ctx, 1);
    return s == ncclSuccess ? out.commitPlanned() : s;
  }

  static Status decompressReduce(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    if (coccl::isPassthrough(in)) return ncclInvalidUsage;
    Status s = decode(in, out, ctx, ctx.reduceChunks());
    return s == ncclSuccess ? out.commitPlanned() : s;
  }

  static Status decompressReduceCompress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    const size_t reduce = ctx.reduceChunks();
    if (coccl::isPassthrough(in) || reduce == 0 || in.chunks() % reduce != 0) return ncclInvalidArgument;
    const size_t outChunks = in.chunks() / reduce;
    cocclkCodec k = codec();
    const long count = (long)(ctx.originalElements() / outChunks);
    const long stride = cocclkEncodedChunkBytes(&k, count);
    if ((size_t)stride * outChunks > out.capacityBytes()) return ncclInvalidArgument;
    Status s = rcToStatus(cocclkDecodeReduceEncode(in.data(), out.data(), count, (long)outChunks, (long)reduce, stride, stride, &k, ctx.stream()));
    return s == ncclSuccess ? out.commitBytes((size_t)stride * outChunks, outChunks) : s;
  }
};
}  // namespace

COCCL_REGISTER_COMPRESSOR("fp8block", Fp8Block)

extern "C" COCCL_PLUGIN_EXPORT int cocclFusedCodecQuery(const void* config, int ncclDatatype, void* out) {
  if (config == nullptr || out == nullptr || dtypeCode((ncclDataType_t)ncclDatatype) < 0) return 0;
  *static_cast<cocclkCodec*>(out) = codec();
  return 1;
}
