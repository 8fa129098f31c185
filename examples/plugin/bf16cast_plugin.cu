// libbf16cast.so: a complete third-party compressor plugin in one file, as a starting point for a new codec.
//
// The codec sends fp32 data as bf16 (2 : 1). It shows every piece a fixed-size codec needs:
//   * a Config struct filled from the [<policy>.config] table of the policy file (`rounding`),
//   * encodedSizeBound(): how many bytes a message of a given shape needs (and which datatypes are taken at all:
//     anything the codec refuses with ncclInvalidUsage is sent uncompressed by the router),
//   * compress() / decompress() on the stream the runtime hands over,
//   * decompressReduce(): optional; sums several encoded copies while decoding, which saves the runtime a separate
//     reduction pass (reduce-scatter and all-reduce call it).
// Nothing else is required: chunking, slicing, workspace, transport, the choice of algorithm and the fallback to
// the native library are the runtime's job. Build and try it with examples/plugin/build.sh.
#include <cuda_bf16.h>

#include <string>

#include "compressor_plugin/coccl_compressor_plugin.h"

namespace {
using coccl::Status;

struct CastConfig {
  std::string rounding = "nearest";   // "nearest" (round to nearest even) or "truncate"
};

// A message is `chunks` equal chunks (one per destination rank for a scattered operation); chunk c of the encoded
// form starts at c * elementsPerChunk * 2 bytes, so any chunk can be sent or decoded on its own.
__global__ void encodeKernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n, bool truncate) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = in[i];
    out[i] = truncate ? __ushort_as_bfloat16((unsigned short)(__float_as_uint(v) >> 16)) : __float2bfloat16_rn(v);
  }
}

// Copy r of output chunk c is input chunk r * outChunks + c (reduce == 1: a plain decode).
__global__ void decodeSumKernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, size_t perChunk,
                                size_t outChunks, size_t reduce) {
  const size_t n = perChunk * outChunks;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (size_t r = 0; r < reduce; ++r) acc += __bfloat162float(in[r * n + i]);
    out[i] = acc;
  }
}

unsigned gridFor(size_t n) {
  const size_t blocks = (n + 255) / 256;
  return (unsigned)(blocks < 1 ? 1 : (blocks > 4096 ? 4096 : blocks));
}

struct Bf16Cast {
  using Config = CastConfig;

  static Status configure(coccl::ConfigReader& r, Config& c, const coccl::ConfigContext&) {
    r.get("rounding", c.rounding);
    if (!r.ok()) return ncclInvalidArgument;   // unknown keys and wrong types are reported by the reader
    if (c.rounding != "nearest" && c.rounding != "truncate") {
      r.fail("rounding", "must be \"nearest\" or \"truncate\"");
      return ncclInvalidArgument;
    }
    return ncclSuccess;
  }

  static Status encodedSizeBound(const coccl::Shape& s, size_t* bytes, const coccl::SizeContext&) {
    if (s.datatype() != ncclFloat32 || s.chunks() == 0 || s.elements() % s.chunks() != 0) return ncclInvalidUsage;
    *bytes = s.elements() * sizeof(__nv_bfloat16);
    return ncclSuccess;
  }

  static Status compress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    if (in.datatype() != ncclFloat32 || in.chunks() == 0 || in.elements() % in.chunks() != 0) return ncclInvalidArgument;
    const size_t bytes = in.elements() * sizeof(__nv_bfloat16);
    if (bytes > out.capacityBytes()) return ncclInvalidArgument;
    const bool truncate = ctx.config<Config>().rounding == "truncate";
    encodeKernel<<<gridFor(in.elements()), 256, 0, ctx.stream()>>>(in.dataAs<float>(), out.dataAs<__nv_bfloat16>(),
                                                                  in.elements(), truncate);
    const Status s = coccl::fromCuda(cudaGetLastError());
    return s == ncclSuccess ? out.commitBytes(bytes, in.chunks()) : s;
  }

  static Status decode(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx, size_t reduce) {
    if (out.datatype() != ncclFloat32 || out.chunks() == 0 || out.elements() % out.chunks() != 0 || reduce == 0 ||
        in.chunks() != out.chunks() * reduce || in.bytes() < out.elements() * reduce * sizeof(__nv_bfloat16))
      return ncclInvalidArgument;
    decodeSumKernel<<<gridFor(out.elements()), 256, 0, ctx.stream()>>>(in.dataAs<__nv_bfloat16>(), out.dataAs<float>(),
                                                                      out.elements() / out.chunks(), out.chunks(), reduce);
    const Status s = coccl::fromCuda(cudaGetLastError());
    return s == ncclSuccess ? out.commitPlanned() : s;
  }

  static Status decompress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) { return decode(in, out, ctx, 1); }

  static Status decompressReduce(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    return decode(in, out, ctx, ctx.reduceChunks());
  }
};
}  // namespace

COCCL_REGISTER_COMPRESSOR("bf16cast", Bf16Cast)
