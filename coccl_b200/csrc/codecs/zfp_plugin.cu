// libzfp.so: ZFP fixed-rate compression of 1-D blocks of four values as a compressor plugin.
//
// Option (reference: zfp/coccl_interface/zfp_plugin.cc:13-15,57-60): rate = bits per value, here 1..32 (4);
// every block of four values takes maxbits = max(4 * rate, 9) bits (zfp/src/zfp.c:773-803). fp16 / bf16
// inputs are widened to fp32 inside the kernel, as the reference does (zfp/src/cuda_zfp/encode1.cuh:17-51).
// Stream: per chunk, block i at bit i * maxbits of a little-endian word stream, chunk size rounded up to 8
// bytes (cuda_zfp/encode.cuh:224-231). The block coder is the shared host/device code of oracle/zfp1d.h.
//
// Kernel shape: one thread codes one block in registers/local words; a warp's 32 blocks occupy exactly
// `maxbits` consecutive 32-bit words, which the warp assembles in shared memory (shared-memory ORs, no global
// atomics) and writes with coalesced stores. The decoder stages the same words and lets every lane cut out
// its block.
#include "compressor_plugin/coccl_compressor_plugin.h"
#include "kernels/common.cuh"
#include "kernels/kernels_api.h"
#include "oracle/zfp1d.h"

namespace {
using coccl::Status;
using namespace coccl;
using namespace coccl::zfp1d;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxRate = 32;
constexpr int kMaxRegionWords = 4 * kMaxRate;  // words of 32 blocks at the largest rate

struct ZfpConfig { int rate = 4; };

struct ZfpArgs {
  const void* in;
  void* out;
  long count, chunks, rawPitch, encStride;
  int maxbits;
};

__host__ __device__ inline long zfpChunkBytes(long count, int maxbits) {
  const long blocks = (count + 3) / 4;
  return (blocks * maxbits + 63) / 64 * 8;
}

template <typename T> __device__ __forceinline__ float toF(T x);
template <> __device__ __forceinline__ float toF<float>(float x) { return x; }
template <> __device__ __forceinline__ float toF<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float toF<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T fromF(float x);
template <> __device__ __forceinline__ float fromF<float>(float x) { return x; }
template <> __device__ __forceinline__ __half fromF<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 fromF<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <typename T>
__global__ void __launch_bounds__(kThreads) zfpEncodeKernel(const ZfpArgs a) {
  __shared__ uint32_t region[kWarps][kMaxRegionWords];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long blocks = (a.count + 3) / 4;
  const long warpItems = (blocks + 31) / 32;  // groups of 32 blocks per chunk
  const long chunkWords = a.encStride / 4;
  for (long it = (long)blockIdx.x * kWarps + warp; it < warpItems * a.chunks; it += (long)gridDim.x * kWarps) {
    const long ch = it / warpItems, g = it % warpItems;
    const T* src = reinterpret_cast<const T*>(a.in) + ch * a.rawPitch;
    uint32_t* dst = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(a.out) + ch * a.encStride);
    for (int i = lane; i < a.maxbits; i += 32) region[warp][i] = 0;
    __syncwarp();
    const long b = g * 32 + lane;
    if (b < blocks) {
      float x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = (4 * b + i < a.count) ? toF<T>(src[4 * b + i]) : 0.f;
      BitWindow s;
#pragma unroll
      for (int i = 0; i < kMaxWords; ++i) s.w[i] = 0;
      const int bit0 = lane * a.maxbits;
      s.pos = bit0 & 31;
      encodeBlock(x, a.maxbits, s);
      const int words = ((bit0 & 31) + a.maxbits + 31) >> 5;
      for (int i = 0; i < words; ++i)
        if (s.w[i]) atomicOr(&region[warp][(bit0 >> 5) + i], s.w[i]);
    }
    __syncwarp();
    const long w0 = g * a.maxbits;  // 32 blocks * maxbits bits = maxbits words
    for (int i = lane; i < a.maxbits && w0 + i < chunkWords; i += 32) dst[w0 + i] = region[warp][i];
    __syncwarp();
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) zfpDecodeKernel(const ZfpArgs a) {
  __shared__ uint32_t region[kWarps][kMaxRegionWords + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long blocks = (a.count + 3) / 4;
  const long warpItems = (blocks + 31) / 32;
  const long chunkWords = a.encStride / 4;
  for (long it = (long)blockIdx.x * kWarps + warp; it < warpItems * a.chunks; it += (long)gridDim.x * kWarps) {
    const long ch = it / warpItems, g = it % warpItems;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(a.in) + ch * a.encStride);
    T* dst = reinterpret_cast<T*>(a.out) + ch * a.rawPitch;
    const long w0 = g * a.maxbits;
    for (int i = lane; i <= a.maxbits; i += 32) region[warp][i] = (i < a.maxbits && w0 + i < chunkWords) ? __ldg(src + w0 + i) : 0u;
    __syncwarp();
    const long b = g * 32 + lane;
    if (b < blocks) {
      BitWindow s;
      const int bit0 = lane * a.maxbits;
      const int words = ((bit0 & 31) + a.maxbits + 31) >> 5;
#pragma unroll
      for (int i = 0; i < kMaxWords; ++i) s.w[i] = i < words ? region[warp][(bit0 >> 5) + i] : 0u;
      s.pos = bit0 & 31;
      float x[4];
      decodeBlock(s, a.maxbits, x);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (4 * b + i < a.count) dst[4 * b + i] = fromF<T>(x[i]);
    }
    __syncwarp();
  }
}

int gridFor(long warpItems) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const long ctas = (warpItems + kWarps - 1) / kWarps, cap = (long)sms * 8;
  return (int)(ctas < cap ? (ctas > 0 ? ctas : 1) : cap);
}

template <class F>
bool dispatch(ncclDataType_t t, F&& f) {
  if (t == ncclFloat32) { f(float{}); return true; }
  if (t == ncclFloat16) { f(__half{}); return true; }
  if (t == ncclBfloat16) { f(__nv_bfloat16{}); return true; }
  return false;
}

// Rates whose blocks fit a 64-bit register run on the library's tile kernels (kernels/codecs.cuh ZfpCodec): a
// thread codes eight blocks and writes whole words of the same stream. They also give this codec a fused
// decompress-reduce. Other rates use the generic kernels above.
inline bool tileRate(int rate) { return rate == 4 || rate == 8 || rate == 16; }
inline cocclkCodec tileCodec(int rate) {
  cocclkCodec k = {};
  k.kind = 4; k.bits = rate; k.group = 4; k.paramBytes = 0;
  return k;
}
inline int tileDtype(ncclDataType_t t) { return t == ncclFloat32 ? 0 : t == ncclFloat16 ? 1 : t == ncclBfloat16 ? 2 : -1; }

struct Zfp {
  using Config = ZfpConfig;

  static Status configure(coccl::ConfigReader& r, Config& c, const coccl::ConfigContext&) {
    r.get("rate", c.rate, 1, kMaxRate);
    return r.ok() ? ncclSuccess : ncclInvalidArgument;
  }
  static bool supported(ncclDataType_t t) { return t == ncclFloat32 || t == ncclFloat16 || t == ncclBfloat16; }

  static Status encodedSizeBound(const coccl::Shape& s, size_t* bytes, const coccl::SizeContext& ctx) {
    if (s.chunks() == 0 || s.elements() % s.chunks() != 0 || !supported(s.datatype())) return ncclInvalidUsage;
    *bytes = (size_t)zfpChunkBytes((long)s.elementsPerChunk(), maxBits(ctx.config<Config>().rate)) * s.chunks();
    return ncclSuccess;
  }

  static Status compress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    if (!supported(in.datatype()) || in.chunks() == 0 || in.elements() % in.chunks() != 0) return ncclInvalidArgument;
    ZfpArgs a{};
    a.in = in.data(); a.out = out.data(); a.count = (long)in.elementsPerChunk(); a.chunks = (long)in.chunks();
    a.rawPitch = a.count; a.maxbits = maxBits(ctx.config<Config>().rate);
    a.encStride = zfpChunkBytes(a.count, a.maxbits);
    const size_t total = (size_t)a.encStride * in.chunks();
    // a stream as large as the input gains nothing: pass the bytes through (the reference reaches the same through
    // the header slack in its size bound, zfp_plugin.cc:121-137)
    if (coccl::shouldPassthrough(in, total) || total == in.bytes()) return out.passthrough(in, ctx.stream());
    if (total > out.capacityBytes()) return ncclInvalidArgument;
    const int rate = ctx.config<Config>().rate;
    if (tileRate(rate)) {
      cocclkCodec k = tileCodec(rate);
      const int rc = cocclkEncode(in.data(), out.data(), a.count, a.chunks, a.count, a.encStride, tileDtype(in.datatype()), &k, ctx.stream());
      if (rc != 0) return rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError;
      return out.commitBytes(total, in.chunks());
    }
    const long items = ((a.count + 3) / 4 + 31) / 32 * a.chunks;
    dispatch(in.datatype(), [&](auto t) {
      using T = decltype(t);
      zfpEncodeKernel<T><<<gridFor(items), kThreads, 0, ctx.stream()>>>(a);
    });
    if (cudaGetLastError() != cudaSuccess) return ncclUnhandledCudaError;
    return out.commitBytes(total, in.chunks());
  }

  static Status decompress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    if (coccl::isPassthrough(in)) {
      if (in.bytes() != out.elements() * coccl::dataTypeSize(out.datatype())) return ncclInvalidArgument;
      if (in.data() != out.data() &&
          cudaMemcpyAsync(out.data(), in.data(), in.bytes(), cudaMemcpyDeviceToDevice, ctx.stream()) != cudaSuccess)
        return ncclUnhandledCudaError;
      return out.commitPlanned();
    }
    if (!supported(out.datatype()) || out.chunks() == 0 || out.elements() % out.chunks() != 0 || in.chunks() != out.chunks())
      return ncclInvalidArgument;
    ZfpArgs a{};
    a.in = in.data(); a.out = out.data(); a.count = (long)(out.elements() / out.chunks()); a.chunks = (long)out.chunks();
    a.rawPitch = a.count; a.maxbits = maxBits(ctx.config<Config>().rate);
    a.encStride = zfpChunkBytes(a.count, a.maxbits);
    if ((size_t)a.encStride * out.chunks() > in.bytes()) return ncclInvalidArgument;
    const int rate = ctx.config<Config>().rate;
    if (tileRate(rate)) {
      cocclkCodec k = tileCodec(rate);
      const int rc = cocclkDecodeReduce(in.data(), out.data(), a.count, a.chunks, 1, a.count, a.encStride, tileDtype(out.datatype()), &k, ctx.stream());
      if (rc != 0) return rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError;
      return out.commitPlanned();
    }
    const long items = ((a.count + 3) / 4 + 31) / 32 * a.chunks;
    dispatch(out.datatype(), [&](auto t) {
      using T = decltype(t);
      zfpDecodeKernel<T><<<gridFor(items), kThreads, 0, ctx.stream()>>>(a);
    });
    if (cudaGetLastError() != cudaSuccess) return ncclUnhandledCudaError;
    return out.commitPlanned();
  }

  // Sum of `reduceChunks` decoded copies per output chunk in one pass (tile rates only; other rates leave the
  // reduction to the runtime's generic decompress + reduce).
  static Status decompressReduce(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    const int rate = ctx.config<Config>().rate;
    const size_t reduce = ctx.reduceChunks();
    if (!tileRate(rate) || coccl::isPassthrough(in)) return ncclInvalidUsage;
    if (!supported(out.datatype()) || out.chunks() == 0 || out.elements() % out.chunks() != 0 || reduce == 0 ||
        in.chunks() != out.chunks() * reduce)
      return ncclInvalidArgument;
    const long count = (long)(out.elements() / out.chunks());
    const long stride = zfpChunkBytes(count, maxBits(rate));
    if ((size_t)stride * in.chunks() > in.bytes()) return ncclInvalidArgument;
    cocclkCodec k = tileCodec(rate);
    const int rc = cocclkDecodeReduce(in.data(), out.data(), count, (long)out.chunks(), (long)reduce, count, stride,
                                      tileDtype(out.datatype()), &k, ctx.stream());
    if (rc != 0) return rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError;
    return out.commitPlanned();
  }
};
}  // namespace

COCCL_REGISTER_COMPRESSOR("zfp", Zfp)

// Rates 4, 8 and 16 are tile codecs of the library's fused collectives (kernels/codecs.cuh ZfpCodec: a run of 32
// values is exactly `rate` words of the same stream); other rates stay on this plugin's kernels and the staged path.
extern "C" COCCL_PLUGIN_EXPORT int cocclFusedCodecQuery(const void* config, int ncclDatatype, void* out) {
  if (config == nullptr || out == nullptr || !Zfp::supported((ncclDataType_t)ncclDatatype)) return 0;
  const int rate = static_cast<const ZfpConfig*>(config)->rate;
  if (!tileRate(rate)) return 0;
  *static_cast<cocclkCodec*>(out) = tileCodec(rate);
  return 1;
}
