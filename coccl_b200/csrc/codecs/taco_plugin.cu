// libtaco.so: TACO-style adaptive FP8 codec as a compressor plugin.
//
// Options (reference: taco/taco.cu:16-33,347-362): fp8Format E4M3|E5M2 (E4M3), saturate (true),
// groupSize 32|64|128|256|512 (128), targetRange (448), lambda (1e-6), fp8MaxValue (0 => 448 / 57344).
// Numerics per group of G values (taco/taco.cu:118-218):
//   ada  = clamp(fp8max * rsqrt(mean(x^2) + lambda), 1e-3, 1e3)
//   y    = H_G(x * ada) / sqrt(G)            (Walsh-Hadamard over the whole group)
//   qs   = clamp(max|y| / targetRange, 1e-12, 1e6)
//   code = fp8(clamp(y / qs, -448, 448))     (the clamp is +-448 for both formats, as in the reference)
//   x^   = H_G(code * qs) / sqrt(G) / ada
// Encoded chunk: [fp8 bytes of whole groups: the transform spreads a partial last group over all of its
// coefficients][groups x f32 qs][groups x f32 ada]; 1024 fp32 values in
// 4 chunks at G = 128 take 1088 bytes (tests/coccl-tests/src/coccl_fixed_compressor_test.cc:143-144).
//
// Kernel shape: a thread owns one aligned run of 32 values (coalesced tile I/O through swizzled shared memory,
// kernels/tile_io.cuh); the first five Hadamard stages are register butterflies, the remaining log2(G/32)
// stages and the group statistics are warp shuffles over the G/32 lanes of the group.
#include "compressor_plugin/coccl_compressor_plugin.h"
#include "kernels/kernels_api.h"
#include "kernels/tile_io.cuh"
#include <cuda_fp8.h>

namespace {
using coccl::Status;
using namespace coccl;

struct TacoConfig {
  int e5m2 = 0;
  bool saturate = true;
  int groupSize = 128;
  float targetRange = 448.f;
  float lambda = 1e-6f;
  float fp8MaxValue = 0.f;
};

struct TacoArgs {
  const void* in;
  void* out;
  long count, chunks, rawPitch, encStride;
  int group, e5m2, saturate;
  float targetRange, lambda, fp8max;
};

struct TacoLayout { long groups, payloadBytes, totalBytes; };
__host__ __device__ inline TacoLayout tacoLayout(long count, int group) {
  TacoLayout L;
  L.groups = (count + group - 1) / group;
  L.payloadBytes = L.groups * group;
  L.totalBytes = L.payloadBytes + L.groups * 8;
  return L;
}

__device__ __forceinline__ void hadamardRun(float (&v)[32]) {
#pragma unroll
  for (int s = 1; s < 32; s <<= 1)
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if ((i & s) == 0) { const float a = v[i], b = v[i | s]; v[i] = a + b; v[i | s] = a - b; }
}
// stages 32, 64, ... of the group transform: partners are lanes of the same group
__device__ __forceinline__ void hadamardLanes(float (&v)[32], int lpg) {
  const int lane = threadIdx.x & 31;
  for (int s = 1; s < lpg; s <<= 1) {
    const bool upper = (lane & s) != 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], s);
      v[i] = upper ? o - v[i] : v[i] + o;
    }
  }
}
__device__ __forceinline__ float laneSum(float x, int lpg) {
  for (int o = 1; o < lpg; o <<= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float laneMax(float x, int lpg) {
  for (int o = 1; o < lpg; o <<= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

template <typename T>
__global__ void __launch_bounds__(kTileThreads) tacoEncodeKernel(const TacoArgs a) {
  __shared__ TileStage<T> stage;
  const TacoLayout L = tacoLayout(a.count, a.group);
  const long tiles = (a.count + kTileElems - 1) / kTileElems;
  const int lpg = a.group >> 5;
  const float rsG = rsqrtf((float)a.group);
  const __nv_fp8_interpretation_t fmt = a.e5m2 ? __NV_E5M2 : __NV_E4M3;
  const __nv_saturation_t sat = a.saturate ? __NV_SATFINITE : __NV_NOSAT;
  for (long it = blockIdx.x; it < tiles * a.chunks; it += gridDim.x) {
    const long ch = it / tiles, t = it % tiles;
    const T* src = reinterpret_cast<const T*>(a.in) + ch * a.rawPitch;
    uint8_t* dst = reinterpret_cast<uint8_t*>(a.out) + ch * a.encStride;
    const long e0 = t * kTileElems, e = e0 + (long)threadIdx.x * 32;
    float v[32];
    TileIO<T>::load(src, a.count, e0, TileIO<T>::fastTile(src, a.count, e0), stage, v);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) ss = fmaf(v[i], v[i], ss);
    ss = laneSum(ss, lpg);
    const float ada = fminf(fmaxf(a.fp8max * rsqrtf(ss / (float)a.group + a.lambda), 1e-3f), 1e3f);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= ada;
    hadamardRun(v);
    hadamardLanes(v, lpg);
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) { v[i] *= rsG; m = fmaxf(m, fabsf(v[i])); }
    m = laneMax(m, lpg);
    const float qs = fminf(fmaxf(m / a.targetRange, 1e-12f), 1e6f);
    const float inv = 1.f / qs;
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float c[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] = fminf(fmaxf(v[4 * k + i] * inv, -448.f), 448.f);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(c[0], c[1]), sat, fmt);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c[2], c[3]), sat, fmt);
      w[k] = lo | (hi << 16);
    }
    if (e < L.payloadBytes) {  // runs of the padded last group included
      uint8_t* pw = dst + e;
      if (aligned16(pw)) {
        reinterpret_cast<uint4*>(pw)[0] = make_uint4(w[0], w[1], w[2], w[3]);
        reinterpret_cast<uint4*>(pw)[1] = make_uint4(w[4], w[5], w[6], w[7]);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) reinterpret_cast<uint32_t*>(pw)[k] = w[k];
      }
      if ((e & (a.group - 1)) == 0) {
        float* ps = reinterpret_cast<float*>(dst + L.payloadBytes);
        ps[e / a.group] = qs;
        ps[L.groups + e / a.group] = ada;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kTileThreads) tacoDecodeKernel(const TacoArgs a) {
  __shared__ TileStage<T> stage;
  const TacoLayout L = tacoLayout(a.count, a.group);
  const long tiles = (a.count + kTileElems - 1) / kTileElems;
  const int lpg = a.group >> 5;
  const float rsG = rsqrtf((float)a.group);
  const __nv_fp8_interpretation_t fmt = a.e5m2 ? __NV_E5M2 : __NV_E4M3;
  for (long it = blockIdx.x; it < tiles * a.chunks; it += gridDim.x) {
    const long ch = it / tiles, t = it % tiles;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.in) + ch * a.encStride;
    T* dst = reinterpret_cast<T*>(a.out) + ch * a.rawPitch;
    const long e0 = t * kTileElems, e = e0 + (long)threadIdx.x * 32;
    float v[32];
    float qs = 0.f, ada = 1.f;
    uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (e < L.payloadBytes) {
      const uint8_t* pw = src + e;
      if (aligned16(pw)) {
        const uint4 x0 = __ldg(reinterpret_cast<const uint4*>(pw)), x1 = __ldg(reinterpret_cast<const uint4*>(pw) + 1);
        w[0] = x0.x; w[1] = x0.y; w[2] = x0.z; w[3] = x0.w; w[4] = x1.x; w[5] = x1.y; w[6] = x1.z; w[7] = x1.w;
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) w[k] = __ldg(reinterpret_cast<const uint32_t*>(pw) + k);
      }
      const float* ps = reinterpret_cast<const float*>(src + L.payloadBytes);
      qs = ps[e / a.group];
      ada = ps[L.groups + e / a.group];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[k] >> (16 * h)), fmt);
        const float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
        v[4 * k + 2 * h] = f.x * qs;
        v[4 * k + 2 * h + 1] = f.y * qs;
      }
    }
    hadamardRun(v);
    hadamardLanes(v, lpg);
    const float post = rsG / ada;
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= post;
    TileIO<T>::store(dst, a.count, e0, TileIO<T>::fastTile(dst, a.count, e0), stage, v);
  }
}

int gridFor(long items) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const long cap = (long)sms * 4;
  return (int)(items < cap ? (items > 0 ? items : 1) : cap);
}

struct Taco {
  using Config = TacoConfig;

  static Status configure(coccl::ConfigReader& r, Config& c, const coccl::ConfigContext&) {
    static const coccl::EnumEntry<int> formats[] = {{"E4M3", 0}, {"E5M2", 1}};
    r.getEnum("fp8Format", c.e5m2, formats).get("saturate", c.saturate).get("groupSize", c.groupSize)
        .get("targetRange", c.targetRange).get("lambda", c.lambda).get("fp8MaxValue", c.fp8MaxValue);
    if (!r.ok()) return ncclInvalidArgument;
    if (c.groupSize != 32 && c.groupSize != 64 && c.groupSize != 128 && c.groupSize != 256 && c.groupSize != 512) {
      r.fail("groupSize", "must be 32, 64, 128, 256 or 512");
      return ncclInvalidArgument;
    }
    if (!(c.targetRange > 0.f) || c.lambda < 0.f || c.fp8MaxValue < 0.f) { r.fail("targetRange", "must be positive"); return ncclInvalidArgument; }
    return ncclSuccess;
  }

  static bool supported(ncclDataType_t t) { return t == ncclFloat32 || t == ncclBfloat16; }  // taco/taco.cu:377-378

  static Status encodedSizeBound(const coccl::Shape& s, size_t* bytes, const coccl::SizeContext& ctx) {
    if (s.chunks() == 0 || s.elements() % s.chunks() != 0 || !supported(s.datatype())) return ncclInvalidUsage;
    const Config& c = ctx.config<Config>();
    *bytes = (size_t)tacoLayout((long)s.elementsPerChunk(), c.groupSize).totalBytes * s.chunks();
    return ncclSuccess;
  }

  static TacoArgs args(const Config& c, const void* in, void* out, long count, long chunks) {
    TacoArgs a{};
    a.in = in; a.out = out; a.count = count; a.chunks = chunks; a.rawPitch = count;
    a.encStride = tacoLayout(count, c.groupSize).totalBytes;
    a.group = c.groupSize; a.e5m2 = c.e5m2; a.saturate = c.saturate ? 1 : 0;
    a.targetRange = c.targetRange; a.lambda = c.lambda;
    a.fp8max = c.fp8MaxValue > 0.f ? c.fp8MaxValue : (c.e5m2 ? 57344.f : 448.f);
    return a;
  }

  static Status compress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    const Config& c = ctx.config<Config>();
    if (!supported(in.datatype()) || in.chunks() == 0 || in.elements() % in.chunks() != 0) return ncclInvalidArgument;
    const long count = (long)in.elementsPerChunk();
    TacoArgs a = args(c, in.data(), out.data(), count, (long)in.chunks());
    const size_t total = (size_t)a.encStride * in.chunks();
    if (coccl::shouldPassthrough(in, total)) return out.passthrough(in, ctx.stream());
    if (total > out.capacityBytes()) return ncclInvalidArgument;
    const long tiles = (count + kTileElems - 1) / kTileElems;
    const int grid = gridFor(tiles * a.chunks);
    if (in.datatype() == ncclFloat32) tacoEncodeKernel<float><<<grid, kTileThreads, 0, ctx.stream()>>>(a);
    else tacoEncodeKernel<__nv_bfloat16><<<grid, kTileThreads, 0, ctx.stream()>>>(a);
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
    const Config& c = ctx.config<Config>();
    if (!supported(out.datatype()) || out.chunks() == 0 || out.elements() % out.chunks() != 0 || in.chunks() != out.chunks())
      return ncclInvalidArgument;
    const long count = (long)(out.elements() / out.chunks());
    TacoArgs a = args(c, in.data(), out.data(), count, (long)out.chunks());
    if ((size_t)a.encStride * out.chunks() > in.bytes()) return ncclInvalidArgument;
    const long tiles = (count + kTileElems - 1) / kTileElems;
    const int grid = gridFor(tiles * a.chunks);
    if (out.datatype() == ncclFloat32) tacoDecodeKernel<float><<<grid, kTileThreads, 0, ctx.stream()>>>(a);
    else tacoDecodeKernel<__nv_bfloat16><<<grid, kTileThreads, 0, ctx.stream()>>>(a);
    if (cudaGetLastError() != cudaSuccess) return ncclUnhandledCudaError;
    return out.commitPlanned();
  }

  static cocclkCodec tileCodec(const Config& c) {
    cocclkCodec k = {};
    k.kind = 3; k.bits = 8; k.group = c.groupSize; k.paramBytes = 8;
    k.aux = (c.e5m2 ? 1 : 0) | (c.saturate ? 2 : 0);
    k.f0 = c.targetRange; k.f1 = c.lambda;
    k.f2 = c.fp8MaxValue > 0.f ? c.fp8MaxValue : (c.e5m2 ? 57344.f : 448.f);
    return k;
  }

  // Fused reductions (the reference's TACO offers compress / decompress only, taco/taco.cu:297-345, and leaves
  // reductions to the runtime's decompress-to-scratch + reduce). Copies from different ranks carry different
  // adaptive scales, but code * qs / ada is H_G(x) / sqrt(G) for every one of them, so they add up before the
  // inverse transform (kernels/codecs.cuh TacoCodec).
  static Status decompressReduce(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    const size_t reduce = ctx.reduceChunks();
    if (coccl::isPassthrough(in)) return ncclInvalidUsage;
    if (!supported(out.datatype()) || out.chunks() == 0 || out.elements() % out.chunks() != 0 || reduce == 0 ||
        in.chunks() != out.chunks() * reduce)
      return ncclInvalidArgument;
    const Config& c = ctx.config<Config>();
    const long count = (long)(out.elements() / out.chunks());
    const long stride = tacoLayout(count, c.groupSize).totalBytes;
    if ((size_t)stride * in.chunks() > in.bytes()) return ncclInvalidArgument;
    cocclkCodec k = tileCodec(c);
    const int rc = cocclkDecodeReduce(in.data(), out.data(), count, (long)out.chunks(), (long)reduce, count, stride,
                                      out.datatype() == ncclFloat32 ? 0 : 2, &k, ctx.stream());
    if (rc != 0) return rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError;
    return out.commitPlanned();
  }

  static Status decompressReduceCompress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    const size_t reduce = ctx.reduceChunks();
    if (coccl::isPassthrough(in)) return ncclInvalidUsage;
    if (reduce == 0 || in.chunks() % reduce != 0 || !supported(ctx.originalDatatype())) return ncclInvalidArgument;
    const Config& c = ctx.config<Config>();
    const size_t outChunks = in.chunks() / reduce;
    const long count = (long)(ctx.originalElements() / outChunks);
    const long stride = tacoLayout(count, c.groupSize).totalBytes;
    if ((size_t)stride * in.chunks() > in.bytes() || (size_t)stride * outChunks > out.capacityBytes()) return ncclInvalidArgument;
    cocclkCodec k = tileCodec(c);
    const int rc = cocclkDecodeReduceEncode(in.data(), out.data(), count, (long)outChunks, (long)reduce, stride, stride, &k, ctx.stream());
    if (rc != 0) return rc < 0 ? ncclInvalidArgument : ncclUnhandledCudaError;
    return out.commitBytes((size_t)stride * outChunks, outChunks);
  }
};
}  // namespace

COCCL_REGISTER_COMPRESSOR("taco", Taco)

// The library's fused collectives carry this codec as a tile codec (kernels/codecs.cuh TacoCodec, same numerics and
// chunk layout): report the configuration so that the executor can take the one-kernel path.
extern "C" COCCL_PLUGIN_EXPORT int cocclFusedCodecQuery(const void* config, int ncclDatatype, void* out) {
  if (config == nullptr || out == nullptr || !Taco::supported((ncclDataType_t)ncclDatatype)) return 0;
  *static_cast<cocclkCodec*>(out) = Taco::tileCodec(*static_cast<const TacoConfig*>(config));
  return 1;
}
