// Launchers for the standalone codec kernels (see collective_kernels.cuh).
#include "launch_count.h"
#include "collective_kernels.cuh"
#include "kernels_api.h"
#include <type_traits>

using namespace coccl;

static_assert(sizeof(cocclkCodec) == sizeof(CodecCfg), "codec POD mismatch");

static inline CodecCfg toCfg(const cocclkCodec* c) {
  CodecCfg r;
  r.kind = c->kind; r.bits = c->bits; r.group = c->group; r.asym = c->asym; r.hadamard = c->hadamard;
  r.stochastic = c->stochastic; r.paramBytes = c->paramBytes; r.seed = c->seed;
  r.aux = c->aux; r.f0 = c->f0; r.f1 = c->f1; r.f2 = c->f2;
  return r;
}

static int smCount() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

static inline int gridFor(long items) {
  long cap = (long)smCount() * 4;
  return (int)(items < cap ? (items > 0 ? items : 1) : cap);
}

template <class F>
static bool dispatchDtype(int dtype, F&& f) {
  switch (dtype) {
    case kF32: f(float{}); return true;
    case kF16: f(__half{}); return true;
    case kBF16: f(__nv_bfloat16{}); return true;
  }
  return false;
}

extern "C" long cocclkEncodedChunkBytes(const cocclkCodec* codec, long count) {
  return makeChunkLayout(toCfg(codec), count, 4).totalBytes;
}

extern "C" int cocclkTileCodecSupported(const cocclkCodec* codec) { return tileCodecSupported(toCfg(codec)) ? 1 : 0; }

extern "C" int cocclkEncode(const void* in, void* out, long count, long chunks, long rawPitch, long encStride,
                            int dtype, const cocclkCodec* codec, cudaStream_t stream) {
  CodecArgs a{};
  a.in = in; a.out = out; a.count = count; a.chunks = chunks; a.reduce = 1; a.rawPitch = rawPitch;
  a.encStrideOut = encStride; a.dtype = dtype; a.codec = toCfg(codec);
  if (!tileCodecSupported(a.codec) || count <= 0 || chunks <= 0) return -1;
  const long tiles = (count + kTileElems - 1) / kTileElems;
  const int grid = gridFor(tiles * chunks);
  bool ok = dispatchCodec(a.codec, [&](auto codecTag) {
    using C = decltype(codecTag);
    dispatchDtype(dtype, [&](auto t) {
      using T = decltype(t);
      encodeKernel<T, C><<<grid, kTileThreads, 0, stream>>>(a);
    });
  });
  if (!ok) return -1;
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

extern "C" int cocclkDecodeReduce(const void* in, void* out, long count, long chunks, long reduce, long rawPitch,
                                  long encStride, int dtype, const cocclkCodec* codec, cudaStream_t stream) {
  CodecArgs a{};
  a.in = in; a.out = out; a.count = count; a.chunks = chunks; a.reduce = reduce; a.rawPitch = rawPitch;
  a.encStrideIn = encStride; a.dtype = dtype; a.codec = toCfg(codec);
  if (!tileCodecSupported(a.codec) || count <= 0 || chunks <= 0 || reduce <= 0) return -1;
  const long tiles = (count + kTileElems - 1) / kTileElems;
  const int grid = gridFor(tiles * chunks);
  bool ok = dispatchCodec(a.codec, [&](auto codecTag) {
    using C = decltype(codecTag);
    dispatchDtype(dtype, [&](auto t) {
      using T = decltype(t);
      decodeReduceKernel<T, C><<<grid, kTileThreads, 0, stream>>>(a);
    });
  });
  if (!ok) return -1;
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

extern "C" int cocclkDecodeReduceEncode(const void* in, void* out, long count, long chunks, long reduce,
                                        long encStrideIn, long encStrideOut, const cocclkCodec* codec,
                                        cudaStream_t stream) {
  CodecArgs a{};
  a.in = in; a.out = out; a.count = count; a.chunks = chunks; a.reduce = reduce;
  a.encStrideIn = encStrideIn; a.encStrideOut = encStrideOut; a.codec = toCfg(codec);
  if (!tileCodecSupported(a.codec) || count <= 0 || chunks <= 0 || reduce <= 0) return -1;
  const long tiles = (count + kTileElems - 1) / kTileElems;
  const int grid = gridFor(tiles * chunks);
  bool ok = dispatchCodec(a.codec, [&](auto codecTag) {
    using C = decltype(codecTag);
    decodeReduceEncodeKernel<C><<<grid, kTileThreads, 0, stream>>>(a);
  });
  if (!ok) return -1;
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

// Bounds-checked build: the error word of this translation unit's codec kernels (see codecs.cuh).
extern "C" int cocclkBoundsWordCodec(unsigned int* out, int reset) {
#ifdef COCCL_BOUNDS_CHECK
  cudaError_t e = cudaMemcpyFromSymbol(out, coccl::gBoundsWord, 8 * sizeof(unsigned int));
  if (e == cudaSuccess && reset) {
    const unsigned int zero[8] = {};
    e = cudaMemcpyToSymbol(coccl::gBoundsWord, zero, sizeof(zero));
  }
  return (int)e;
#else
  for (int i = 0; i < 8; ++i) out[i] = 0;
  (void)reset;
  return 0;
#endif
}
