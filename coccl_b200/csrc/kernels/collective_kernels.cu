// Launcher of the fused compressed collectives (see collective_kernels.cuh).
#include "launch_count.h"
#include "collective_kernels.cuh"
#include "kernels_api.h"
#include <string.h>

using namespace coccl;

static_assert(sizeof(cocclkCollArgs) == sizeof(CollArgs), "collective POD mismatch");
static_assert(COCCLK_MAX_SLICES == kMaxSlices && COCCLK_MAX_RANKS == kMaxRanks, "constant mismatch");

extern "C" long cocclkFlagBytes(void) { return 2L * kMaxRanks * kMaxSlices * (long)sizeof(unsigned int); }

extern "C" int cocclkTileElems(void) { return kTileElems; }

extern "C" long cocclkSlotBytes(const cocclkCodec* codec, long count) {
  CodecCfg c;
  memcpy(&c, codec, sizeof(c));
  return makeChunkLayout(c, count, 16).stride;
}

template <typename T, class C>
static int launchOne(const CollArgs& a, int emulatedRanks, int maxCtas, cudaStream_t stream) {
  auto kern = fusedCollectiveKernel<T, C>;
  static int perSm = 0, sms = 0;
  if (perSm == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kern, kTileThreads, 0);
    if (e != cudaSuccess) return (int)e;
    if (perSm <= 0) return -1;
  }
  const long tiles = (a.count + kTileElems - 1) / kTileElems;
  const long slices = (tiles + a.sliceTiles - 1) / a.sliceTiles;
  if (slices > kMaxSlices) return -1;
  long items = slices * a.nRanks;
  long cap = (long)perSm * sms / emulatedRanks;
  if (maxCtas > 0 && maxCtas < cap) cap = maxCtas;
  if (cap < 1) cap = 1;
  int gx = (int)(items < cap ? items : cap);
  dim3 grid(gx, emulatedRanks, 1);
  CollArgs copy = a;
  cocclkCountLaunches(1);
  void* params[] = {&copy};
  if (emulatedRanks > 1) {
    // the emulated ranks wait on one another: co-residency must be guaranteed
    return (int)cudaLaunchCooperativeKernel((const void*)kern, grid, dim3(kTileThreads), params, 0, stream);
  }
  return (int)cudaLaunchKernel((const void*)kern, grid, dim3(kTileThreads), params, 0, stream);
}

extern "C" int cocclkFusedCollective(const cocclkCollArgs* args, int emulatedRanks, int maxCtas,
                                     cudaStream_t stream) {
  CollArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.nRanks < 1 || a.nRanks > kMaxRanks || a.count <= 0 || a.sliceTiles <= 0) return -1;
  if (emulatedRanks != 1 && emulatedRanks != a.nRanks) return -1;
  if (!tileCodecSupported(a.codec)) return -1;
  int rc = -1;
  bool ok = dispatchCodec(a.codec, [&](auto codecTag) {
    using C = decltype(codecTag);
    switch (a.dtype) {
      case kF32: rc = launchOne<float, C>(a, emulatedRanks, maxCtas, stream); break;
      case kF16: rc = launchOne<__half, C>(a, emulatedRanks, maxCtas, stream); break;
      case kBF16: rc = launchOne<__nv_bfloat16, C>(a, emulatedRanks, maxCtas, stream); break;
      default: rc = -1;
    }
  });
  return ok ? rc : -1;
}

// ---------------------------------------------------------------------------------------------
// Bounds-checked build (libcoccl_checked.so, -DCOCCL_BOUNDS_CHECK): 1 when the codec accesses of the fused collectives
// and the stand-alone codec kernels are range-checked, and the first violation they recorded:
// out[0] = 0x80000000 | site (1 encode store, 2 decode fetch, 3 re-encode store of the two-shot all-reduce) or 0,
// out[1..2] = element index, out[3] / out[4] = payload end touched / payload bytes, out[5] / out[6] = chunk end touched /
// chunk bytes. Synchronises the device.
extern "C" int cocclkBoundsWordCodec(unsigned int* out, int reset);
extern "C" int cocclkBoundsChecked(void) {
#ifdef COCCL_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}
extern "C" int cocclkBoundsWord(unsigned int* out, int reset) {
  if (out == nullptr) return -1;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  unsigned int other[8];
  int rc = cocclkBoundsWordCodec(other, reset);
  if (rc != 0) return rc;
#ifdef COCCL_BOUNDS_CHECK
  e = cudaMemcpyFromSymbol(out, coccl::gBoundsWord, 8 * sizeof(unsigned int));
  if (e == cudaSuccess && reset) {
    const unsigned int zero[8] = {};
    e = cudaMemcpyToSymbol(coccl::gBoundsWord, zero, sizeof(zero));
  }
  if (e != cudaSuccess) return (int)e;
#else
  for (int i = 0; i < 8; ++i) out[i] = 0;
#endif
  if (out[0] == 0) for (int i = 0; i < 8; ++i) out[i] = other[i];
  return 0;
}
