// Persistent, warp-specialised bf16 GEMM for sm_100a:
//   C[M,N] = A[M,K] * B[N,K]^T   (either operand may instead be stored with its
//   M/N dimension contiguous, which covers dgrad and wgrad without transposes)
// TMA (128-byte swizzle, no multicast) -> 4-stage shared-memory ring ->
// tcgen05.mma (128x256x16, cta_group::1) -> two 256-column TMEM accumulators so
// the epilogue of tile i overlaps the main loop of tile i+1 -> tcgen05.ld ->
// fused epilogue (bias, GELU, fp32 accumulate) -> global stores.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 =
// epilogue (TMEM lane quadrant = warp % 4). Every mbarrier wait is bounded; on
// a timeout the kernel raises the error word, drains its outstanding copies,
// frees TMEM and returns.
#include <atomic>
#include "launch_count.h"
#include "gemm_epilogue.cuh"
#include <stdio.h>
#include <string.h>
#include <stdlib.h>

namespace coccl {
using namespace sm100;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;            // 16 KiB
constexpr int kBBytes = BN * BK * 2;            // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;  // 48 KiB
constexpr int kGemmThreads = 192;
constexpr int kGroupM = 16;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s


struct __align__(8) GemmBarriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmemFull[2];
  uint64_t tmemEmpty[2];
  uint32_t tmemBase;
  int abortFlag;
};

__device__ __forceinline__ void tileCoord(int t, int numM, int numN, int& tm, int& tn) {
  const int perGroup = kGroupM * numN;
  const int g = t / perGroup;
  const int firstM = g * kGroupM;
  const int rows = min(numM - firstM, kGroupM);
  const int r = t - g * perGroup;
  tm = firstM + r % rows;
  tn = r / rows;
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemmBf16Kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const GemmArgs g) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* epiStage = smem + kStages * kStageBytes;  // TMA boxes of the fp32 epilogues
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(epiStage + kEpiStageBytes);
  volatile int* abortFlag = &bars->abortFlag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int numM = (g.M + BM - 1) / BM, numN = (g.N + BN - 1) / BN;
  const int numTiles = numM * numN;
  const int kBlocks = (g.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbarInit(&bars->full[s], 1); mbarInit(&bars->empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbarInit(&bars->tmemFull[i], 1); mbarInit(&bars->tmemEmpty[i], 4); }
    bars->abortFlag = 0;
    mbarFenceInit();
    prefetchTensorMap(&tmA);
    prefetchTensorMap(&tmB);
  }
  if (warp == 1) {
    tmemAlloc(&bars->tmemBase, 512);
    tmemRelinquish();
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = bars->tmemBase;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
        int tm, tn;
        tileCoord(t, numM, numN, tm, tn);
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbarWait(&bars->empty[s], ph ^ 1, abortFlag, kWaitLimitNs)) { ok = false; break; }
          uint8_t* sa = smem + s * kStageBytes;
          uint8_t* sb = sa + kABytes;
          mbarArriveExpectTx(&bars->full[s], kStageBytes);
          if (!g.aMN) {
            tmaLoad2d(sa, &tmA, &bars->full[s], kb * BK, tm * BM);
          } else {
            for (int i = 0; i < BM / 64; ++i) tmaLoad2d(sa + i * 8192, &tmA, &bars->full[s], tm * BM + i * 64, kb * BK);
          }
          if (!g.bMN) {
            tmaLoad2d(sb, &tmB, &bars->full[s], kb * BK, tn * BN);
          } else {
            for (int i = 0; i < BN / 64; ++i) tmaLoad2d(sb + i * 8192, &tmB, &bars->full[s], tn * BN + i * 64, kb * BK);
          }
        }
      }
      if (!ok) {
        // drain: give the copies already issued a bounded time to land
        for (uint32_t back = 1; back <= (uint32_t)kStages && back <= it; ++back) {
          const uint32_t j = it - back;
          const unsigned long long start = gtimer();
          while (!mbarTryWait(&bars->full[j % kStages], (j / kStages) & 1)) {
            if (gtimer() - start > 100000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    const uint32_t idesc = makeInstrDescBf16(BM, BN, g.aMN != 0, g.bMN != 0);
    uint32_t it = 0, tileIdx = 0;
    bool ok = true;
    // a single thread issues every MMA and commit (they are single-thread instructions)
    for (int t = blockIdx.x; lane == 0 && t < numTiles && ok; t += gridDim.x, ++tileIdx) {
      const int acc = tileIdx & 1;
      const uint32_t accPhase = (tileIdx >> 1) & 1;
      if (!mbarWait(&bars->tmemEmpty[acc], accPhase ^ 1, abortFlag, kWaitLimitNs)) { ok = false; break; }
      tcFenceAfter();
      const uint32_t dTmem = tmemBase + acc * BN;
      for (int kb = 0; kb < kBlocks; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbarWait(&bars->full[s], ph, abortFlag, kWaitLimitNs)) { ok = false; break; }
        tcFenceAfter();
        {
          const uint32_t sa = smemAddr(smem + s * kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = g.aMN ? makeSmemDesc(sa + k * 2048, 8192, 1024) : makeSmemDesc(sa + k * 32, 16, 1024);
            const uint64_t db = g.bMN ? makeSmemDesc(sb + k * 2048, 8192, 1024) : makeSmemDesc(sb + k * 32, 16, 1024);
            umma(dTmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ummaCommit(&bars->empty[s]);
          if (kb == kBlocks - 1) ummaCommit(&bars->tmemFull[acc]);
        }
      }
    }
  } else {
    // ------------------------------------------------ epilogue warps
    const int quad = warp & 3;
    const bool f32 = g.epi == GEMM_EPI_F32 || g.epi == GEMM_EPI_F32_ACC;
    uint32_t tileIdx = 0, boxes = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++tileIdx) {
      int tm, tn;
      tileCoord(t, numM, numN, tm, tn);
      const int acc = tileIdx & 1;
      const uint32_t accPhase = (tileIdx >> 1) & 1;
      ok = mbarWait(&bars->tmemFull[acc], accPhase, abortFlag, kWaitLimitNs);
      ok = __all_sync(0xffffffffu, ok) != 0;  // tcgen05.ld below needs the whole warp
      if (!ok) break;
      tcFenceAfter();
      const int row0 = tm * BM + quad * 32;
      const uint32_t tbase = tmemBase + acc * BN + ((uint32_t)(quad * 32) << 16);
      if (f32) {
        if (row0 < g.M)
          epilogueTmaTileF32(&tmC, g.epi == GEMM_EPI_F32_ACC, tbase, row0, tn * BN, g.N, epiStage + quad * kEpiStageBytesPerWarp, boxes);
      } else if (row0 < g.M) {
        epilogueTmaTileBf16(g, &tmC, tbase, row0, tn * BN, epiStage + quad * kEpiStageBytesPerWarp, boxes);
      }
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArrive(&bars->tmemEmpty[acc]);
    }
    if (lane == 0) bulkWaitGroup<0>();  // the boxes must have left shared memory before the CTA ends
  }

  tcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    tcFenceAfter();
    tmemDealloc(tmemBase, 512);
  }
  if (threadIdx.x == 0 && bars->abortFlag && g.err) atomicExch(g.err, 0x80000001u);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encodeTiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor maps are a pure function of (address, extents, pitch, box, type): the driver call that encodes one costs
// about a microsecond, and a training step asks for the same few hundred maps several thousand times (weights,
// activations and gradients sit at fixed addresses). A small direct-mapped table per thread returns the encoded
// map for a repeated request; a colliding request simply replaces the entry.
struct MapKey {
  const void* base;
  long d0, d1, ld;
  int b0, b1, kind;
  bool operator==(const MapKey& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && ld == o.ld && b0 == o.b0 && b1 == o.b1 && kind == o.kind;
  }
};
struct MapSlot { MapKey key; CUtensorMap map; bool valid; };
constexpr int kMapSlots = 1024;
static MapSlot* mapSlot(const MapKey& k) {
  static thread_local MapSlot* table = nullptr;
  if (table == nullptr) table = new MapSlot[kMapSlots]();
  uint64_t h = reinterpret_cast<uintptr_t>(k.base) >> 4;
  h = (h ^ (uint64_t)k.d0 * 0x9e3779b97f4a7c15ull ^ (uint64_t)k.d1 * 0xc2b2ae3d27d4eb4full ^ (uint64_t)k.ld * 0x165667b19e3779f9ull ^
       (uint64_t)(k.b0 * 131 + k.b1 * 17 + k.kind)) * 0xff51afd7ed558ccdull;
  return &table[(h >> 40) % kMapSlots];
}
static std::atomic<unsigned long long> gMapHits{0}, gMapMisses{0};

// 2-D tensor map of an output matrix for the epilogue boxes: 32 rows x 128 bytes (32 fp32 or 64 bf16 columns),
// 128-byte swizzle.
int makeOutputMap(CUtensorMap* m, void* base, long cols, long rows, long ld, bool f32) {
  EncodeTiledFn f = encodeTiled();
  if (!f) return -2;
  static thread_local bool ctxBound = false;
  if (!ctxBound) { cudaFree(nullptr); ctxBound = true; }
  const int es_ = f32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((ld * es_) & 15)) return -3;
  const MapKey key{base, cols, rows, ld, 128 / es_, 32, f32 ? 2 : 1};
  MapSlot* slot = mapSlot(key);
  if (slot->valid && slot->key == key) { *m = slot->map; ++gMapHits; return 0; }
  ++gMapMisses;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * es_};
  cuuint32_t box[2] = {(cuuint32_t)(128 / es_), 32};
  cuuint32_t es[2] = {1, 1};
  CUresult r = f(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "coccl: cuTensorMapEncodeTiled (output) failed (%d): base=%p dims={%ld,%ld} ld=%ld\n", (int)r, base, cols, rows, ld);
    return -4;
  }
  slot->key = key; slot->map = *m; slot->valid = true;
  return 0;
}

// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows `ld` elements apart.
static int makeMap(CUtensorMap* m, const void* base, long inner, long outer, long ld, int boxInner, int boxOuter) {
  EncodeTiledFn f = encodeTiled();
  if (!f) return -2;
  // The driver call needs a current context; a thread that has only ever been handed work (an
  // autograd worker) may not have bound the primary context yet.
  static thread_local bool ctxBound = false;
  if (!ctxBound) { cudaFree(nullptr); ctxBound = true; }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((ld * 2) & 15)) return -3;
  const MapKey key{base, inner, outer, ld, boxInner, boxOuter, 0};
  MapSlot* slot = mapSlot(key);
  if (slot->valid && slot->key == key) { *m = slot->map; ++gMapHits; return 0; }
  ++gMapMisses;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)boxInner, (cuuint32_t)boxOuter};
  cuuint32_t es[2] = {1, 1};
  CUresult r = f(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "coccl: cuTensorMapEncodeTiled failed (%d): base=%p dims={%ld,%ld} ld=%ld box={%d,%d}\n", (int)r,
            base, inner, outer, ld, boxInner, boxOuter);
    return -4;
  }
  slot->key = key; slot->map = *m; slot->valid = true;
  return 0;
}

int makeBf16TensorMap(CUtensorMap* m, const void* base, long inner, long outer, long ld, int boxInner, int boxOuter) {
  return makeMap(m, base, inner, outer, ld, boxInner, boxOuter);
}

}  // namespace coccl

// (hits, misses) of the tensor-map table since the library was loaded, all threads.
extern "C" void cocclkTensorMapCacheStats(unsigned long long* hits, unsigned long long* misses) {
  if (hits) *hits = coccl::gMapHits.load();
  if (misses) *misses = coccl::gMapMisses.load();
}

using namespace coccl;

extern "C" int cocclkGemmBf16Pair(const void* A, long lda, int aMN, const void* B, long ldb, int bMN, void* C, long ldc,
                                  int M, int N, int K, int epi, const void* bias, void* Z, unsigned int* err, int maxCtas,
                                  cudaStream_t stream);

// 0 = choose by shape, 1 = always the single-CTA kernel, 2 = the CTA-pair kernel whenever the shape allows it.
// The initial value comes from COCCL_GEMM_VARIANT ("1cta" / "2cta").
static int gGemmVariant = -1;
extern "C" void cocclkGemmSetVariant(int v) { gGemmVariant = v; }
extern "C" int cocclkGemmGetVariant() {
  if (gGemmVariant < 0) {
    const char* e = getenv("COCCL_GEMM_VARIANT");
    gGemmVariant = (e && !strcmp(e, "1cta")) ? 1 : (e && !strcmp(e, "2cta")) ? 2 : 0;
  }
  return gGemmVariant;
}

extern "C" int cocclkGemmBf16Single(const void* A, long lda, int aMN, const void* B, long ldb, int bMN, void* C, long ldc,
                              int M, int N, int K, int epi, const void* bias, void* Z, unsigned int* err,
                              int maxCtas, cudaStream_t stream) {
  // K-major operands have rows of K elements (16-byte multiples for TMA); operands stored with M / N contiguous put
  // no constraint on K (rows past K read as zeros)
  if (M <= 0 || N <= 0 || K <= 0 || (N & 7) || ((!aMN || !bMN) && (K & 7))) return -1;
  if ((epi == GEMM_EPI_BIAS || epi == GEMM_EPI_BIAS_GELU) && bias == nullptr) return -1;
  CUtensorMap ta, tb;
  int rc;
  // K-major: inner = K, outer = rows, box {64, rows}; MN-major: inner = rows, outer = K, box {64, 64}
  rc = aMN ? makeMap(&ta, A, M, K, lda, 64, 64) : makeMap(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = bMN ? makeMap(&tb, B, N, K, ldb, 64, 64) : makeMap(&tb, B, K, N, ldb, BK, BN);
  if (rc) return rc;
  static int sms = 0;
  static bool attrSet = false;
  CUtensorMap tc;
  rc = makeOutputMap(&tc, C, N, M, ldc, epi == GEMM_EPI_F32 || epi == GEMM_EPI_F32_ACC);
  if (rc) return rc;
  const int smemBytes = kStages * kStageBytes + kEpiStageBytes + (int)sizeof(GemmBarriers) + 1024;
  if (!attrSet) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(gemmBf16Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes);
    if (e != cudaSuccess) return (int)e;
    attrSet = true;
  }
  GemmArgs g;
  g.C = C; g.Z = Z; g.bias = bias; g.M = M; g.N = N; g.K = K; g.ldc = ldc; g.epi = epi; g.aMN = aMN; g.bMN = bMN;
  g.err = err;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tiles < sms ? tiles : sms;
  if (maxCtas > 0 && grid > maxCtas) grid = maxCtas;
  g.stages = kStages;
  gemmBf16Kernel<<<grid, kGemmThreads, smemBytes, stream>>>(ta, tb, tc, g);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

extern "C" int cocclkGemmBf16(const void* A, long lda, int aMN, const void* B, long ldb, int bMN, void* C, long ldc,
                              int M, int N, int K, int epi, const void* bias, void* Z, unsigned int* err,
                              int maxCtas, cudaStream_t stream) {
  const int v = cocclkGemmGetVariant();
  // The pair kernel works on 256-row tiles: below that half of each pair would idle. A CTA limit of one
  // cannot host a pair.
  const bool pairOk = M > 128 && maxCtas != 1;
  if (v != 1 && pairOk)
    return cocclkGemmBf16Pair(A, lda, aMN, B, ldb, bMN, C, ldc, M, N, K, epi, bias, Z, err, maxCtas, stream);
  return cocclkGemmBf16Single(A, lda, aMN, B, ldb, bMN, C, ldc, M, N, K, epi, bias, Z, err, maxCtas, stream);
}
