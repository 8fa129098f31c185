// CTA-pair variant of the bf16 GEMM: two CTAs of a cluster (two SMs) work on one 256x256 output
// tile with tcgen05.mma.cta_group::2 (M = 256). Each CTA loads its 128 rows of A and its 128-row half
// of B, so a stage is 32 KiB per SM instead of 48 KiB: six stages and the epilogue boxes fit and the L2->SM traffic per FLOP
// drops by a third, which is what limited the single-CTA kernel (tensor pipe ~72 % busy).
//
// Per CTA: warp 0 = TMA producer (both CTAs; completion bytes are credited to the LEADER's "full"
// barrier, no multicast), warp 1 = MMA issuer (leader CTA only) + TMEM owner, warps 2..5 = epilogue
// over this CTA's 128 accumulator rows. "empty" and "accumulator full" barriers are signalled in both
// CTAs by tcgen05.commit with a CTA mask; "accumulator empty" lives in the leader and collects the
// eight epilogue warps of the pair. Every wait is bounded; a timeout raises the abort flag in both
// CTAs, and both leave through the common cluster barrier after freeing TMEM.
#include "gemm_epilogue.cuh"
#include "launch_count.h"

#include <stdio.h>

namespace coccl {
using namespace sm100;

namespace pair {
constexpr int BM = 128;        // rows per CTA (256 per pair)
constexpr int BN = 256;        // accumulator columns
constexpr int BNH = 128;       // B rows loaded per CTA
constexpr int BK = 64;
constexpr int kStages = 7;      // bf16 outputs (direct stores); fp32 outputs run 6 stages + 32 KiB of TMA boxes
constexpr int kABytes = BM * BK * 2;    // 16 KiB
constexpr int kBBytes = BNH * BK * 2;   // 16 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 192;
constexpr int kGroupM = 8;     // in 256-row tiles
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

struct __align__(8) Barriers {
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
}  // namespace pair

// F32OUT: fp32 output (store or accumulate) through TMA boxes with a 6-stage ring; otherwise bf16 output with direct
// stores and a 7-stage ring (measured faster for bf16 than boxes + 6 stages).
template <bool F32OUT>
__global__ void __launch_bounds__(pair::kThreads, 1)
gemmBf16PairKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, const GemmArgs g) {
  using namespace pair;
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  constexpr int stages = F32OUT ? kStages - 1 : kStages;  // compile-time: the ring index is a division by a constant
  constexpr bool f32 = F32OUT;
  uint8_t* epiStage = smem + stages * kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(epiStage + (F32OUT ? kEpiStageBytes : 0));
  volatile int* abortFlag = &bars->abortFlag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = clusterCtaRank();  // 0 = leader
  const bool leader = cta == 0;
  const int numM = (g.M + 2 * BM - 1) / (2 * BM), numN = (g.N + BN - 1) / BN;
  const int numTiles = numM * numN;
  const int kBlocks = (g.K + BK - 1) / BK;
  const int clusterId = blockIdx.x >> 1, numClusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbarInit(&bars->full[s], 1); mbarInit(&bars->empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbarInit(&bars->tmemFull[i], 1); mbarInit(&bars->tmemEmpty[i], 8); }
    bars->abortFlag = 0;
    mbarFenceInit();
    prefetchTensorMap(&tmA);
    prefetchTensorMap(&tmB);
  }
  if (warp == 1) {
    tmemAlloc2(&bars->tmemBase, 512);
    tmemRelinquish2();
  }
  tcFenceBefore();
  clusterSync();  // barriers of both CTAs exist before anything signals them remotely
  tcFenceAfter();
  const uint32_t tmemBase = bars->tmemBase;
  const uint32_t peerAbort = mapToCta(smemAddr(&bars->abortFlag), cta ^ 1u);
  auto raiseAbort = [&]() { stSharedRemote(peerAbort, 1); };

  if (warp == 0) {
    // ------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = clusterId; t < numTiles && ok; t += numClusters) {
        int tm, tn;
        tileCoord(t, numM, numN, tm, tn);
        const int m0 = tm * 2 * BM + (int)cta * BM;
        const int n0 = tn * BN + (int)cta * BNH;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (!mbarWait(&bars->empty[s], ph ^ 1, abortFlag, kWaitLimitNs)) { ok = false; raiseAbort(); break; }
          if (*abortFlag) { ok = false; break; }
          uint8_t* sa = smem + s * kStageBytes;
          uint8_t* sb = sa + kABytes;
          if (leader) mbarArriveExpectTx(&bars->full[s], 2 * kStageBytes);  // bytes of both CTAs
          const uint32_t fullLeader = mapToCta(smemAddr(&bars->full[s]), 0);
          if (!g.aMN) {
            tmaLoad2dPair(sa, &tmA, fullLeader, kb * BK, m0);
          } else {
            for (int i = 0; i < BM / 64; ++i) tmaLoad2dPair(sa + i * 8192, &tmA, fullLeader, m0 + i * 64, kb * BK);
          }
          if (!g.bMN) {
            tmaLoad2dPair(sb, &tmB, fullLeader, kb * BK, n0);
          } else {
            for (int i = 0; i < BNH / 64; ++i) tmaLoad2dPair(sb + i * 8192, &tmB, fullLeader, n0 + i * 64, kb * BK);
          }
        }
      }
      if (!ok) {
        // The copies in flight signal a barrier of the leader, which the peer cannot poll: give them a
        // fixed time (far longer than any copy takes) before this CTA may leave.
        const unsigned long long start = gtimer();
        while (gtimer() - start < 1000000ull) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (leader only, one thread)
    if (leader && lane == 0) {
      const uint32_t idesc = makeInstrDescBf16(2 * BM, BN, g.aMN != 0, g.bMN != 0);
      uint32_t it = 0, tileIdx = 0;
      bool ok = true;
      for (int t = clusterId; t < numTiles && ok; t += numClusters, ++tileIdx) {
        const int acc = tileIdx & 1;
        const uint32_t accPhase = (tileIdx >> 1) & 1;
        if (!mbarWait(&bars->tmemEmpty[acc], accPhase ^ 1, abortFlag, kWaitLimitNs)) { ok = false; raiseAbort(); break; }
        tcFenceAfter();
        const uint32_t dTmem = tmemBase + acc * BN;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (!mbarWait(&bars->full[s], ph, abortFlag, kWaitLimitNs)) { ok = false; raiseAbort(); break; }
          tcFenceAfter();
          const uint32_t sa = smemAddr(smem + s * kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = g.aMN ? makeSmemDesc(sa + k * 2048, 8192, 1024) : makeSmemDesc(sa + k * 32, 16, 1024);
            const uint64_t db = g.bMN ? makeSmemDesc(sb + k * 2048, 8192, 1024) : makeSmemDesc(sb + k * 32, 16, 1024);
            umma2(dTmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ummaCommit2(&bars->empty[s], 3);                               // frees the stage in both CTAs
          if (kb == kBlocks - 1) ummaCommit2(&bars->tmemFull[acc], 3);   // accumulator ready in both CTAs
        }
      }
    }
  } else {
    // ------------------------------------------------ epilogue warps (both CTAs)
    const int quad = warp & 3;
    uint32_t tileIdx = 0, boxes = 0;
    bool ok = true;
    for (int t = clusterId; t < numTiles && ok; t += numClusters, ++tileIdx) {
      int tm, tn;
      tileCoord(t, numM, numN, tm, tn);
      const int acc = tileIdx & 1;
      const uint32_t accPhase = (tileIdx >> 1) & 1;
      ok = mbarWait(&bars->tmemFull[acc], accPhase, abortFlag, kWaitLimitNs);
      ok = __all_sync(0xffffffffu, ok) != 0;
      if (!ok) { if (lane == 0) raiseAbort(); break; }
      tcFenceAfter();
      const int row0 = tm * 2 * BM + (int)cta * BM + quad * 32;
      const uint32_t tbase = tmemBase + acc * BN + ((uint32_t)(quad * 32) << 16);
      if (f32) {
        if (row0 < g.M)
          epilogueTmaTileF32(&tmC, g.epi == GEMM_EPI_F32_ACC, tbase, row0, tn * BN, g.N, epiStage + quad * kEpiStageBytesPerWarp, boxes);
      } else {
        epilogueStoreTile(g, tbase, row0 + lane, tn * BN);
      }
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArriveRemote(mapToCta(smemAddr(&bars->tmemEmpty[acc]), 0));
    }
    if (f32 && lane == 0) bulkWaitGroup<0>();  // the boxes must have left shared memory before the CTA ends
  }

  __syncwarp();
  tcFenceBefore();
  clusterSync();  // nobody leaves while its partner may still read its shared memory or signal its barriers
  if (warp == 1) {
    tcFenceAfter();
    tmemDealloc2(tmemBase, 512);
  }
  if (threadIdx.x == 0 && bars->abortFlag && g.err) atomicExch(g.err, 0x80000002u);
}

// shared with gemm_kernels.cu
int makeOutputMap(CUtensorMap* m, void* base, long cols, long rows, long ld, bool f32);
int makeBf16TensorMap(CUtensorMap* m, const void* base, long inner, long outer, long ld, int boxInner, int boxOuter);

}  // namespace coccl

using namespace coccl;

extern "C" int cocclkGemmBf16Pair(const void* A, long lda, int aMN, const void* B, long ldb, int bMN, void* C, long ldc,
                                  int M, int N, int K, int epi, const void* bias, void* Z, unsigned int* err, int maxCtas,
                                  cudaStream_t stream) {
  using namespace pair;
  // K-major operands have rows of K elements (16-byte multiples for TMA); operands stored with M / N contiguous put
  // no constraint on K (rows past K read as zeros)
  if (M <= 0 || N <= 0 || K <= 0 || (N & 7) || ((!aMN || !bMN) && (K & 7))) return -1;
  if ((epi == GEMM_EPI_BIAS || epi == GEMM_EPI_BIAS_GELU) && bias == nullptr) return -1;
  CUtensorMap ta, tb;
  int rc = aMN ? makeBf16TensorMap(&ta, A, M, K, lda, 64, 64) : makeBf16TensorMap(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = bMN ? makeBf16TensorMap(&tb, B, N, K, ldb, 64, 64) : makeBf16TensorMap(&tb, B, K, N, ldb, BK, BNH);
  if (rc) return rc;
  static int maxClusters = 0;
  static bool attrSet = false;
  const bool f32 = epi == GEMM_EPI_F32 || epi == GEMM_EPI_F32_ACC;
  CUtensorMap tc = ta;  // placeholder for bf16 outputs (direct stores)
  if (f32) {
    rc = makeOutputMap(&tc, C, N, M, ldc, true);
    if (rc) return rc;
  }
  const int stages = f32 ? kStages - 1 : kStages;
  const int smemBytes = stages * kStageBytes + (f32 ? kEpiStageBytes : 0) + (int)sizeof(Barriers) + 1024;
  if (!attrSet) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(gemmBf16PairKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kStages * kStageBytes + (int)sizeof(Barriers) + 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemmBf16PairKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (kStages - 1) * kStageBytes + kEpiStageBytes + (int)sizeof(Barriers) + 1024);
    if (e != cudaSuccess) return (int)e;
    maxClusters = sms / 2;
    // how many pairs the device can hold at once (SMs pair up inside a GPC)
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3((unsigned)(sms / 2) * 2, 1, 1);
    q.blockDim = dim3(kThreads, 1, 1);
    q.dynamicSmemBytes = (size_t)(kStages * kStageBytes + (int)sizeof(Barriers) + 1024);
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
    q.attrs = qa; q.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemmBf16PairKernel<false>, &q) == cudaSuccess && n > 0 && n < maxClusters) maxClusters = n;
    (void)cudaGetLastError();
    attrSet = true;
  }
  GemmArgs g;
  g.C = C; g.Z = Z; g.bias = bias; g.M = M; g.N = N; g.K = K; g.ldc = ldc; g.epi = epi; g.aMN = aMN; g.bMN = bMN; g.err = err;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  int clusters = maxClusters;
  if (tiles < clusters) clusters = tiles;
  if (maxCtas > 1 && clusters > maxCtas / 2) clusters = maxCtas / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)clusters * 2, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  g.stages = stages;
  cudaError_t e = f32 ? cudaLaunchKernelEx(&cfg, gemmBf16PairKernel<true>, ta, tb, tc, g)
                      : cudaLaunchKernelEx(&cfg, gemmBf16PairKernel<false>, ta, tb, tc, g);
  cocclkCountLaunches(1);
  return (int)e;
}
