// Tensor-parallel fusions on the CTA-pair main loop (tcgen05.mma.cta_group::2, 256x256 tiles per pair of SMs).
//
//  agGemmPairKernel  C = gather(A) * B^T. Warps 6-7 of every CTA push this rank's activation shard into the peers'
//                    gather buffers in RING ORDER: the whole shard for rank-1 first, then rank-2, ... so that at
//                    every moment each GPU sends to one peer and receives from one, and the shard the local tensor
//                    cores need next is the one on the wire. A shard travels as pieces of 16 rows x K/4 columns
//                    with one release flag each; the TMA producer of a CTA waits for the flags of its 128 rows
//                    right before it loads them (from LOCAL memory; no multicast anywhere). With agPayload = 1 the
//                    pieces travel as E4M3 + UE8M0 scales (MX-FP8, half the bytes): after pushing ring step s the
//                    push warps dequantise the pieces of step s that arrive from the other side into the bf16 gather
//                    buffer and raise a second, local set of flags, which the producer then waits for instead.
//  gemmRsPairKernel  out = reduce_scatter(A * B^T). Tiles for the next rank in the ring are computed first, own rows
//                    last. For a foreign row block the epilogue quantises the fp32 accumulator to E4M3 with one
//                    UE8M0 scale per 32 columns and pushes it into the destination's slot. For an OWN row block the
//                    epilogue IS the reducer: it waits for the flags of the N-1 copies that arrived during the
//                    earlier steps, adds their dequantised values to the accumulator it just read from TMEM (the
//                    own contribution never gets quantised) and writes bf16. No reduction pass trails the GEMM.
//
// Per CTA: warp 0 TMA producer (both CTAs; bytes are credited to the leader's barrier), warp 1 MMA issuer (leader
// only) + TMEM owner, warps 2..5 epilogue over this CTA's 128 accumulator rows, warps 6..7 push (all-gather) or
// idle (reduce-scatter). blockIdx.y lets one launch play every rank on one GPU for tests. Every wait is bounded; a
// wait that runs out raises the abort flag in both CTAs of the pair, reports through the status / error words and
// the kernel leaves through the common cluster barrier after freeing TMEM.
//
// The reference has no GEMM; these kernels serve the traffic of its policy slots
// training.tp.{all_gather,reduce_scatter} (src/coccl-extend/core/config/coccl_config.cc:669-695).
#include "codecs.cuh"
#include "gemm_epilogue.cuh"
#include "launch_count.h"
#include "tp_api.h"

#include <string.h>

namespace coccl {
using namespace sm100;

int makeBf16TensorMap(CUtensorMap* m, const void* base, long inner, long outer, long ld, int boxInner, int boxOuter);

namespace tp2 {
constexpr int BM = 128;    // rows per CTA (256 per pair)
constexpr int BN = 256;    // accumulator columns
constexpr int BNH = 128;   // B rows loaded per CTA
constexpr int BK = 64;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BNH * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;  // 32 KiB
constexpr int kAgStages = 7;
constexpr int kRsStages = 6;                    // one stage goes to the epilogue's staging rows
constexpr int kThreads = 256;
constexpr int kPartRows = 16;                   // rows per pushed piece of the gather
constexpr int kFlagStride = 4096;               // flags per source rank
constexpr int kReadyRegion = COCCLK_TP_MAX_RANKS;  // flag rows [kReadyRegion + shard]: piece dequantised (FP8 payload)
constexpr int kStageRowBytes = 128 + 16;        // staging row: half a tile row of fp8 + padding against bank conflicts
constexpr int kEpiStageBytes = 4 * 32 * kStageRowBytes;
constexpr unsigned long long kPipeWaitNs = 4000000000ull;

struct __align__(8) Barriers {
  uint64_t full[kAgStages];
  uint64_t empty[kAgStages];
  uint64_t tmemFull[2];
  uint64_t tmemEmpty[2];
  uint32_t tmemBase;
  int abortFlag;
};

struct Params {
  cocclkTpArgs a;
  int pieces;  // all-gather: column pieces per 16-row part
  CUtensorMap maps[COCCLK_TP_MAX_EMULATED][3];  // [emulated rank][A gathered / full, A local shard, B]
};

constexpr int smemBytes(int stages, bool staging) {
  return stages * kStageBytes + (staging ? kEpiStageBytes : 0) + (int)sizeof(Barriers) + 1024;
}

__device__ __forceinline__ void fenceProxyAsyncGlobal() { asm volatile("fence.proxy.async;" ::: "memory"); }

struct Pipe {
  uint8_t* smem;
  uint8_t* epiStage;
  Barriers* bars;
  volatile int* abortFlag;
  uint32_t tmemBase;
  uint32_t peerAbort;
  uint32_t cta;
};

template <int STAGES, bool STAGING>
__device__ __forceinline__ Pipe pipeSetup(uint8_t* smemRaw, const CUtensorMap* m0, const CUtensorMap* m1, const CUtensorMap* m2) {
  Pipe p;
  p.smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  p.epiStage = p.smem + STAGES * kStageBytes;
  p.bars = reinterpret_cast<Barriers*>(p.epiStage + (STAGING ? kEpiStageBytes : 0));
  p.abortFlag = &p.bars->abortFlag;
  p.cta = clusterCtaRank();
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbarInit(&p.bars->full[s], 1); mbarInit(&p.bars->empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbarInit(&p.bars->tmemFull[i], 1); mbarInit(&p.bars->tmemEmpty[i], 8); }
    p.bars->abortFlag = 0;
    mbarFenceInit();
    prefetchTensorMap(m0);
    prefetchTensorMap(m1);
    prefetchTensorMap(m2);
  }
  if (warp == 1) {
    tmemAlloc2(&p.bars->tmemBase, 512);
    tmemRelinquish2();
  }
  tcFenceBefore();
  clusterSync();  // the barriers of both CTAs exist before anything signals them remotely
  tcFenceAfter();
  p.tmemBase = p.bars->tmemBase;
  p.peerAbort = mapToCta(smemAddr(&p.bars->abortFlag), p.cta ^ 1u);
  return p;
}

__device__ __forceinline__ void raiseAbort(const Pipe& p) {
  *p.abortFlag = 1;
  stSharedRemote(p.peerAbort, 1);
}

__device__ __forceinline__ void pipeTeardown(const Pipe& p, unsigned int* err, unsigned int code) {
  __syncwarp();
  tcFenceBefore();
  clusterSync();  // nobody leaves while its partner may still read its shared memory or signal its barriers
  if ((threadIdx.x >> 5) == 1) {
    tcFenceAfter();
    tmemDealloc2(p.tmemBase, 512);
  }
  if (threadIdx.x == 0 && p.bars->abortFlag && err) atomicExch(err, code);
}

// One k-block of this CTA's operands: 128 rows of A at (arow, kb) and this CTA's 128-row half of B.
__device__ __forceinline__ void loadStage(const Pipe& p, int s, const CUtensorMap* tmA, const CUtensorMap* tmB, int kb,
                                          int arow, int n0, bool bMN) {
  uint8_t* sa = p.smem + s * kStageBytes;
  uint8_t* sb = sa + kABytes;
  if (p.cta == 0) mbarArriveExpectTx(&p.bars->full[s], 2 * kStageBytes);  // bytes of both CTAs
  const uint32_t fullLeader = mapToCta(smemAddr(&p.bars->full[s]), 0);
  tmaLoad2dPair(sa, tmA, fullLeader, kb * BK, arow);
  if (!bMN) {
    tmaLoad2dPair(sb, tmB, fullLeader, kb * BK, n0);
  } else {
    for (int i = 0; i < BNH / 64; ++i) tmaLoad2dPair(sb + i * 8192, tmB, fullLeader, n0 + i * 64, kb * BK);
  }
}

// After a failed wait the copies already in flight signal a barrier of the leader, which the partner cannot poll:
// give them a fixed time, far longer than any copy takes, before this CTA may leave.
__device__ __forceinline__ void drainWait() {
  const unsigned long long start = gtimer();
  while (gtimer() - start < 1000000ull) {}
}

template <int STAGES>
__device__ __forceinline__ void mmaRole(const Pipe& p, int firstTile, int numTiles, int tileStep, int kBlocks, bool bMN) {
  const uint32_t idesc = makeInstrDescBf16(2 * BM, BN, false, bMN);
  uint32_t it = 0, tileIdx = 0;
  for (int t = firstTile; t < numTiles; t += tileStep, ++tileIdx) {
    const int acc = tileIdx & 1;
    const uint32_t accPhase = (tileIdx >> 1) & 1;
    if (!mbarWait(&p.bars->tmemEmpty[acc], accPhase ^ 1, p.abortFlag, kPipeWaitNs)) { raiseAbort(p); return; }
    tcFenceAfter();
    const uint32_t dTmem = p.tmemBase + acc * BN;
    for (int kb = 0; kb < kBlocks; ++kb, ++it) {
      const int s = it % STAGES;
      const uint32_t ph = (it / STAGES) & 1;
      if (!mbarWait(&p.bars->full[s], ph, p.abortFlag, kPipeWaitNs)) { raiseAbort(p); return; }
      tcFenceAfter();
      const uint32_t sa = smemAddr(p.smem + s * kStageBytes);
      const uint32_t sb = sa + kABytes;
#pragma unroll
      for (int k = 0; k < BK / 16; ++k) {
        const uint64_t db = bMN ? makeSmemDesc(sb + k * 2048, 8192, 1024) : makeSmemDesc(sb + k * 32, 16, 1024);
        umma2(dTmem, makeSmemDesc(sa + k * 32, 16, 1024), db, idesc, (kb | k) != 0 ? 1u : 0u);
      }
      ummaCommit2(&p.bars->empty[s], 3);                              // frees the stage in both CTAs
      if (kb == kBlocks - 1) ummaCommit2(&p.bars->tmemFull[acc], 3);  // accumulator ready in both CTAs
    }
  }
}

// ---------------------------------------------------------------------------------------------
// all-gather -> GEMM
// ---------------------------------------------------------------------------------------------
// Tile t -> (ring step, 256-row tile inside the shard, column tile). Inside a shard the column tile runs fastest:
// the clusters that work at the same time then share a few row tiles, so a remote shard is needed in the order in
// which it arrives instead of all at once.
__device__ __forceinline__ void agTile(int t, int tilesPerShard, int tps, int numN, int& step, int& tmL, int& tn) {
  step = t / tilesPerShard;
  const int r = t - step * tilesPerShard;
  tmL = r / numN;
  tn = r - tmL * numN;
  (void)tps;
}

// One warp copies a piece of 16 rows x pcv 16-byte vectors (row pitch rowVecs) with eight loads in flight per lane.
// CG: the source was written by a peer during this launch, so the loads must not come from L1.
template <bool CG>
__device__ __forceinline__ void copyPiece(const uint4* src, uint4* dst, long base, long rowVecs, int pcv, int lane) {
  if ((pcv & 31) == 0) {
    for (int c0 = 0; c0 < pcv; c0 += 32) {
#pragma unroll 1
      for (int r0 = 0; r0 < kPartRows; r0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint4* q = src + base + (long)(r0 + u) * rowVecs + c0 + lane;
          v[u] = CG ? __ldcg(q) : __ldg(q);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) dst[base + (long)(r0 + u) * rowVecs + c0 + lane] = v[u];
      }
    }
  } else {
    for (int r0 = 0; r0 < kPartRows; ++r0)
      for (int c = lane; c < pcv; c += 32) {
        const uint4* q = src + base + (long)r0 * rowVecs + c;
        dst[base + (long)r0 * rowVecs + c] = CG ? __ldcg(q) : __ldg(q);
      }
  }
}

// Where the FP8 rows and their scales of the gather live inside a rank's workspace (behind the bf16 gather buffer).
__device__ __host__ __forceinline__ long ag8Offset(long M, long K) { return (M * K * 2 + 255) & ~255L; }
__device__ __host__ __forceinline__ long agScaleOffset(long M, long K) { return ag8Offset(M, K) + ((M * K + 255) & ~255L); }

// One warp quantises a piece of 16 rows x (blocks * 32) columns: bf16 rows (pitch K) -> E4M3 rows (pitch K bytes) and
// one UE8M0 byte per 32 columns (pitch K / 32), both in the PEER's memory. A lane owns whole 32-column blocks.
__device__ __forceinline__ void quantPiece(const __nv_bfloat16* src, uint8_t* dst8, uint8_t* dstScale, long K, int blocks, int lane) {
  const CodecCfg cfg{};
  const int total = kPartRows * blocks;
  for (int i = lane; i < total; i += 32) {
    const int r = i / blocks, b = i - r * blocks;
    const uint4* q = reinterpret_cast<const uint4*>(src + (long)r * K + b * 32);
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) raw[u] = __ldg(q + u);
    float v[32];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[8 * u + 2 * k] = __uint_as_float(w[k] << 16);
        v[8 * u + 2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
      }
    }
    const MxFp8Codec::Enc e = MxFp8Codec::encode(v, cfg, false, nullptr, 0);
    uint4* d = reinterpret_cast<uint4*>(dst8 + (long)r * K + b * 32);
    d[0] = make_uint4(e.w[0], e.w[1], e.w[2], e.w[3]);
    d[1] = make_uint4(e.w[4], e.w[5], e.w[6], e.w[7]);
    dstScale[(long)r * (K / 32) + b] = (uint8_t)e.scaleByte;
  }
}

// The inverse on the receiving side: E4M3 rows + scales that a peer stored during this launch (L2 loads) -> bf16 rows of
// the local gather buffer.
__device__ __forceinline__ void dequantPiece(const uint8_t* src8, const uint8_t* srcScale, __nv_bfloat16* dst, long K, int blocks, int lane) {
  const int total = kPartRows * blocks;
  for (int i = lane; i < total; i += 32) {
    const int r = i / blocks, b = i - r * blocks;
    const uint4* q = reinterpret_cast<const uint4*>(src8 + (long)r * K + b * 32);
    MxFp8Codec::Raw raw;
    const uint4 x = __ldcg(q), y = __ldcg(q + 1);
    raw.w[0] = x.x; raw.w[1] = x.y; raw.w[2] = x.z; raw.w[3] = x.w; raw.w[4] = y.x; raw.w[5] = y.y; raw.w[6] = y.z; raw.w[7] = y.w;
    raw.biased = __ldcg(srcScale + (long)r * (K / 32) + b);
    raw.valid = true;
    float v[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) v[k] = 0.f;
    MxFp8Codec::accumulate(raw, v);
    uint4* d = reinterpret_cast<uint4*>(dst + (long)r * K + b * 32);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * u + 2 * k], v[8 * u + 2 * k + 1]);
        w[k] = *reinterpret_cast<const uint32_t*>(&h);
      }
      d[u] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1) agGemmPairKernel(const __grid_constant__ Params P) {
  extern __shared__ uint8_t smemRaw[];
  const cocclkTpArgs& a = P.a;
  const int e = blockIdx.y;
  const int rank = a.rankBase + e;
  const int N = a.nRanks;
  const CUtensorMap* tmGather = &P.maps[e][0];
  const CUtensorMap* tmLocal = &P.maps[e][1];
  const CUtensorMap* tmB = &P.maps[e][2];
  Pipe p = pipeSetup<kAgStages, false>(smemRaw, tmGather, tmLocal, tmB);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int clusterId = blockIdx.x >> 1, numClusters = gridDim.x >> 1;
  const int rowsPerShard = a.M / N;
  const int tps = rowsPerShard / (2 * BM);  // 256-row tiles per shard
  const int numN = (a.N + BN - 1) / BN;
  const int tilesPerShard = tps * numN;
  const int numTiles = tilesPerShard * N;
  const int kBlocks = (a.K + BK - 1) / BK;
  const int pieces = P.pieces;
  StatusWord* st = reinterpret_cast<StatusWord*>(a.status[rank]);

  if (warp == 0) {
    // The whole warp walks the tiles: the flags of a remote tile are polled by all lanes at once (one acquire load
    // over the fabric takes about a microsecond; 32 of them in sequence would cost as much as the tile's main loop),
    // the copies are issued by lane 0.
    uint32_t it = 0;
    bool ok = true;
    for (int t = clusterId; t < numTiles && ok; t += numClusters) {
      int step, tmL, tn;
      agTile(t, tilesPerShard, tps, numN, step, tmL, tn);
      const int shard = (rank + step) % N;
      const int rowInShard = tmL * 2 * BM + (int)p.cta * BM;
      if (step > 0) {
        // this CTA's 128 rows of a remote shard: every piece of their eight 16-row parts must have landed
        // (FP8 payload: the flags the local push warps raise after dequantising a piece)
        const unsigned int* f = a.flags[rank] + (long)((a.agPayload ? kReadyRegion : 0) + shard) * kFlagStride +
                                (long)(rowInShard / kPartRows) * pieces;
        const int nFlags = (BM / kPartRows) * pieces;
        bool got = true;
        for (int i = lane; i < nFlags; i += 32) {
          if (*p.abortFlag || !waitFlag(f + i, a.epoch, a.timeoutNs)) {
            reportTimeout(st, 4, shard, tmL);
            got = false;
          }
        }
        ok = __all_sync(0xffffffffu, got) != 0;
        if (!ok) { if (lane == 0) raiseAbort(p); break; }
      }
      if (lane == 0) {
        if (step > 0) fenceProxyAsyncGlobal();  // peer stores (generic proxy) -> TMA reads (async proxy)
        const CUtensorMap* tmA = step == 0 ? tmLocal : tmGather;
        const int arow = step == 0 ? rowInShard : shard * rowsPerShard + rowInShard;
        const int n0 = tn * BN + (int)p.cta * BNH;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const int s = it % kAgStages;
          const uint32_t ph = (it / kAgStages) & 1;
          if (!mbarWait(&p.bars->empty[s], ph ^ 1, p.abortFlag, kPipeWaitNs)) { ok = false; raiseAbort(p); break; }
          if (*p.abortFlag) { ok = false; break; }
          loadStage(p, s, tmA, tmB, kb, arow, n0, a.bMN != 0);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    if (!ok && lane == 0) drainWait();
    __syncwarp();
  } else if (warp == 1) {
    if (p.cta == 0 && lane == 0) mmaRole<kAgStages>(p, clusterId, numTiles, numClusters, kBlocks, a.bMN != 0);
  } else if (warp < 6) {
    GemmArgs g;
    g.C = a.c[rank]; g.Z = a.z[rank]; g.bias = a.bias[rank]; g.M = a.M; g.N = a.N; g.K = a.K; g.ldc = a.N;
    g.epi = a.epi; g.aMN = 0; g.bMN = 0; g.err = nullptr; g.stages = kAgStages;
    const int quad = warp & 3;
    uint32_t tileIdx = 0;
    for (int t = clusterId; t < numTiles; t += numClusters, ++tileIdx) {
      int step, tmL, tn;
      agTile(t, tilesPerShard, tps, numN, step, tmL, tn);
      const int shard = (rank + step) % N;
      const int acc = tileIdx & 1;
      const uint32_t accPhase = (tileIdx >> 1) & 1;
      bool ok = mbarWait(&p.bars->tmemFull[acc], accPhase, p.abortFlag, kPipeWaitNs);
      ok = __all_sync(0xffffffffu, ok) != 0;
      if (!ok) { if (lane == 0) raiseAbort(p); break; }
      tcFenceAfter();
      const int row = shard * rowsPerShard + tmL * 2 * BM + (int)p.cta * BM + quad * 32 + lane;
      const uint32_t tbase = p.tmemBase + acc * BN + ((uint32_t)(quad * 32) << 16);
      epilogueStoreTile(g, tbase, row, tn * BN);
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArriveRemote(mapToCta(smemAddr(&p.bars->tmemEmpty[acc]), 0));
    }
  } else {
    // ---------------- gather push, ring order: everything for rank-1, then rank-2, ... ----------------
    const int cw = blockIdx.x * 2 + (warp - 6), W = gridDim.x * 2;
    const int pieceCols = a.K / pieces;
    const int pcv = pieceCols / 8;                     // 16-byte vectors per row of a piece
    const long rowVecs = a.K / 8;
    const long items = (long)(rowsPerShard / kPartRows) * pieces;
    const uint4* src0 = reinterpret_cast<const uint4*>(a.a[rank]);
    const bool fp8 = a.agPayload != 0;
    const long K = a.K;
    const int blocks = pieceCols / 32;                  // 32-column scale blocks per row of a piece (FP8 payload)
    bool pushAlive = true;
    for (int step = 1; step < N && pushAlive; ++step) {
      const int peer = (rank - step + N) % N;        // the peer whose ring step `step` reads this shard
      uint4* dst0 = reinterpret_cast<uint4*>(a.ws[peer]) + (long)rank * rowsPerShard * rowVecs;
      unsigned int* pf = a.flags[peer] + (long)rank * kFlagStride;
      uint8_t* peer8 = reinterpret_cast<uint8_t*>(a.ws[peer]) + ag8Offset(a.M, K) + (long)rank * rowsPerShard * K;
      uint8_t* peerScale = reinterpret_cast<uint8_t*>(a.ws[peer]) + agScaleOffset(a.M, K) + (long)rank * rowsPerShard * (K / 32);
      for (long itx = cw; itx < items; itx += W) {
        const long part = itx / pieces;
        const int piece = (int)(itx - part * pieces);
        if (fp8) {
          const long row0 = part * kPartRows, col0 = (long)piece * pieceCols;
          quantPiece(reinterpret_cast<const __nv_bfloat16*>(a.a[rank]) + row0 * K + col0, peer8 + row0 * K + col0,
                     peerScale + row0 * (K / 32) + col0 / 32, K, blocks, lane);
        } else {
          const long base = part * kPartRows * rowVecs + (long)piece * pcv;
          copyPiece<false>(src0, dst0, base, rowVecs, pcv, lane);
        }
        __syncwarp();
        if (lane == 0) {
          __threadfence_system();
          stReleaseSys(pf + itx, a.epoch);
        }
      }
      if (!fp8) continue;
      // the same ring step seen from the receiving side: the shard of rank+step lands here piece by piece
      const int shard = (rank + step) % N;
      const unsigned int* arrived = a.flags[rank] + (long)shard * kFlagStride;
      unsigned int* ready = a.flags[rank] + (long)(kReadyRegion + shard) * kFlagStride;
      const uint8_t* my8 = reinterpret_cast<const uint8_t*>(a.ws[rank]) + ag8Offset(a.M, K) + (long)shard * rowsPerShard * K;
      const uint8_t* myScale = reinterpret_cast<const uint8_t*>(a.ws[rank]) + agScaleOffset(a.M, K) + (long)shard * rowsPerShard * (K / 32);
      __nv_bfloat16* myRows = reinterpret_cast<__nv_bfloat16*>(a.ws[rank]) + (long)shard * rowsPerShard * K;
      for (long itx = cw; itx < items; itx += W) {
        bool got = true;
        if (lane == 0) {
          got = !*p.abortFlag && waitFlag(arrived + itx, a.epoch, a.timeoutNs);
          if (!got) { reportTimeout(st, 5, shard, (int)itx); raiseAbort(p); }
        }
        pushAlive = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (!pushAlive) break;
        const long part = itx / pieces;
        const int piece = (int)(itx - part * pieces);
        const long row0 = part * kPartRows, col0 = (long)piece * pieceCols;
        dequantPiece(my8 + row0 * K + col0, myScale + row0 * (K / 32) + col0 / 32, myRows + row0 * K + col0, K, blocks, lane);
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          stReleaseSys(ready + itx, a.epoch);
        }
      }
    }
    // ---------------- optional copy-out of the whole gathered operand (kept for the weight gradient) ----------------
    // own shard from the input, remote shards from the gather buffer as their pieces arrive (ring order again)
    uint4* keep = reinterpret_cast<uint4*>(a.gathered[rank]);
    if (keep != nullptr) {
      const uint4* wsLocal = reinterpret_cast<const uint4*>(a.ws[rank]);
      bool alive = pushAlive;
      for (int step = 0; step < N && alive; ++step) {
        const int shard = (rank + step) % N;
        const uint4* from = step == 0 ? src0 : wsLocal + (long)shard * rowsPerShard * rowVecs;
        uint4* to = keep + (long)shard * rowsPerShard * rowVecs;
        const unsigned int* f = a.flags[rank] + (long)((fp8 ? kReadyRegion : 0) + shard) * kFlagStride;
        for (long itx = cw; itx < items && alive; itx += W) {
          if (step > 0) {
            bool got = true;
            if (lane == 0) got = !*p.abortFlag && waitFlag(f + itx, a.epoch, a.timeoutNs);
            alive = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;  // the producer reports the missing piece
            if (!alive) break;
          }
          const long part = itx / pieces;
          const int piece = (int)(itx - part * pieces);
          const long base = part * kPartRows * rowVecs + (long)piece * pcv;
          if (step == 0) copyPiece<false>(from, to, base, rowVecs, pcv, lane);
          else copyPiece<true>(from, to, base, rowVecs, pcv, lane);
        }
      }
    }
  }
  pipeTeardown(p, a.err[rank], 0x80000005u);
}

// ---------------------------------------------------------------------------------------------
// GEMM -> FP8-compressed reduce-scatter, the reduction folded into the epilogue of the own rows
// ---------------------------------------------------------------------------------------------
// Receive slot of one source rank: [rowsPerRank][N] E4M3 bytes, then [rowsPerRank][N/32] UE8M0 scale bytes.
__host__ __device__ inline long rsSlotBytes(int rowsPerRank, int N) {
  return alignUp((long)rowsPerRank * N + (long)rowsPerRank * (N / 32), 256);
}

__global__ void __launch_bounds__(kThreads, 1) gemmRsPairKernel(const __grid_constant__ Params P) {
  extern __shared__ uint8_t smemRaw[];
  const cocclkTpArgs& a = P.a;
  const int e = blockIdx.y;
  const int rank = a.rankBase + e;
  const int N = a.nRanks;
  const CUtensorMap* tmA = &P.maps[e][0];
  const CUtensorMap* tmB = &P.maps[e][2];
  Pipe p = pipeSetup<kRsStages, true>(smemRaw, tmA, tmA, tmB);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int clusterId = blockIdx.x >> 1, numClusters = gridDim.x >> 1;
  const int rowsPerRank = a.M / N;
  const int tps = rowsPerRank / (2 * BM);
  const int numN = a.N / BN;
  const int tilesPerDest = tps * numN;
  const int numTiles = tilesPerDest * N;
  const int kBlocks = (a.K + BK - 1) / BK;
  const long slotBytes = rsSlotBytes(rowsPerRank, a.N);
  const long payloadBytes = (long)rowsPerRank * a.N;
  const int scalesPerRow = a.N / 32;
  StatusWord* st = reinterpret_cast<StatusWord*>(a.status[rank]);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = clusterId; t < numTiles && ok; t += numClusters) {
        const int step = t / tilesPerDest, r = t - step * tilesPerDest;
        const int tmL = r % tps, tn = r / tps;
        const int dest = (rank + 1 + step) % N;  // own rows last
        const int arow = dest * rowsPerRank + tmL * 2 * BM + (int)p.cta * BM;
        const int n0 = tn * BN + (int)p.cta * BNH;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const int s = it % kRsStages;
          const uint32_t ph = (it / kRsStages) & 1;
          if (!mbarWait(&p.bars->empty[s], ph ^ 1, p.abortFlag, kPipeWaitNs)) { ok = false; raiseAbort(p); break; }
          if (*p.abortFlag) { ok = false; break; }
          loadStage(p, s, tmA, tmB, kb, arow, n0, a.bMN != 0);
        }
      }
      if (!ok) drainWait();
    }
  } else if (warp == 1) {
    if (p.cta == 0 && lane == 0) mmaRole<kRsStages>(p, clusterId, numTiles, numClusters, kBlocks, a.bMN != 0);
  } else if (warp < 6) {
    const int quad = warp & 3;
    uint8_t* stage = p.epiStage + quad * (32 * kStageRowBytes);
    CodecCfg dummy{};
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.c[rank]);
    const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(a.bias[rank]);
    const uint8_t* myWs = reinterpret_cast<const uint8_t*>(a.ws[rank]);
    uint32_t tileIdx = 0;
    for (int t = clusterId; t < numTiles; t += numClusters, ++tileIdx) {
      const int step = t / tilesPerDest, r = t - step * tilesPerDest;
      const int tmL = r % tps, tn = r / tps;
      const int dest = (rank + 1 + step) % N;
      const int acc = tileIdx & 1;
      const uint32_t accPhase = (tileIdx >> 1) & 1;
      bool ok = mbarWait(&p.bars->tmemFull[acc], accPhase, p.abortFlag, kPipeWaitNs);
      ok = __all_sync(0xffffffffu, ok) != 0;
      if (!ok) { if (lane == 0) raiseAbort(p); break; }
      tcFenceAfter();
      const uint32_t tbase = p.tmemBase + acc * BN + ((uint32_t)(quad * 32) << 16);
      const int rowInDest0 = tmL * 2 * BM + (int)p.cta * BM + quad * 32;  // first row of this warp inside the destination's rows
      const int flagIdx = ((tmL * numN + tn) * 2 + (int)p.cta) * 4 + quad;
      if (dest != rank) {
        // ---------------- foreign rows: quantise, stage, push into the destination's slot ----------------
        uint8_t* slot = reinterpret_cast<uint8_t*>(a.ws[dest]) + (long)rank * slotBytes;
        uint32_t scaleLo = 0, scaleHi = 0;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t rr[32];
            tmemLd32x32(tbase + (half * 4 + c) * 32, rr);
            tmemLdWait();
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rr[i]);
            const MxFp8Codec::Enc enc = MxFp8Codec::encode(v, dummy, false, nullptr, 0);
            uint4* sp = reinterpret_cast<uint4*>(stage + lane * kStageRowBytes + c * 32);
            sp[0] = make_uint4(enc.w[0], enc.w[1], enc.w[2], enc.w[3]);
            sp[1] = make_uint4(enc.w[4], enc.w[5], enc.w[6], enc.w[7]);
            if (half == 0) scaleLo |= enc.scaleByte << (8 * c);
            else scaleHi |= enc.scaleByte << (8 * c);
          }
          __syncwarp();
          // 32 rows x 128 bytes leave as 8 warp-wide stores of 4 full rows each
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int row = k * 4 + (lane >> 3), piece = lane & 7;
            const uint4 x = *reinterpret_cast<const uint4*>(stage + row * kStageRowBytes + piece * 16);
            uint8_t* dst = slot + (long)(rowInDest0 + row) * a.N + tn * BN + half * 128 + piece * 16;
            *reinterpret_cast<uint4*>(dst) = x;
          }
          __syncwarp();
        }
        // the accumulator is drained: hand it back before the flag round trip over the link
        tcFenceBefore();
        __syncwarp();
        if (lane == 0) mbarArriveRemote(mapToCta(smemAddr(&p.bars->tmemEmpty[acc]), 0));
        uint8_t* sc = slot + payloadBytes + (long)(rowInDest0 + lane) * scalesPerRow + tn * (BN / 32);
        *reinterpret_cast<uint2*>(sc) = make_uint2(scaleLo, scaleHi);
        __syncwarp();
        if (lane == 0) {
          __threadfence_system();
          stReleaseSys(a.flags[dest] + (long)rank * kFlagStride + flagIdx, a.epoch);
        }
      } else {
        // ---------------- own rows: the epilogue is the reducer ----------------
        bool got = true;
        if (lane < N - 1) {
          const int src = (rank + 1 + lane) % N;
          got = waitFlag(a.flags[rank] + (long)src * kFlagStride + flagIdx, a.epoch, a.timeoutNs);
          if (!got) reportTimeout(st, 5, src, tmL * numN + tn);
        }
        got = __all_sync(0xffffffffu, got) != 0;
        if (!got) { if (lane == 0) raiseAbort(p); break; }
        const int row = rowInDest0 + lane;
        const long pbase = (long)row * a.N + tn * BN;
        const long sbase = payloadBytes + (long)row * scalesPerRow + tn * (BN / 32);
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t rr[32];
          tmemLd32x32(tbase + c * 32, rr);
          tmemLdWait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rr[i]);
          for (int q = 1; q < N; q += 2) {
            MxFp8Codec::Raw raw[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              raw[u].valid = q + u < N;
              if (raw[u].valid) {
                const uint8_t* sl = myWs + (long)((rank + q + u) % N) * slotBytes;
                const uint4 x0 = __ldcg(reinterpret_cast<const uint4*>(sl + pbase + c * 32));
                const uint4 x1 = __ldcg(reinterpret_cast<const uint4*>(sl + pbase + c * 32) + 1);
                raw[u].w[0] = x0.x; raw[u].w[1] = x0.y; raw[u].w[2] = x0.z; raw[u].w[3] = x0.w;
                raw[u].w[4] = x1.x; raw[u].w[5] = x1.y; raw[u].w[6] = x1.z; raw[u].w[7] = x1.w;
                raw[u].biased = __ldcg(sl + sbase + c);
              }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) MxFp8Codec::accumulate(raw[u], v);
          }
          if (bias != nullptr) {  // added once, to the reduced sum
            const uint4* bp = reinterpret_cast<const uint4*>(bias + tn * BN + c * 32);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint4 bw = __ldg(bp + k);
              const uint32_t w[4] = {bw.x, bw.y, bw.z, bw.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                v[8 * k + 2 * i] += __uint_as_float(w[i] << 16);
                v[8 * k + 2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
              }
            }
          }
          uint4* op = reinterpret_cast<uint4*>(out + (long)row * a.N + tn * BN + c * 32);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * k + 2 * i], v[8 * k + 2 * i + 1]);
              w[i] = *reinterpret_cast<uint32_t*>(&h);
            }
            op[k] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        tcFenceBefore();
        __syncwarp();
        if (lane == 0) mbarArriveRemote(mapToCta(smemAddr(&p.bars->tmemEmpty[acc]), 0));
      }
    }
  }
  pipeTeardown(p, a.err[rank], 0x80000006u);
}

// -------------------------------------------------------------------------------------------- launch
static int gMaxClusters = 0;

template <class Kern>
static int prepare(Kern kern, int smem) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  if (gMaxClusters == 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    gMaxClusters = sms / 2;
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3((unsigned)(sms / 2) * 2, 1, 1);
    q.blockDim = dim3(kThreads, 1, 1);
    q.dynamicSmemBytes = (size_t)smem;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
    q.attrs = qa; q.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &q) == cudaSuccess && n > 0 && n < gMaxClusters) gMaxClusters = n;
    (void)cudaGetLastError();
  }
  return 0;
}

template <class Kern>
static int launch(Kern kern, int smem, Params& P, int emulatedRanks, int maxCtas, long tilesPerRank, cudaStream_t stream) {
  int rc = prepare(kern, smem);
  if (rc) return rc;
  long clusters = gMaxClusters / emulatedRanks;  // one CTA per SM; emulated ranks must all be resident at once
  if (maxCtas > 1 && maxCtas / 2 < clusters) clusters = maxCtas / 2;
  if (tilesPerRank < clusters) clusters = tilesPerRank;
  if (clusters < 1) return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)clusters * 2, (unsigned)emulatedRanks, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (emulatedRanks > 1) {
    // the emulated ranks wait on one another: ask the driver to guarantee that the whole grid is resident
    attr[1].id = cudaLaunchAttributeCooperative;
    attr[1].val.cooperative = 1;
    cfg.numAttrs = 2;
  }
  cocclkCountLaunches(1);
  return (int)cudaLaunchKernelEx(&cfg, kern, P);
}

}  // namespace tp2
}  // namespace coccl

using namespace coccl;
using namespace coccl::tp2;

// Whether the pair kernels take a problem (the callers in tp_kernels.cu fall back to the single-CTA kernels otherwise).
extern "C" int cocclkTpPairUsable(const cocclkTpArgs* a, int isRs) {
  if (a->nRanks < 2 || a->M % (a->nRanks * 2 * BM) != 0 || (a->K & 7)) return 0;
  const int rows = a->M / a->nRanks;
  if (isRs) return a->N % BN == 0 && (long)(rows / (2 * BM)) * (a->N / BN) * 8 <= kFlagStride;
  return (a->N & 7) == 0 && (long)(rows / kPartRows) <= kFlagStride;
}

static int agPieces(int rowsPerShard, int K, int payload) {
  // column pieces per 16-row part: finer pieces let the first tiles of a shard start earlier; a piece stays a
  // multiple of 16 bytes per row (of 32 columns with the FP8 payload: whole scale blocks), at least 256 columns wide,
  // and the flags of one source must fit its stride
  const int unit = payload ? 32 : 8;
  for (int pcs = 4; pcs > 1; pcs >>= 1)
    if (K % (pcs * unit) == 0 && K / pcs >= 256 && (long)(rowsPerShard / kPartRows) * pcs <= kFlagStride) return pcs;
  return 1;
}

extern "C" long cocclkAgGemmWorkspaceBytesFor(int M, int K, int agPayload) {
  if (!agPayload) return (long)M * K * 2;
  return agScaleOffset(M, K) + (((long)M * (K / 32) + 255) & ~255L);
}

extern "C" int cocclkAgGemmPair(const cocclkTpArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream) {
  const int N = args->nRanks, rowsPerShard = args->M / N;
  Params P;
  memcpy(&P.a, args, sizeof(cocclkTpArgs));
  if (args->agPayload && (args->K % 32) != 0) return -1;
  P.pieces = agPieces(rowsPerShard, args->K, args->agPayload);
  for (int e = 0; e < emulatedRanks; ++e) {
    const int r = args->rankBase + e;
    if ((args->epi != GEMM_EPI_NONE) && args->bias[r] == nullptr) return -1;
    int rc = makeBf16TensorMap(&P.maps[e][0], args->ws[r], args->K, args->M, args->K, BK, BM);
    if (rc) return rc;
    rc = makeBf16TensorMap(&P.maps[e][1], args->a[r], args->K, rowsPerShard, args->K, BK, BM);
    if (rc) return rc;
    rc = args->bMN ? makeBf16TensorMap(&P.maps[e][2], args->b[r], args->N, args->K, args->N, 64, 64)
                   : makeBf16TensorMap(&P.maps[e][2], args->b[r], args->K, args->N, args->K, BK, BNH);
    if (rc) return rc;
  }
  const long tiles = (long)(args->M / (2 * BM)) * ((args->N + BN - 1) / BN);
  return launch(agGemmPairKernel, smemBytes(kAgStages, false), P, emulatedRanks, maxCtas, tiles, stream);
}

extern "C" int cocclkGemmRsPair(const cocclkTpArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream) {
  Params P;
  memcpy(&P.a, args, sizeof(cocclkTpArgs));
  P.pieces = 1;
  for (int e = 0; e < emulatedRanks; ++e) {
    const int r = args->rankBase + e;
    int rc = makeBf16TensorMap(&P.maps[e][0], args->a[r], args->K, args->M, args->K, BK, BM);
    if (rc) return rc;
    P.maps[e][1] = P.maps[e][0];
    rc = args->bMN ? makeBf16TensorMap(&P.maps[e][2], args->b[r], args->N, args->K, args->N, 64, 64)
                   : makeBf16TensorMap(&P.maps[e][2], args->b[r], args->K, args->N, args->K, BK, BNH);
    if (rc) return rc;
  }
  const long tiles = (long)(args->M / (2 * BM)) * (args->N / BN);
  return launch(gemmRsPairKernel, smemBytes(kRsStages, true), P, emulatedRanks, maxCtas, tiles, stream);
}
