// Tensor-parallel fusions on sm_100a: one persistent tcgen05 kernel per operation, with the collective
// inside the kernel.
//
//  agGemmKernel  C = gather(A) * B^T. Two spare warps of every CTA copy the local activation shard into the
//                peers' gather buffers (plain peer stores, 16-row parts, one release flag per part) while the
//                tensor cores already work on the local shard; the TMA producer waits for the flags of a
//                remote shard's rows right before it loads them (from LOCAL memory, no multicast). Shards are
//                visited in ring order, so at every step each GPU sends to one peer and receives from one.
//  gemmRsKernel  out = reduce_scatter(A * B^T). The epilogue quantises every fp32 accumulator row segment to
//                E4M3 with one UE8M0 scale per 32 columns (a thread holds exactly one block per tcgen05.ld),
//                stages it in shared memory and pushes it with coalesced peer stores into the destination
//                rank's slot; tiles of the next rank in the ring are computed first, own rows last. When its
//                tiles are done a CTA turns into a reducer: it waits for the tile flags of all sources, sums the
//                dequantised copies and writes bf16.
//
// Pipeline (both): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5 epilogue, 128x256x64 tiles,
// 4 stages, two TMEM accumulators. `rankBase`/blockIdx.y let one cooperative launch play all ranks on one
// GPU for tests. Every wait is bounded and reports through the status / error words.
#include "codecs.cuh"
#include "gemm_epilogue.cuh"
#include "launch_count.h"
#include "tp_api.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace coccl {
using namespace sm100;

namespace tp {
constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BN * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 256;       // gemmRsKernel: producer, MMA, 4 epilogue warps, 2 spare
constexpr int kAgThreads = 384;     // upper bound of the block size of agGemmKernel (push warps = warps beyond the sixth)
constexpr int kParts = 8;                 // flag granularity of the gather: 16 rows
constexpr int kPartRows = BM / kParts;
constexpr int kFlagStride = 4096;         // flags per source rank
constexpr int kStageRowBytes = 128 + 16;  // epilogue staging row (half a tile row of fp8 + padding)
constexpr int kEpiStageBytes = 4 * 32 * kStageRowBytes;
constexpr unsigned long long kPipeWaitNs = 4000000000ull;

struct __align__(8) Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmemFull[2];
  uint64_t tmemEmpty[2];
  uint32_t tmemBase;
  int abortFlag;
};

struct Params {
  cocclkTpArgs a;
  CUtensorMap maps[COCCLK_TP_MAX_EMULATED][3];  // [emulated rank][A remote/full, A local, B]
};

constexpr int kSmemBytes = kStages * kStageBytes + kEpiStageBytes + (int)sizeof(Barriers) + 1024;

__device__ __forceinline__ void fenceProxyAsync() { asm volatile("fence.proxy.async;" ::: "memory"); }

struct Pipe {
  uint8_t* smem;
  Barriers* bars;
  volatile int* abortFlag;
  uint32_t tmemBase;
};

__device__ __forceinline__ Pipe pipeSetup(uint8_t* smemRaw, const CUtensorMap* m0, const CUtensorMap* m1,
                                          const CUtensorMap* m2) {
  Pipe p;
  p.smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  p.bars = reinterpret_cast<Barriers*>(p.smem + kStages * kStageBytes + kEpiStageBytes);
  p.abortFlag = &p.bars->abortFlag;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbarInit(&p.bars->full[s], 1); mbarInit(&p.bars->empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbarInit(&p.bars->tmemFull[i], 1); mbarInit(&p.bars->tmemEmpty[i], 4); }
    p.bars->abortFlag = 0;
    mbarFenceInit();
    prefetchTensorMap(m0);
    prefetchTensorMap(m1);
    prefetchTensorMap(m2);
  }
  if (warp == 1) {
    tmemAlloc(&p.bars->tmemBase, 512);
    tmemRelinquish();
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  p.tmemBase = p.bars->tmemBase;
  return p;
}

__device__ __forceinline__ void pipeTeardown(const Pipe& p, unsigned int* err, unsigned int code) {
  tcFenceBefore();
  __syncthreads();
  if ((threadIdx.x >> 5) == 1) {
    tcFenceAfter();
    tmemDealloc(p.tmemBase, 512);
  }
  if (threadIdx.x == 0 && p.bars->abortFlag && err) atomicExch(err, code);
}

// B tile of one stage: 256 weight rows x 64 k (K-major), or four 64-column x 64-k boxes (stored [K, N])
__device__ __forceinline__ void loadB(uint8_t* sb, const CUtensorMap* tmB, uint64_t* bar, int kb, int tn, bool bMN) {
  if (!bMN) {
    tmaLoad2d(sb, tmB, bar, kb * BK, tn * BN);
  } else {
    for (int i = 0; i < BN / 64; ++i) tmaLoad2d(sb + i * 8192, tmB, bar, tn * BN + i * 64, kb * BK);
  }
}

// give copies already issued a bounded time to land before the CTA may leave
__device__ __forceinline__ void drainProducer(const Pipe& p, uint32_t it) {
  for (uint32_t back = 1; back <= (uint32_t)kStages && back <= it; ++back) {
    const uint32_t j = it - back;
    const unsigned long long start = gtimer();
    while (!mbarTryWait(&p.bars->full[j % kStages], (j / kStages) & 1)) {
      if (gtimer() - start > 100000000ull) break;
    }
  }
}

// MMA issuer: identical for both kernels (K-major operands).
__device__ __forceinline__ void mmaRole(const Pipe& p, int numTiles, int kBlocks, bool bMN) {
  const uint32_t idesc = makeInstrDescBf16(BM, BN, false, bMN);
  uint32_t it = 0, tileIdx = 0;
  bool ok = true;
  for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++tileIdx) {
    const int acc = tileIdx & 1;
    const uint32_t accPhase = (tileIdx >> 1) & 1;
    if (!mbarWait(&p.bars->tmemEmpty[acc], accPhase ^ 1, p.abortFlag, kPipeWaitNs)) { ok = false; break; }
    tcFenceAfter();
    const uint32_t dTmem = p.tmemBase + acc * BN;
    for (int kb = 0; kb < kBlocks; ++kb, ++it) {
      const int s = it % kStages;
      const uint32_t ph = (it / kStages) & 1;
      if (!mbarWait(&p.bars->full[s], ph, p.abortFlag, kPipeWaitNs)) { ok = false; break; }
      tcFenceAfter();
      const uint32_t sa = smemAddr(p.smem + s * kStageBytes);
      const uint32_t sb = sa + kABytes;
#pragma unroll
      for (int k = 0; k < BK / 16; ++k) {
        const uint64_t db = bMN ? makeSmemDesc(sb + k * 2048, 8192, 1024) : makeSmemDesc(sb + k * 32, 16, 1024);
        umma(dTmem, makeSmemDesc(sa + k * 32, 16, 1024), db, idesc, (kb | k) != 0 ? 1u : 0u);
      }
      ummaCommit(&p.bars->empty[s]);
      if (kb == kBlocks - 1) ummaCommit(&p.bars->tmemFull[acc]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// all-gather -> GEMM
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kAgThreads, 1) agGemmKernel(const __grid_constant__ Params P) {
  extern __shared__ uint8_t smemRaw[];
  const cocclkTpArgs& a = P.a;
  const int e = blockIdx.y;
  const int rank = a.rankBase + e;
  const int N = a.nRanks;
  const CUtensorMap* tmGather = &P.maps[e][0];
  const CUtensorMap* tmLocal = &P.maps[e][1];
  const CUtensorMap* tmB = &P.maps[e][2];
  Pipe p = pipeSetup(smemRaw, tmGather, tmLocal, tmB);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rowsPerShard = a.M / N;
  const int tps = rowsPerShard / BM;  // m-tiles per shard
  const int numN = (a.N + BN - 1) / BN;
  const int tilesPerShard = tps * numN;
  const int numTiles = tilesPerShard * N;
  const int kBlocks = (a.K + BK - 1) / BK;
  StatusWord* st = reinterpret_cast<StatusWord*>(a.status[rank]);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
        const int step = t / tilesPerShard, r = t - step * tilesPerShard;
        const int tmL = r % tps, tn = r / tps;
        const int shard = (rank + step) % N;
        if (step > 0) {
          // rows of a remote shard: all 16-row parts of this m-tile must have landed in the gather buffer
          const unsigned int* f = a.flags[rank] + (long)shard * kFlagStride + tmL * kParts;
          for (int part = 0; part < kParts && ok; ++part) {
            if (*p.abortFlag || !waitFlag(f + part, a.epoch, a.timeoutNs)) {
              reportTimeout(st, 4, shard, tmL);
              *p.abortFlag = 1;
              ok = false;
            }
          }
          if (!ok) break;
          fenceProxyAsync();  // peer stores (generic proxy) -> TMA reads (async proxy)
        }
        const CUtensorMap* tmA = step == 0 ? tmLocal : tmGather;
        const int arow = step == 0 ? tmL * BM : shard * rowsPerShard + tmL * BM;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbarWait(&p.bars->empty[s], ph ^ 1, p.abortFlag, kPipeWaitNs)) { ok = false; break; }
          uint8_t* sa = p.smem + s * kStageBytes;
          mbarArriveExpectTx(&p.bars->full[s], kStageBytes);
          tmaLoad2d(sa, tmA, &p.bars->full[s], kb * BK, arow);
          loadB(sa + kABytes, tmB, &p.bars->full[s], kb, tn, a.bMN != 0);
        }
      }
      if (!ok) drainProducer(p, it);
    }
  } else if (warp == 1) {
    if (lane == 0) mmaRole(p, numTiles, kBlocks, a.bMN != 0);
  } else if (warp < 6) {
    GemmArgs g;
    g.C = a.c[rank]; g.Z = a.z[rank]; g.bias = a.bias[rank]; g.M = a.M; g.N = a.N; g.K = a.K; g.ldc = a.N;
    g.epi = a.epi; g.aMN = 0; g.bMN = 0; g.err = nullptr;
    const int quad = warp & 3;
    uint32_t tileIdx = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++tileIdx) {
      const int step = t / tilesPerShard, r = t - step * tilesPerShard;
      const int tmL = r % tps, tn = r / tps;
      const int shard = (rank + step) % N;
      const int acc = tileIdx & 1;
      const uint32_t accPhase = (tileIdx >> 1) & 1;
      ok = mbarWait(&p.bars->tmemFull[acc], accPhase, p.abortFlag, kPipeWaitNs);
      ok = __all_sync(0xffffffffu, ok) != 0;
      if (!ok) break;
      tcFenceAfter();
      const int row = shard * rowsPerShard + tmL * BM + quad * 32 + lane;
      const uint32_t tbase = p.tmemBase + acc * BN + ((uint32_t)(quad * 32) << 16);
      epilogueStoreTile(g, tbase, row, tn * BN);
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArrive(&p.bars->tmemEmpty[acc]);
    }
  } else {
    // ---------------- gather push: this rank's shard -> every peer's gather buffer ----------------
    // two push warps per CTA: six were measured slower at 2 and at 8 ranks (the copy is not limited by issue slots)
    const int commWarps = (int)(blockDim.x >> 5) - 6;
    const int cw = blockIdx.x * commWarps + (warp - 6), W = gridDim.x * commWarps;
    const long items = (long)(N - 1) * tps * kParts;
    const long partVecs = (long)kPartRows * a.K * 2 / 16;  // uint4 per 16-row part
    const uint4* src0 = reinterpret_cast<const uint4*>(a.a[rank]);
    for (long itx = cw; itx < items; itx += W) {
      const int step = 1 + (int)(itx / (tps * kParts));
      const int r = (int)(itx % (tps * kParts));
      const int peer = (rank - step + N) % N;  // the peer that needs this shard at ring step `step`
      const uint4* src = src0 + (long)r * partVecs;
      uint4* dst = reinterpret_cast<uint4*>(a.ws[peer]) + ((long)rank * tps * kParts + r) * partVecs;
      long j = lane;
      for (; j + 7 * 32 < partVecs; j += 8 * 32) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldg(src + j + u * 32);
#pragma unroll
        for (int u = 0; u < 8; ++u) dst[j + u * 32] = v[u];
      }
      for (; j < partVecs; j += 32) dst[j] = __ldg(src + j);
      __syncwarp();
      if (lane == 0) {
        __threadfence_system();
        stReleaseSys(a.flags[peer] + (long)rank * kFlagStride + r, a.epoch);
      }
    }
  }
  pipeTeardown(p, a.err[rank], 0x80000003u);
}

// ---------------------------------------------------------------------------------------------
// GEMM -> FP8-compressed reduce-scatter
// ---------------------------------------------------------------------------------------------
// Receive slot of one source rank: [rowsPerRank][N] E4M3 bytes, then [rowsPerRank][N/32] UE8M0 scale bytes.
__host__ __device__ inline long rsSlotBytes(int rowsPerRank, int N) {
  return alignUp((long)rowsPerRank * N + (long)rowsPerRank * (N / 32), 256);
}

__global__ void __launch_bounds__(kThreads, 1) gemmRsKernel(const __grid_constant__ Params P) {
  extern __shared__ uint8_t smemRaw[];
  const cocclkTpArgs& a = P.a;
  const int e = blockIdx.y;
  const int rank = a.rankBase + e;
  const int N = a.nRanks;
  const CUtensorMap* tmA = &P.maps[e][0];
  const CUtensorMap* tmB = &P.maps[e][2];
  Pipe p = pipeSetup(smemRaw, tmA, tmA, tmB);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rowsPerRank = a.M / N;
  const int tps = rowsPerRank / BM;
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
      for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
        const int step = t / tilesPerDest, r = t - step * tilesPerDest;
        const int tmL = r % tps, tn = r / tps;
        const int dest = (rank + 1 + step) % N;  // own rows last
        const int arow = dest * rowsPerRank + tmL * BM;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbarWait(&p.bars->empty[s], ph ^ 1, p.abortFlag, kPipeWaitNs)) { ok = false; break; }
          uint8_t* sa = p.smem + s * kStageBytes;
          mbarArriveExpectTx(&p.bars->full[s], kStageBytes);
          tmaLoad2d(sa, tmA, &p.bars->full[s], kb * BK, arow);
          loadB(sa + kABytes, tmB, &p.bars->full[s], kb, tn, a.bMN != 0);
        }
      }
      if (!ok) drainProducer(p, it);
    }
  } else if (warp == 1) {
    if (lane == 0) mmaRole(p, numTiles, kBlocks, a.bMN != 0);
  } else if (warp < 6) {
    // ---------------- epilogue: quantise, stage, push to the destination's slot ----------------
    const int quad = warp & 3;
    uint8_t* stage = p.smem + kStages * kStageBytes + quad * (32 * kStageRowBytes);
    CodecCfg dummy{};
    uint32_t tileIdx = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++tileIdx) {
      const int step = t / tilesPerDest, r = t - step * tilesPerDest;
      const int tmL = r % tps, tn = r / tps;
      const int dest = (rank + 1 + step) % N;
      const int acc = tileIdx & 1;
      const uint32_t accPhase = (tileIdx >> 1) & 1;
      ok = mbarWait(&p.bars->tmemFull[acc], accPhase, p.abortFlag, kPipeWaitNs);
      ok = __all_sync(0xffffffffu, ok) != 0;
      if (!ok) break;
      tcFenceAfter();
      const uint32_t tbase = p.tmemBase + acc * BN + ((uint32_t)(quad * 32) << 16);
      uint8_t* slot = reinterpret_cast<uint8_t*>(a.ws[dest]) + (long)rank * slotBytes;
      const int rowInDest0 = tmL * BM + quad * 32;  // first row of this warp inside the destination's rows
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
      // the accumulator is drained: hand it back before the (slow) flag round trip
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArrive(&p.bars->tmemEmpty[acc]);
      uint8_t* sc = slot + payloadBytes + (long)(rowInDest0 + lane) * scalesPerRow + tn * (BN / 32);
      *reinterpret_cast<uint2*>(sc) = make_uint2(scaleLo, scaleHi);
      // one flag per (tile, lane quadrant): no cross-warp barrier on a path that can be aborted
      __syncwarp();
      if (lane == 0) {
        __threadfence_system();
        stReleaseSys(a.flags[dest] + (long)rank * kFlagStride + (tmL * numN + tn) * 4 + quad, a.epoch);
      }
    }
  }
  tcFenceBefore();
  __syncthreads();

  // ---------------- reducer: sum the N dequantised copies of every tile of this rank's rows ----------------
  {
    __shared__ int sOk;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.c[rank]);
    const uint8_t* myWs = reinterpret_cast<const uint8_t*>(a.ws[rank]);
    bool failed = *p.abortFlag != 0;
    for (int it = blockIdx.x; it < tilesPerDest; it += gridDim.x) {
      const int tmL = it % tps, tn = it / tps;
      if (threadIdx.x == 0) sOk = 1;
      __syncthreads();
      if (!failed && threadIdx.x < 4 * N) {
        const int src = threadIdx.x >> 2, quad = threadIdx.x & 3;
        if (!waitFlag(a.flags[rank] + (long)src * kFlagStride + (tmL * numN + tn) * 4 + quad, a.epoch, a.timeoutNs)) {
          reportTimeout(st, 5, src, it);
          sOk = 0;
        }
      }
      __syncthreads();
      if (!sOk) failed = true;
      const int cb = threadIdx.x & 7, rbase = threadIdx.x >> 3;
#pragma unroll 1
      for (int j = 0; j < 4; ++j) {
        const int row = tmL * BM + rbase + 32 * j;
        const long poff = (long)row * a.N + tn * BN + cb * 32;
        const long soff = payloadBytes + (long)row * scalesPerRow + tn * (BN / 32) + cb;
        float acc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.f;
        for (int q = 0; q < N; q += 2) {
          MxFp8Codec::Raw raw[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            raw[u].valid = q + u < N;
            if (raw[u].valid) {
              const uint8_t* sl = myWs + (long)(q + u) * slotBytes;
              const uint4 x0 = __ldcg(reinterpret_cast<const uint4*>(sl + poff));
              const uint4 x1 = __ldcg(reinterpret_cast<const uint4*>(sl + poff) + 1);
              raw[u].w[0] = x0.x; raw[u].w[1] = x0.y; raw[u].w[2] = x0.z; raw[u].w[3] = x0.w;
              raw[u].w[4] = x1.x; raw[u].w[5] = x1.y; raw[u].w[6] = x1.z; raw[u].w[7] = x1.w;
              raw[u].biased = __ldcg(sl + soff);
            }
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) MxFp8Codec::accumulate(raw[u], acc);
        }
        uint4* op = reinterpret_cast<uint4*>(out + (long)row * a.N + tn * BN + cb * 32);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(acc[8 * k + 2 * i], acc[8 * k + 2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
          }
          op[k] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
  // TMEM and error word (the pipeline barrier above already ordered every tcgen05 access)
  if (warp == 1) {
    tcFenceAfter();
    tmemDealloc(p.tmemBase, 512);
  }
  if (threadIdx.x == 0 && p.bars->abortFlag && a.err[rank]) atomicExch(a.err[rank], 0x80000004u);
}

}  // namespace tp

int makeBf16TensorMap(CUtensorMap* m, const void* base, long inner, long outer, long ld, int boxInner, int boxOuter);

}  // namespace coccl

using namespace coccl;
using namespace coccl::tp;

extern "C" long cocclkAgGemmWorkspaceBytes(int M, int K) { return alignUp((long)M * K * 2, 256); }

extern "C" long cocclkGemmRsWorkspaceBytes(int M, int N, int nRanks) {
  if (nRanks <= 0) return 0;
  return rsSlotBytes(M / nRanks, N) * nRanks;
}

template <class Kern>
static int launchTp(Kern kern, int threads, Params& P, int emulatedRanks, int maxCtas, long tilesPerRank, cudaStream_t stream) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return (int)e;
  long cap = sms / emulatedRanks;  // one CTA per SM (shared memory); emulated ranks must be co-resident
  if (maxCtas > 0 && maxCtas < cap) cap = maxCtas;
  if (cap < 1) return -1;
  const int gx = (int)(tilesPerRank < cap ? tilesPerRank : cap);
  dim3 grid(gx, emulatedRanks, 1);
  void* params[] = {&P};
  cocclkCountLaunches(1);
  if (emulatedRanks > 1)
    return (int)cudaLaunchCooperativeKernel((const void*)kern, grid, dim3(threads), params, kSmemBytes, stream);
  return (int)cudaLaunchKernel((const void*)kern, grid, dim3(threads), params, kSmemBytes, stream);
}

static int checkCommon(const cocclkTpArgs* a, int emulatedRanks) {
  if (!a || a->nRanks < 1 || a->nRanks > COCCLK_TP_MAX_RANKS) return -1;
  if (emulatedRanks != 1 && (emulatedRanks != a->nRanks || emulatedRanks > COCCLK_TP_MAX_EMULATED || a->rankBase != 0)) return -1;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || (a->K & 7) || (a->N & 7)) return -1;
  if (a->M % (a->nRanks * BM) != 0) return -1;
  return 0;
}

// CTA-pair kernels (tp2_kernels.cu): taken whenever the shape allows it (rows per rank a multiple of 256).
extern "C" int cocclkTpPairUsable(const cocclkTpArgs* a, int isRs);
extern "C" int cocclkAgGemmPair(const cocclkTpArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream);
extern "C" int cocclkGemmRsPair(const cocclkTpArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream);

// 0 = pair kernels where the shape allows, 1 = always the single-CTA kernels, 2 = pair kernels or an error.
// The initial value comes from COCCL_TP_VARIANT ("1cta" / "2cta").
static int gTpVariant = -1;
extern "C" void cocclkTpSetVariant(int v) { gTpVariant = v; }
extern "C" int cocclkTpGetVariant() {
  if (gTpVariant < 0) {
    const char* e = getenv("COCCL_TP_VARIANT");
    gTpVariant = (e && !strcmp(e, "1cta")) ? 1 : (e && !strcmp(e, "2cta")) ? 2 : 0;
  }
  return gTpVariant;
}
// which kernel served the last call of this process: 1 = single CTA, 2 = pair
static int gTpLast = 0;
extern "C" int cocclkTpLastVariant() { return gTpLast; }

// Returns 1 when the pair kernel was launched (rc holds its result), 0 when the caller should use the single-CTA one.
static int tryPair(const cocclkTpArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream, int isRs, int* rc) {
  const int v = cocclkTpGetVariant();
  if (v == 1) return 0;
  // "auto": the CTA-pair kernels up to four ranks. At eight ranks (2048 rows per rank on the MLP shapes) they were
  // measured slower than the single-CTA kernels (all-gather GEMM 0.442 against 0.360 ms, reduce-scatter GEMM 0.457
  // against 0.361 ms): with seven ring steps the two push warps of 74 pairs cannot keep the next shard ahead of the
  // tensor cores, and the own-rows reducer waits for seven copies.
  if (v == 0 && args->nRanks > 4) return 0;
  if (!cocclkTpPairUsable(args, isRs)) {
    if (v == 2) { *rc = -1; return 1; }
    return 0;
  }
  *rc = isRs ? cocclkGemmRsPair(args, emulatedRanks, maxCtas, stream) : cocclkAgGemmPair(args, emulatedRanks, maxCtas, stream);
  if (*rc != 0 && emulatedRanks > 1 && v != 2) {
    // a cooperative launch of clusters is refused on some configurations: the emulation then runs on the single-CTA
    // kernels (a refused launch has not started anything)
    (void)cudaGetLastError();
    return 0;
  }
  gTpLast = 2;
  return 1;
}

extern "C" int cocclkAgGemm(const cocclkTpArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream) {
  if (checkCommon(args, emulatedRanks)) return -1;
  if ((args->epi == GEMM_EPI_BIAS || args->epi == GEMM_EPI_BIAS_GELU) == false && args->epi != GEMM_EPI_NONE) return -1;
  {
    int rc = 0;
    if (tryPair(args, emulatedRanks, maxCtas, stream, 0, &rc)) return rc;
    gTpLast = 1;
  }
  const int N = args->nRanks, rowsPerShard = args->M / N;
  if ((long)(rowsPerShard / BM) * kParts > kFlagStride) return -1;
  Params P;
  memcpy(&P.a, args, sizeof(cocclkTpArgs));
  for (int e = 0; e < emulatedRanks; ++e) {
    const int r = args->rankBase + e;
    if ((args->epi != GEMM_EPI_NONE) && args->bias[r] == nullptr) return -1;
    int rc = makeBf16TensorMap(&P.maps[e][0], args->ws[r], args->K, args->M, args->K, BK, BM);
    if (rc) return rc;
    rc = makeBf16TensorMap(&P.maps[e][1], args->a[r], args->K, rowsPerShard, args->K, BK, BM);
    if (rc) return rc;
    rc = args->bMN ? makeBf16TensorMap(&P.maps[e][2], args->b[r], args->N, args->K, args->N, 64, 64)
                   : makeBf16TensorMap(&P.maps[e][2], args->b[r], args->K, args->N, args->K, BK, BN);
    if (rc) return rc;
  }
  const long tiles = (long)(args->M / BM) * ((args->N + BN - 1) / BN);
  return launchTp(agGemmKernel, kThreads, P, emulatedRanks, maxCtas, tiles, stream);
}

extern "C" int cocclkGemmRs(const cocclkTpArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream) {
  if (checkCommon(args, emulatedRanks)) return -1;
  if (args->N % BN != 0) return -1;
  {
    int rc = 0;
    if (tryPair(args, emulatedRanks, maxCtas, stream, 1, &rc)) return rc;
    gTpLast = 1;
  }
  const int N = args->nRanks, rowsPerRank = args->M / N;
  if ((long)(rowsPerRank / BM) * (args->N / BN) * 4 > kFlagStride) return -1;
  Params P;
  memcpy(&P.a, args, sizeof(cocclkTpArgs));
  for (int e = 0; e < emulatedRanks; ++e) {
    const int r = args->rankBase + e;
    int rc = makeBf16TensorMap(&P.maps[e][0], args->a[r], args->K, args->M, args->K, BK, BM);
    if (rc) return rc;
    P.maps[e][1] = P.maps[e][0];
    rc = args->bMN ? makeBf16TensorMap(&P.maps[e][2], args->b[r], args->N, args->K, args->N, 64, 64)
                   : makeBf16TensorMap(&P.maps[e][2], args->b[r], args->K, args->N, args->K, BK, BN);
    if (rc) return rc;
  }
  const long tiles = (long)(args->M / BM) * (args->N / BN);
  return launchTp(gemmRsKernel, kThreads, P, emulatedRanks, maxCtas, tiles, stream);
}
