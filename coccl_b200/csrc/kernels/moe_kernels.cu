// Expert-parallel token exchange with the routing inside the kernels (see moe_api.h).
//
// Layout of a rank's workspace half (all offsets 256-byte aligned):
//   [dispatch payload]  nRanks x capacity rows of `hidden` E4M3 bytes, block (source rank, position)
//   [dispatch scales]   nRanks x capacity rows of hidden/32 UE8M0 bytes
//   [counts]            nRanks x localExperts ints, row s written by source rank s
//   [return rows]       nRanks x capacity rows of `hidden` bf16, block (expert rank, position)
// A source rank sorts its (token, choice) entries by expert (cocclkMoeLayout), so the rows it sends to one
// destination are grouped by local expert and the destination needs only the per-expert counts to place
// them; the same positions route the expert outputs back.
//
// One warp moves one row. Flags: one per (source rank, CTA) and direction, carrying the call's epoch; every
// wait is bounded and reports through the status word.
#include "codecs.cuh"
#include "launch_count.h"
#include "moe_api.h"

#include <string.h>

namespace coccl {
namespace moe {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kFlagStride = 4096;
constexpr int kMaxSeg = COCCLK_MOE_MAX_RANKS * COCCLK_MOE_MAX_LOCAL_EXPERTS;

struct Layout {
  long payloadOff, scalesOff, countsOff, retOff, total;
};
__host__ __device__ inline Layout makeLayout(int nRanks, int capacity, int hidden, int localExperts) {
  Layout L;
  L.payloadOff = 0;
  L.scalesOff = alignUp((long)nRanks * capacity * hidden, 256);
  L.countsOff = L.scalesOff + alignUp((long)nRanks * capacity * (hidden / 32), 256);
  L.retOff = L.countsOff + alignUp((long)nRanks * localExperts * 4, 256);
  L.total = L.retOff + alignUp((long)nRanks * capacity * hidden * 2, 256);
  return L;
}

// ------------------------------------------------------------------ routing layout
// Stable counting sort of the entries by expert: warp w owns a contiguous segment of entries; a first walk
// builds per-warp histograms, a scan turns them into bases, a second walk hands out the positions.
__global__ void __launch_bounds__(1024) moeLayoutKernel(const int* __restrict__ ids, int entries, int experts,
                                                        int expertsPerRank, int* __restrict__ pos, int* __restrict__ counts) {
  __shared__ int hist[32][COCCLK_MOE_MAX_EXPERTS];  // becomes the running base of (warp, expert)
  __shared__ int expertBase[COCCLK_MOE_MAX_EXPERTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * COCCLK_MOE_MAX_EXPERTS; i += blockDim.x) (&hist[0][0])[i] = 0;
  __syncthreads();
  const int seg = ((entries + 31) / 32 + 31) / 32 * 32;  // entries per warp, a multiple of 32
  const int begin = warp * seg, end = min(entries, begin + seg);
  for (int i = begin + lane; i - lane < end; i += 32) {
    const bool valid = i < end;
    const int e = valid ? ids[i] : -1;
    const unsigned act = __ballot_sync(0xffffffffu, valid);
    if (valid) {
      const unsigned same = __match_any_sync(act, e);
      if ((same & ((1u << lane) - 1)) == 0) hist[warp][e] += __popc(same);
    }
    __syncwarp();
  }
  __syncthreads();
  // totals per expert, then bases inside the destination rank's block
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < 32; ++w) { const int c = hist[w][e]; hist[w][e] = run; run += c; }
    counts[e] = run;
    expertBase[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int d = 0; d < experts / expertsPerRank; ++d) {
      int run = 0;
      for (int le = 0; le < expertsPerRank; ++le) {
        const int e = d * expertsPerRank + le;
        const int c = expertBase[e];
        expertBase[e] = run;
        run += c;
      }
    }
  }
  __syncthreads();
  for (int i = begin + lane; i - lane < end; i += 32) {
    const bool valid = i < end;
    const int e = valid ? ids[i] : -1;
    const unsigned act = __ballot_sync(0xffffffffu, valid);
    if (valid) {
      const unsigned same = __match_any_sync(act, e);
      const int rank = __popc(same & ((1u << lane) - 1));
      pos[i] = expertBase[e] + hist[warp][e] + rank;
    }
    __syncwarp();
    if (valid) {
      const unsigned same = __match_any_sync(act, e);
      if ((same & ((1u << lane) - 1)) == 0) hist[warp][e] += __popc(same);
    }
    __syncwarp();
  }
}

// ------------------------------------------------------------------ shared pieces
struct SegTable {
  int segStart[kMaxSeg + 1];  // expert-major (le, src) segments of the received rows
  int srcBase[kMaxSeg];       // position of the segment inside the source's block
};

// cnt: [nRanks][LE] rows per (source, local expert). Every thread of the CTA must call this.
__device__ __forceinline__ void buildSegments(const int* cnt, int N, int LE, SegTable& T) {
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int le = 0; le < LE; ++le)
      for (int s = 0; s < N; ++s) {
        T.segStart[le * N + s] = run;
        run += cnt[s * LE + le];
      }
    T.segStart[LE * N] = run;
  }
  if (threadIdx.x < N) {
    int run = 0;
    for (int le = 0; le < LE; ++le) {
      T.srcBase[le * N + threadIdx.x] = run;
      run += cnt[threadIdx.x * LE + le];
    }
  }
  __syncthreads();
}

__device__ __forceinline__ int findSegment(const SegTable& T, int nSeg, int row) {
  int lo = 0, hi = nSeg;  // last segment with segStart <= row
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (T.segStart[mid] <= row) lo = mid; else hi = mid;
  }
  return lo;
}

// all flags [src][cta] of one direction; returns false for the whole CTA on timeout
__device__ __forceinline__ bool waitAllCtas(const unsigned int* base, int N, int ctas, unsigned int epoch,
                                            unsigned long long timeoutNs, StatusWord* st, int phase) {
  bool ok = true;
  for (int i = threadIdx.x; i < N * ctas && ok; i += blockDim.x) {
    const int s = i / ctas, c = i - s * ctas;
    if (!waitFlag(base + (long)s * kFlagStride + c, epoch, timeoutNs)) {
      reportTimeout(st, phase, s, c);
      ok = false;
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

__device__ __forceinline__ void publishToAll(unsigned int* const* flags, int region, int N, int rank, unsigned int epoch) {
  __syncthreads();
  if (threadIdx.x < N) {
    __threadfence_system();
    stReleaseSys(flags[threadIdx.x] + ((long)region * COCCLK_MOE_MAX_RANKS + rank) * kFlagStride + blockIdx.x, epoch);
  }
}

// ------------------------------------------------------------------ dispatch
__global__ void __launch_bounds__(kThreads) moeDispatchKernel(const cocclkMoeArgs a) {
  __shared__ SegTable T;
  __shared__ int sCnt[kMaxSeg];
  const int N = a.nRanks, rank = a.rankBase + blockIdx.y;
  const int LE = a.experts / N, H = a.hidden, cap = a.capacity;
  const Layout L = makeLayout(N, cap, H, LE);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * kWarps + warp, GW = gridDim.x * kWarps;
  StatusWord* st = reinterpret_cast<StatusWord*>(a.status[rank]);
  const int scalesPerRow = H / 32;

  // ---- phase 1: gather, quantise, push
  {
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x[rank]);
    const int* ids = a.expertIds[rank];
    const int* pos = a.pos[rank];
    const float* rowScale = a.rowScale[rank];
    const int entries = a.tokens * a.topk;
    for (int en = gw; en < entries; en += GW) {
      const int t = en / a.topk, e = ids[en], p = pos[en];
      const int d = e / LE;
      if (p >= cap) continue;  // over capacity: dropped (cannot happen with capacity = tokens * topk)
      const float rs = rowScale ? rowScale[en] : 1.f;
      const uint4* src = reinterpret_cast<const uint4*>(x + (long)t * H);
      uint8_t* wsd = reinterpret_cast<uint8_t*>(a.ws[d]);
      uint2* dp = reinterpret_cast<uint2*>(wsd + L.payloadOff + ((long)rank * cap + p) * H);
      uint8_t* ds = wsd + L.scalesOff + ((long)rank * cap + p) * scalesPerRow;
      // four 256-value pieces per pass: their loads are in flight together
      for (int it0 = 0; it0 < H / 256; it0 += 4) {
        uint4 rawv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (it0 + u < H / 256) rawv[u] = __ldg(src + (it0 + u) * 32 + lane);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
        const int it = it0 + u;
        if (it >= H / 256) break;
        const uint4 raw = rawv[u];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v[2 * i] = __uint_as_float(w[i] << 16) * rs;
          v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u) * rs;
        }
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        int biased = 0;
        if (m > 0.f && m < INFINITY) {
          const uint32_t rb = __float_as_uint(m * (1.f / 448.f));
          int ex = (int)((rb >> 23) & 0xff);
          if (rb & 0x7fffffu) ex += 1;
          biased = max(0, min(254, ex));
        }
        const int invExp = 254 - biased;
        const float inv = invExp > 0 ? __uint_as_float((uint32_t)invExp << 23) : __uint_as_float(0x00400000u);
        uint32_t o[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * k] * inv, v[4 * k + 1] * inv), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * k + 2] * inv, v[4 * k + 3] * inv), __NV_SATFINITE, __NV_E4M3);
          o[k] = lo | (hi << 16);
        }
        dp[it * 32 + lane] = make_uint2(o[0], o[1]);
        if ((lane & 3) == 0) ds[it * 8 + (lane >> 2)] = (uint8_t)biased;
        }
      }
    }
    if (blockIdx.x == 0) {
      const int* sc = a.sendCounts[rank];
      for (int i = threadIdx.x; i < N * LE; i += blockDim.x) {
        const int d = i / LE, le = i - d * LE;
        reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(a.ws[d]) + L.countsOff)[rank * LE + le] = sc[d * LE + le];
      }
    }
    publishToAll(a.flags, 0, N, rank, a.epoch);
  }

  // ---- phase 2: wait for every source, place the rows expert-major, dequantise
  const bool ok = waitAllCtas(a.flags[rank], N, gridDim.x, a.epoch, a.timeoutNs, st, 6);
  const uint8_t* myWs = reinterpret_cast<const uint8_t*>(a.ws[rank]);
  const int* cntG = reinterpret_cast<const int*>(myWs + L.countsOff);
  for (int i = threadIdx.x; i < N * LE; i += blockDim.x) sCnt[i] = ok ? __ldcg(cntG + i) : 0;
  __syncthreads();
  if (threadIdx.x < N) {
    // a source drops the rows whose position in its block reaches the capacity: cut its counts there
    int run = 0;
    for (int le = 0; le < LE; ++le) {
      const int c = sCnt[threadIdx.x * LE + le];
      sCnt[threadIdx.x * LE + le] = max(0, min(c, cap - run));
      run += c;
    }
  }
  buildSegments(sCnt, N, LE, T);
  const int nSeg = N * LE, rows = T.segStart[nSeg];
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < N * LE; i += blockDim.x) a.recvCounts[rank][i] = sCnt[i];
    for (int le = threadIdx.x; le <= LE; le += blockDim.x) a.recvOffsets[rank][le] = T.segStart[le * N];
  }
  __nv_bfloat16* recv = reinterpret_cast<__nv_bfloat16*>(a.recv[rank]);
  for (int r = gw; r < rows; r += GW) {
    const int sg = findSegment(T, nSeg, r);
    const int s = sg % N;
    const long sp = (long)s * cap + T.srcBase[sg] + (r - T.segStart[sg]);
    const uint2* pp = reinterpret_cast<const uint2*>(myWs + L.payloadOff + sp * H);
    const uint8_t* ps = myWs + L.scalesOff + sp * scalesPerRow;
    uint4* out = reinterpret_cast<uint4*>(recv + (long)r * H);
    for (int it0 = 0; it0 < H / 256; it0 += 4) {
      uint2 qv[4];
      uint32_t bv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (it0 + u < H / 256) { qv[u] = __ldcg(pp + (it0 + u) * 32 + lane); bv[u] = __ldcg(ps + (it0 + u) * 8 + (lane >> 2)); }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
      const int it = it0 + u;
      if (it >= H / 256) break;
      const uint2 q = qv[u];
      const uint32_t biased = bv[u];
      const float scale = biased > 0 ? __uint_as_float(biased << 23) : __uint_as_float(0x00400000u);
      const uint32_t qw[2] = {q.x, q.y};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint16_t pair = (uint16_t)(qw[k >> 1] >> (16 * (k & 1)));
        __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
        __nv_bfloat162 h = __floats2bfloat162_rn(f.x * scale, f.y * scale);
        o[k] = *reinterpret_cast<uint32_t*>(&h);
      }
      out[it * 32 + lane] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// ------------------------------------------------------------------ combine
// KMAX: compile-time bound of topk (2, 4 or 8): sizes the per-token routing registers and the batch of loads.
template <int KMAX>
__global__ void __launch_bounds__(kThreads) moeCombineKernel(const cocclkMoeArgs a) {
  __shared__ SegTable T;
  __shared__ int sCnt[kMaxSeg];
  const int N = a.nRanks, rank = a.rankBase + blockIdx.y;
  const int LE = a.experts / N, H = a.hidden, cap = a.capacity;
  const Layout L = makeLayout(N, cap, H, LE);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * kWarps + warp, GW = gridDim.x * kWarps;
  StatusWord* st = reinterpret_cast<StatusWord*>(a.status[rank]);
  const int vecsPerRow = H * 2 / 16;

  // ---- phase 1: expert outputs back to the ranks that own the tokens
  for (int i = threadIdx.x; i < N * LE; i += blockDim.x) sCnt[i] = a.recvCounts[rank][i];
  buildSegments(sCnt, N, LE, T);
  const int nSeg = N * LE, rows = T.segStart[nSeg];
  const __nv_bfloat16* y = reinterpret_cast<const __nv_bfloat16*>(a.y[rank]);
  for (int r = gw; r < rows; r += GW) {
    const int sg = findSegment(T, nSeg, r);
    const int s = sg % N;
    const long sp = (long)rank * cap + T.srcBase[sg] + (r - T.segStart[sg]);
    const uint4* src = reinterpret_cast<const uint4*>(y + (long)r * H);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.ws[s]) + L.retOff + sp * H * 2);
    for (int j = lane; j < vecsPerRow; j += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) if (j + u * 32 < vecsPerRow) v[u] = __ldg(src + j + u * 32);
#pragma unroll
      for (int u = 0; u < 4; ++u) if (j + u * 32 < vecsPerRow) dst[j + u * 32] = v[u];
    }
  }
  publishToAll(a.flags, 1, N, rank, a.epoch);

  // ---- phase 2: gate-weighted sum of the returned rows of every token
  const bool ok = waitAllCtas(a.flags[rank] + (long)COCCLK_MOE_MAX_RANKS * kFlagStride, N, gridDim.x, a.epoch,
                              a.timeoutNs, st, 7);
  if (!ok) return;
  const uint8_t* myRet = reinterpret_cast<const uint8_t*>(a.ws[rank]) + L.retOff;
  const int* ids = a.expertIds[rank];
  const int* pos = a.pos[rank];
  const float* gates = a.gates[rank];
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.out[rank]);
  const __nv_bfloat16* dotWith = reinterpret_cast<const __nv_bfloat16*>(a.dotWith[rank]);
  float* dotOut = a.dotOut[rank];
  for (int t = gw; t < a.tokens; t += GW) {
    float dots[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) dots[j] = 0.f;
    // routing of the token's choices, once per token: a dropped or absent choice reads row 0 with gate 0, so that the
    // loop below has no branches and the loads of all choices go out together
    const uint4* rowPtr[KMAX];
    float gate[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      rowPtr[j] = reinterpret_cast<const uint4*>(myRet);
      gate[j] = 0.f;
      if (j < a.topk) {
        const int en = t * a.topk + j;
        const int p = pos[en];
        if (p < cap) {
          rowPtr[j] = reinterpret_cast<const uint4*>(myRet + ((long)(ids[en] / LE) * cap + p) * H * 2);
          gate[j] = gates[en];
        }
      }
    }
    for (int it = 0; it < H / 256; ++it) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      float dw[8];
      if (dotOut != nullptr) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(dotWith + (long)t * H) + it * 32 + lane);
        const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          dw[2 * i] = __uint_as_float(qw[i] << 16);
          dw[2 * i + 1] = __uint_as_float(qw[i] & 0xffff0000u);
        }
      }
      uint4 rawv[KMAX];
#pragma unroll
      for (int j = 0; j < KMAX; ++j)
        if (j < a.topk) rawv[j] = __ldcg(rowPtr[j] + it * 32 + lane);
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        if (j >= a.topk) break;
        const float g = gate[j];
        const uint4 raw = rawv[j];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xffff0000u);
          acc[2 * i] = fmaf(g, lo, acc[2 * i]);
          acc[2 * i + 1] = fmaf(g, hi, acc[2 * i + 1]);
          if (dotOut != nullptr) dots[j] = fmaf(lo, dw[2 * i], fmaf(hi, dw[2 * i + 1], dots[j]));
        }
      }
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        o[i] = *reinterpret_cast<uint32_t*>(&h);
      }
      reinterpret_cast<uint4*>(out + (long)t * H)[it * 32 + lane] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if (dotOut != nullptr) {
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        if (j >= a.topk) break;
        float d = dots[j];
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (lane == 0) dotOut[t * a.topk + j] = d;
      }
    }
  }
}

}  // namespace moe
}  // namespace coccl

using namespace coccl;
using namespace coccl::moe;

extern "C" long cocclkMoeWorkspaceBytes(int nRanks, int capacity, int hidden, int localExperts) {
  return makeLayout(nRanks, capacity, hidden, localExperts).total;
}

extern "C" int cocclkMoeLayout(const int* expertIds, int entries, int experts, int expertsPerRank, int* pos, int* counts,
                               cudaStream_t stream) {
  if (entries <= 0 || experts <= 0 || experts > COCCLK_MOE_MAX_EXPERTS || expertsPerRank <= 0 || experts % expertsPerRank) return -1;
  moeLayoutKernel<<<1, 1024, 0, stream>>>(expertIds, entries, experts, expertsPerRank, pos, counts);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

template <class Kern>
static int launchMoe(Kern kern, const cocclkMoeArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream) {
  const cocclkMoeArgs& a = *args;
  if (a.nRanks < 1 || a.nRanks > COCCLK_MOE_MAX_RANKS || a.experts % a.nRanks || a.hidden % 256 || a.topk < 1 || a.topk > 8)
    return -1;
  if (a.experts / a.nRanks > COCCLK_MOE_MAX_LOCAL_EXPERTS || a.tokens <= 0 || a.capacity <= 0) return -1;
  if (emulatedRanks != 1 && (emulatedRanks != a.nRanks || a.rankBase != 0)) return -1;
  static int sms = 0;
  int perSm = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kern, kThreads, 0);
  if (e != cudaSuccess || perSm <= 0) return e != cudaSuccess ? (int)e : -1;
  // The grid must be the same on every rank (receivers wait for one flag per sender CTA): it depends only on
  // the device type and on maxCtas.
  long ctas = (long)sms * (perSm > 4 ? 4 : perSm) / emulatedRanks;
  if (maxCtas > 0 && maxCtas < ctas) ctas = maxCtas;
  if (ctas > kFlagStride) ctas = kFlagStride;
  if (ctas < 1) ctas = 1;
  dim3 grid((unsigned)ctas, emulatedRanks, 1);
  cocclkMoeArgs copy = a;
  void* params[] = {&copy};
  cocclkCountLaunches(1);
  if (emulatedRanks > 1) return (int)cudaLaunchCooperativeKernel((const void*)kern, grid, dim3(kThreads), params, 0, stream);
  return (int)cudaLaunchKernel((const void*)kern, grid, dim3(kThreads), params, 0, stream);
}

extern "C" int cocclkMoeDispatch(const cocclkMoeArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream) {
  return launchMoe(moeDispatchKernel, args, emulatedRanks, maxCtas, stream);
}
extern "C" int cocclkMoeCombine(const cocclkMoeArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream) {
  if (args->topk <= 2) return launchMoe(moeCombineKernel<2>, args, emulatedRanks, maxCtas, stream);
  if (args->topk <= 4) return launchMoe(moeCombineKernel<4>, args, emulatedRanks, maxCtas, stream);
  return launchMoe(moeCombineKernel<8>, args, emulatedRanks, maxCtas, stream);
}
