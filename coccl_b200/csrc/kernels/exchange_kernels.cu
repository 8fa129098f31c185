// Byte exchange over peer memory for the staged pipeline: all-to-all and all-gather of encoded chunks, and the
// exchange of variable-size frames, without a library collective.
//
// The staged pipeline serves codecs that exist only as plugins (rANS, ZFP at rates without a tile form, third-party
// codecs): compress -> move bytes -> decompress. Moving the bytes was NCCL's job
// (reference: src/coccl-extend/core/pipeline/coccl_pipeline_stage.cc:120-139 calls ncclAllToAll / ncclAllGather, and the
// framed path first brings the frame sizes to the host, coccl_pipeline_execute.cc:218-260). On one NVSwitch domain this
// kernel does it instead: every rank stores its blocks straight into a staging area in the receiver's memory, piece by
// piece, raises one flag per piece, and copies the pieces addressed to it out of its own staging area as their flags
// arrive. For framed codecs the sender reads the frame's size from the metadata the codec left ON THE DEVICE and
// moves only the bytes that exist; the 16-byte metadata record travels with the first piece, so no host round trip
// separates sizes from payloads.
//
// Layout. A rank sends `blocks` (one per destination for all-to-all, the same one to everybody for all-gather); a block
// is `frames` frames of `frameStride` bytes capacity (unframed data: one frame per block, always full). A frame is cut
// into pieces of `pieceBytes`; item (frame f, piece i) of the block from rank s to rank d lives at
// staging[d] + (s * frames + f) * frameStride + i * pieceBytes and is announced by flags[d][s][f * pieces + i].
// The metadata of frame f from s sits in the staging area behind the payload slots.
//
// One launch can play every rank on one GPU (blockIdx.y = rank, cooperative) for tests. Waits are bounded.
#include "common.cuh"
#include "kernels_api.h"
#include "launch_count.h"

#include <string.h>

namespace coccl {

constexpr int kExchangeMaxItems = 4096;   // flags per source rank (one region of the flag block)

struct ExchangeArgs {
  int nRanks, rankBase;
  int gather;                    // 0: block p of `send` goes to rank p; 1: the one block of `send` goes to every rank
  int frames;                    // frames per block
  int pieces;                    // pieces per frame
  long frameStride, pieceBytes;  // multiples of 16
  const uint8_t* send[kMaxRanks];
  uint8_t* recv[kMaxRanks];      // nRanks blocks in source order
  const uint4* sendMeta[kMaxRanks];  // framed: one 16-byte record per frame {payload bytes, encoding}; null = full frames
  uint4* recvMeta[kMaxRanks];
  uint8_t* staging[kMaxRanks];
  unsigned int* flags[kMaxRanks];
  StatusWord* status[kMaxRanks];
  unsigned int epoch;
  unsigned long long timeoutNs;
};

__device__ __forceinline__ long metaOffset(const ExchangeArgs& a) { return (long)a.nRanks * a.frames * a.frameStride; }

// bytes of frame `f` (of the block for `dst`) that exist, rounded up to whole 16-byte vectors
__device__ __forceinline__ long frameBytes(const ExchangeArgs& a, const uint4* meta, long frameIndex) {
  if (meta == nullptr) return a.frameStride;
  const uint4 m = __ldg(meta + frameIndex);
  unsigned long long b = (unsigned long long)m.x | ((unsigned long long)m.y << 32);
  if (b > (unsigned long long)a.frameStride) b = (unsigned long long)a.frameStride;  // a corrupt size must not leave the slot
  return (long)((b + 15) & ~15ull);
}

__device__ __forceinline__ void copyVec(const uint8_t* src, uint8_t* dst, long bytes, bool fromPeerWrite) {
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  const long n = bytes >> 4;
  long i = threadIdx.x;
  // four loads in flight per thread
  for (; i + 3L * blockDim.x < n; i += 4L * blockDim.x) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = fromPeerWrite ? __ldcg(s + i + (long)u * blockDim.x) : __ldg(s + i + (long)u * blockDim.x);
#pragma unroll
    for (int u = 0; u < 4; ++u) d[i + (long)u * blockDim.x] = v[u];
  }
  for (; i < n; i += blockDim.x) d[i] = fromPeerWrite ? __ldcg(s + i) : __ldg(s + i);
}

__global__ void __launch_bounds__(256) peerExchangeKernel(const ExchangeArgs a) {
  const int N = a.nRanks;
  const int rank = a.rankBase + blockIdx.y;
  const long itemsPerBlock = (long)a.frames * a.pieces;
  const long blockStride = (long)a.frames * a.frameStride;
  __shared__ int sOk;
  bool failed = false;

  // ---------------- phase 1: store my blocks into the receivers' staging areas ----------------
  for (long it = blockIdx.x; it < itemsPerBlock * N; it += gridDim.x) {
    const int step = (int)(it / itemsPerBlock);            // ring order: rank+1 first, myself last
    const int dst = (rank + 1 + step) % N;
    const long item = it - (long)step * itemsPerBlock;
    const int f = (int)(item / a.pieces), piece = (int)(item - (long)f * a.pieces);
    const long srcBlock = a.gather ? 0 : dst;
    const uint8_t* from = a.send[rank] + srcBlock * blockStride + (long)f * a.frameStride;
    const uint4* meta = a.sendMeta[rank];
    const long have = frameBytes(a, meta, srcBlock * a.frames + f);
    const long lo = (long)piece * a.pieceBytes;
    const long n = have > lo ? (have - lo < a.pieceBytes ? have - lo : a.pieceBytes) : 0;
    if (dst == rank) {
      // my own block never leaves this GPU
      uint8_t* to = a.recv[rank] + (long)rank * blockStride + (long)f * a.frameStride;
      if (n > 0) copyVec(from + lo, to + lo, n, false);
      if (piece == 0 && meta != nullptr && threadIdx.x == 0) a.recvMeta[rank][(long)rank * a.frames + f] = __ldg(meta + srcBlock * a.frames + f);
      continue;
    }
    uint8_t* to = a.staging[dst] + ((long)rank * a.frames + f) * a.frameStride;
    if (n > 0) copyVec(from + lo, to + lo, n, false);
    if (piece == 0 && meta != nullptr && threadIdx.x == 0)
      reinterpret_cast<uint4*>(a.staging[dst] + metaOffset(a))[(long)rank * a.frames + f] = __ldg(meta + srcBlock * a.frames + f);
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      stReleaseSys(a.flags[dst] + (long)rank * kExchangeMaxItems + item, a.epoch);
    }
  }

  // ---------------- phase 2: copy what arrived for me out of my staging area ----------------
  for (long it = blockIdx.x; it < itemsPerBlock * (N - 1); it += gridDim.x) {
    const int step = (int)(it / itemsPerBlock);
    const int src = (rank + N - 1 - step) % N;             // the rank that sent to me first comes first
    const long item = it - (long)step * itemsPerBlock;
    const int f = (int)(item / a.pieces), piece = (int)(item - (long)f * a.pieces);
    if (threadIdx.x == 0) {
      bool ok = !failed && waitFlag(a.flags[rank] + (long)src * kExchangeMaxItems + item, a.epoch, a.timeoutNs);
      if (!ok && !failed) reportTimeout(a.status[rank], 6, src, (int)item);
      sOk = ok ? 1 : 0;
    }
    __syncthreads();
    const bool ok = sOk != 0;
    __syncthreads();
    if (!ok) { failed = true; continue; }
    const uint8_t* stagedFrame = a.staging[rank] + ((long)src * a.frames + f) * a.frameStride;
    const uint4* stagedMeta = reinterpret_cast<const uint4*>(a.staging[rank] + metaOffset(a));
    long have = a.frameStride;
    if (a.sendMeta[rank] != nullptr) {
      // the record was stored before piece 0's flag; pieces of one frame may be taken by different CTAs, so every
      // piece waits for piece 0 as well before it trusts the size
      if (piece != 0) {
        if (threadIdx.x == 0) sOk = waitFlag(a.flags[rank] + (long)src * kExchangeMaxItems + (long)f * a.pieces, a.epoch, a.timeoutNs) ? 1 : 0;
        __syncthreads();
        const bool ok0 = sOk != 0;
        __syncthreads();
        if (!ok0) { if (threadIdx.x == 0) reportTimeout(a.status[rank], 7, src, (int)item); failed = true; continue; }
      }
      const uint4 m = __ldcg(stagedMeta + (long)src * a.frames + f);
      unsigned long long b = (unsigned long long)m.x | ((unsigned long long)m.y << 32);
      if (b > (unsigned long long)a.frameStride) b = (unsigned long long)a.frameStride;
      have = (long)((b + 15) & ~15ull);
      if (piece == 0 && threadIdx.x == 0) a.recvMeta[rank][(long)src * a.frames + f] = m;
    }
    const long lo = (long)piece * a.pieceBytes;
    const long n = have > lo ? (have - lo < a.pieceBytes ? have - lo : a.pieceBytes) : 0;
    uint8_t* to = a.recv[rank] + (long)src * (long)a.frames * a.frameStride + (long)f * a.frameStride;
    if (n > 0) copyVec(stagedFrame + lo, to + lo, n, true);
  }
}

}  // namespace coccl

using namespace coccl;

extern "C" long cocclkExchangeStagingBytes(int nRanks, int frames, long frameStride) {
  const long payload = (long)nRanks * frames * frameStride;
  return ((payload + (long)nRanks * frames * 16 + 255) / 256) * 256;
}

// Pieces per frame for a frame capacity: pieces of about 256 KiB, as many as the flag block allows.
extern "C" int cocclkExchangePieces(int frames, long frameStride, long* pieceBytes) {
  if (frames < 1 || frameStride < 16 || (frameStride & 15)) return -1;
  if (frames > kExchangeMaxItems) return -1;
  long pieces = (frameStride + (256L << 10) - 1) / (256L << 10);
  const long maxPieces = kExchangeMaxItems / frames;
  if (pieces > maxPieces) pieces = maxPieces;
  if (pieces < 1) pieces = 1;
  long pb = ((frameStride + pieces - 1) / pieces + 15) & ~15L;
  pieces = (frameStride + pb - 1) / pb;
  *pieceBytes = pb;
  return (int)pieces;
}

extern "C" int cocclkPeerExchange(const cocclkExchangeArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream) {
  static_assert(sizeof(cocclkExchangeArgs) == sizeof(ExchangeArgs), "public and device argument blocks must match");
  ExchangeArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.nRanks < 2 || a.nRanks > kMaxRanks || a.frames < 1 || a.pieces < 1 || (long)a.frames * a.pieces > kExchangeMaxItems) return -1;
  if ((a.frameStride & 15) || (a.pieceBytes & 15) || a.pieceBytes * a.pieces < a.frameStride) return -1;
  if (emulatedRanks != 1 && emulatedRanks != a.nRanks) return -1;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long items = (long)a.frames * a.pieces * a.nRanks;
  long cap = (long)sms * 2 / emulatedRanks;   // two CTAs of 256 threads per SM: a copy kernel, little state
  if (maxCtas > 0 && maxCtas < cap) cap = maxCtas;
  if (cap < 1) cap = 1;
  const dim3 grid((unsigned)(items < cap ? items : cap), (unsigned)emulatedRanks, 1);
  cocclkCountLaunches(1);
  void* params[] = {&a};
  if (emulatedRanks > 1)
    return (int)cudaLaunchCooperativeKernel((const void*)peerExchangeKernel, grid, dim3(256), params, 0, stream);
  return (int)cudaLaunchKernel((const void*)peerExchangeKernel, grid, dim3(256), params, 0, stream);
}
