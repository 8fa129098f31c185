// Fused compressed collectives: ONE persistent launch per collective that
// encodes, moves the encoded bytes with direct stores into the peers' receive
// slots over NVLink, signals per-slice flags, and decodes (with reduction and,
// for the two-shot all-reduce, re-encoding) on the receiving side.
//
// What the reference does with host-side stage lists — Compress -> AllToAll ->
// DecompressReduce for ReduceScatter one-shot
// (extensions/primitives/coccl_reducescatter.cc:12-29), Compress -> AllGather
// -> Decompress (coccl_allgather.cc:12-22), Compress -> AllToAll -> Decompress
// (coccl_alltoall.cc:12-21), Compress -> AllGather -> DecompressReduce for
// AllReduce one-shot and Compress -> A2A -> DecompReduceComp -> AllGather ->
// Decompress for two-shot (coccl_allreduce.cc:12-53) — is here three device
// phases of one kernel; `pipeline.depth` becomes the slice granularity.
//
// Work decomposition: a chunk (the elements one rank owns / sends to one peer)
// is cut into slices of `sliceTiles` tiles of 8192 elements. One CTA owns one
// (peer, slice) item at a time; finishing it publishes flag[src][slice]=epoch
// on the receiver with release semantics. Encode items never wait, so every
// wait in a later phase depends only on work that cannot itself block.
// All waits are bounded by a globaltimer deadline and report through the
// status word instead of trapping.
//
// `rankBase`/blockIdx.y let one cooperative launch play all ranks on a single
// GPU (every pointer then refers to local memory); production launches use
// gridDim.y == 1 and peer-mapped pointers.
#pragma once
#include "codecs.cuh"
#include "tile_io.cuh"

namespace coccl {

enum CollOp : int {
  kOpReduceScatter = 0, kOpAllGather = 1, kOpAllToAll = 2, kOpAllReduceOneShot = 3, kOpAllReduceTwoShot = 4,
  // All-gather of DELTAS (the reference's subAdd AllGather, sdp4bit/quantization/sub_quantize.cu:176-262 and
  // dequantize_add.cu:145-275): `out` holds the result of the previous call on every rank, a rank encodes
  // in - out[own chunk] and every rank adds the decoded deltas to all chunks of `out`. Every rank performs the same
  // arithmetic on the same bytes, so the copies of `out` stay identical. The first call must fill `out` exactly.
  kOpAllGatherDelta = 5
};

constexpr int kMaxSlices = 4096;  // per source rank and region

struct CollArgs {
  int op;
  int nRanks;
  int rankBase;
  int dtype;
  long count;            // elements per chunk (AR one-shot: the whole vector; AR two-shot: count/nRanks)
  int sliceTiles;
  unsigned int epoch;
  unsigned long long timeoutNs;
  CodecCfg codec;
  long slotBytes;        // distance between per-source slots inside a region
  long regionBOffset;    // byte offset of region B (two-shot all-reduce)
  const void* in[kMaxRanks];
  void* out[kMaxRanks];
  uint8_t* ws[kMaxRanks];          // workspace of every rank as mapped here (parity offset applied)
  unsigned int* flags[kMaxRanks];  // [2 regions][kMaxRanks sources][kMaxSlices]
  StatusWord* status[kMaxRanks];
  unsigned long long* trace[kMaxRanks];  // optional phase timestamps, 4 per CTA
};

constexpr int kTraceMaxCtas = 2048;
__device__ __forceinline__ void tracePhase(unsigned long long* tr, int phase) {
  if (tr != nullptr && threadIdx.x == 0 && blockIdx.x < kTraceMaxCtas) tr[blockIdx.x * 4 + phase] = globalTimerNs();
}

__device__ __forceinline__ unsigned int* flagPtr(unsigned int* base, int region, int src, int slice) {
  return base + ((long)region * kMaxRanks + src) * kMaxSlices + slice;
}

// Encode the tiles [t0, t1) of one source chunk and store the result into
// nDst destination chunk buffers.
template <typename T, class Codec>
__device__ __forceinline__ void encodeTiles(const T* src, const ChunkLayout& L, const CodecCfg& c, long t0, long t1,
                                            uint8_t* const* dst, int nDst, TileStage<T>& stage, float* sm,
                                            uint64_t rngBase, const T* prev = nullptr) {
  for (long t = t0; t < t1; ++t) {
    const long e0 = t * kTileElems;
    const long e = e0 + (long)threadIdx.x * kElemsPerThread;
    float v[32];
    TileIO<T>::load(src, L.count, e0, TileIO<T>::fastTile(src, L.count, e0), stage, v);
    if (prev != nullptr) {  // delta coding: what is sent is the change since the previous result
      float pv[32];
      TileIO<T>::load(prev, L.count, e0, TileIO<T>::fastTile(prev, L.count, e0), stage, pv);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] -= pv[i];
    }
    const typename Codec::Enc enc = Codec::encode(v, c, true, sm, rngBase + (uint64_t)e);
    if (!COCCL_CHUNK_RANGE_OK(Codec, L, c, e, 1)) continue;
    for (int d = 0; d < nDst; ++d) Codec::store(enc, dst[d], L, c, e);
  }
}

// Publish a flag after every thread of the CTA has finished its stores.
__device__ __forceinline__ void publish(unsigned int* const* flagAddrs, int n, unsigned int epoch) {
  __syncthreads();
  if (threadIdx.x < n) {
    __threadfence_system();
    stReleaseSys(flagAddrs[threadIdx.x], epoch);
  }
}

// Wait for n flags (n <= kMaxRanks). Returns false for the whole CTA on timeout.
__device__ __forceinline__ bool waitAll(unsigned int* const* flagAddrs, int n, unsigned int epoch,
                                        unsigned long long timeoutNs, StatusWord* st, int phase, int slice,
                                        bool skip) {
  bool ok = true;
  if (!skip && threadIdx.x < n) {
    ok = waitFlag(flagAddrs[threadIdx.x], epoch, timeoutNs);
    if (!ok) reportTimeout(st, phase, threadIdx.x, slice);
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

template <typename T, class Codec>
__global__ void __launch_bounds__(kTileThreads, Codec::kMinBlocks) fusedCollectiveKernel(const CollArgs a) {
  __shared__ TileStage<T> stage;
  __shared__ float sm[Codec::kSmemFloats];
  __shared__ uint8_t* sDst[kMaxRanks];
  __shared__ unsigned int* sFlag[kMaxRanks];
  Codec::initShared(sm);
  __syncthreads();

  const int N = a.nRanks;
  const int rank = a.rankBase + blockIdx.y;
  const CodecCfg c = a.codec;
  const ChunkLayout L = makeChunkLayout(c, a.count, 16);
  const long tiles = (a.count + kTileElems - 1) / kTileElems;
  const long slices = (tiles + a.sliceTiles - 1) / a.sliceTiles;
  const T* in = reinterpret_cast<const T*>(a.in[rank]);
  T* out = reinterpret_cast<T*>(a.out[rank]);
  uint8_t* myWs = a.ws[rank];
  unsigned int* myFlags = a.flags[rank];
  StatusWord* st = a.status[rank];
  unsigned long long* tr = a.trace[rank];
  tracePhase(tr, 0);
  // The slot geometry comes from the host: a chunk that does not fit its slot, or a second region that overlaps the
  // first, would make ranks write over each other's data. Checked in every build, before anything is touched.
  if (L.stride > a.slotBytes || (a.op == kOpAllReduceTwoShot && a.regionBOffset < (long)N * a.slotBytes)) {
    if (threadIdx.x == 0) reportTimeout(st, 0xB, rank, 0);
    return;
  }
  bool failed = false;
  const bool perPeer = (a.op == kOpReduceScatter || a.op == kOpAllToAll || a.op == kOpAllReduceTwoShot);

  // ---------------- phase 1: encode + push ----------------
  {
    const long items = perPeer ? slices * N : slices;
    for (long it = blockIdx.x; it < items; it += gridDim.x) {
      const long s = perPeer ? it / N : it;
      const long t0 = s * a.sliceTiles;
      const long t1 = min(tiles, t0 + (long)a.sliceTiles);
      __syncthreads();
      if (perPeer) {
        const int p = (rank + 1 + (int)(it % N)) % N;
        if (threadIdx.x == 0) {
          sDst[0] = a.ws[p] + (long)rank * a.slotBytes;
          sFlag[0] = flagPtr(a.flags[p], 0, rank, (int)s);
        }
        __syncthreads();
        encodeTiles<T, Codec>(in + (long)p * a.count, L, c, t0, t1, sDst, 1, stage, sm,
                              ((uint64_t)(rank * N + p) << 40));
        publish(sFlag, 1, a.epoch);
      } else {
        if (threadIdx.x < N) {
          const int p = (rank + 1 + threadIdx.x) % N;
          sDst[threadIdx.x] = a.ws[p] + (long)rank * a.slotBytes;
          sFlag[threadIdx.x] = flagPtr(a.flags[p], 0, rank, (int)s);
        }
        __syncthreads();
        encodeTiles<T, Codec>(in, L, c, t0, t1, sDst, N, stage, sm, ((uint64_t)rank << 40),
                              a.op == kOpAllGatherDelta ? out + (long)rank * a.count : nullptr);
        publish(sFlag, N, a.epoch);
      }
    }
  }

  tracePhase(tr, 1);
  // ---------------- phase 2: wait + decode ----------------
  const bool reduce = (a.op == kOpReduceScatter || a.op == kOpAllReduceOneShot || a.op == kOpAllReduceTwoShot);
  {
    const long items = reduce ? slices : slices * N;
    for (long it = blockIdx.x; it < items; it += gridDim.x) {
      const long s = reduce ? it : it / N;
      const int q0 = reduce ? 0 : (int)((rank + 1 + it % N) % N);
      const int nq = reduce ? N : 1;
      const long t0 = s * a.sliceTiles;
      const long t1 = min(tiles, t0 + (long)a.sliceTiles);
      __syncthreads();
      if (threadIdx.x < nq) sFlag[threadIdx.x] = flagPtr(myFlags, 0, q0 + threadIdx.x, (int)s);
      __syncthreads();
      if (!waitAll(sFlag, nq, a.epoch, a.timeoutNs, st, 2, (int)s, failed)) failed = true;

      if (a.op == kOpAllReduceTwoShot) {
        if (threadIdx.x < N) {
          const int p = (rank + 1 + threadIdx.x) % N;
          sDst[threadIdx.x] = a.ws[p] + a.regionBOffset + (long)rank * a.slotBytes;
          sFlag[threadIdx.x] = flagPtr(a.flags[p], 1, rank, (int)s);
        }
        __syncthreads();
      }
      T* dstChunk = reduce ? out : out + (long)q0 * a.count;
      for (long t = t0; t < t1; ++t) {
        const long e0 = t * kTileElems;
        const long e = e0 + (long)threadIdx.x * kElemsPerThread;
        float acc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.f;
        decodeSum<Codec>(myWs + (long)q0 * a.slotBytes, a.slotBytes, nq, L, c, e,
                         a.op == kOpAllReduceTwoShot ? 1.f : Codec::finishScale(c), acc, sm);
        if (a.op == kOpAllReduceTwoShot) {
          // stay in the rotated domain: the sum of rotated values is the rotation of the sum
          const typename Codec::Enc enc = Codec::encode(acc, c, false, sm, ((uint64_t)(0x80 + rank) << 40) + (uint64_t)e);
          if (COCCL_CHUNK_RANGE_OK(Codec, L, c, e, 3))
            for (int d = 0; d < N; ++d) Codec::store(enc, sDst[d], L, c, e);
        } else {
          Codec::finish(acc, c);
          const bool fast = TileIO<T>::fastTile(dstChunk, L.count, e0);
          if (a.op == kOpAllGatherDelta) {
            float pv[32];
            TileIO<T>::load(dstChunk, L.count, e0, fast, stage, pv);
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] += pv[i];
          }
          TileIO<T>::store(dstChunk, L.count, e0, fast, stage, acc);
        }
      }
      if (a.op == kOpAllReduceTwoShot) publish(sFlag, N, a.epoch);
    }
  }

  tracePhase(tr, 2);
  // ---------------- phase 3 (two-shot all-reduce): gather reduced chunks ----------------
  if (a.op == kOpAllReduceTwoShot) {
    const long items = slices * N;
    for (long it = blockIdx.x; it < items; it += gridDim.x) {
      const long s = it / N;
      const int q = (int)((rank + 1 + it % N) % N);
      const long t0 = s * a.sliceTiles;
      const long t1 = min(tiles, t0 + (long)a.sliceTiles);
      __syncthreads();
      if (threadIdx.x == 0) sFlag[0] = flagPtr(myFlags, 1, q, (int)s);
      __syncthreads();
      if (!waitAll(sFlag, 1, a.epoch, a.timeoutNs, st, 3, (int)s, failed)) failed = true;
      T* dstChunk = out + (long)q * a.count;
      for (long t = t0; t < t1; ++t) {
        const long e0 = t * kTileElems;
        const long e = e0 + (long)threadIdx.x * kElemsPerThread;
        float acc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.f;
        decodeSum<Codec>(myWs + a.regionBOffset + (long)q * a.slotBytes, 0, 1, L, c, e, Codec::finishScale(c), acc, sm);
        Codec::finish(acc, c);
        TileIO<T>::store(dstChunk, L.count, e0, TileIO<T>::fastTile(dstChunk, L.count, e0), stage, acc);
      }
    }
  }
  tracePhase(tr, 3);
}

// ---------------------------------------------------------------------------
// Standalone codec kernels (plugin path, tests, autotune profiling).
// ---------------------------------------------------------------------------
struct CodecArgs {
  const void* in;      // raw input (encode) or encoded input (decode)
  void* out;           // encoded output (encode / drc) or raw output (decode)
  long count;          // elements per chunk
  long chunks;         // encode: input chunks; decode: OUTPUT chunks
  long reduce;         // decode / drc: encoded copies summed per output chunk (>=1)
  long rawPitch;       // elements between consecutive raw chunks
  long encStrideIn;    // bytes between encoded input chunks
  long encStrideOut;   // bytes between encoded output chunks
  int dtype;
  CodecCfg codec;
  CodecCfg codecOut;   // drc: codec of the re-encoded output (same family)
};

template <typename T, class Codec>
__global__ void __launch_bounds__(kTileThreads) encodeKernel(const CodecArgs a) {
  __shared__ TileStage<T> stage;
  __shared__ float sm[Codec::kSmemFloats];
  __shared__ uint8_t* sDst[1];
  Codec::initShared(sm);
  __syncthreads();
  const ChunkLayout L = makeChunkLayout(a.codec, a.count, 4);
  const long tiles = (a.count + kTileElems - 1) / kTileElems;
  for (long it = blockIdx.x; it < tiles * a.chunks; it += gridDim.x) {
    const long ch = it / tiles, t = it % tiles;
    __syncthreads();
    if (threadIdx.x == 0) sDst[0] = reinterpret_cast<uint8_t*>(a.out) + ch * a.encStrideOut;
    __syncthreads();
    encodeTiles<T, Codec>(reinterpret_cast<const T*>(a.in) + ch * a.rawPitch, L, a.codec, t, t + 1, sDst, 1, stage,
                          sm, (uint64_t)ch << 40);
  }
}

// out chunk j = sum_{i<reduce} decode(in chunk i*chunks + j)
template <typename T, class Codec>
__global__ void __launch_bounds__(kTileThreads) decodeReduceKernel(const CodecArgs a) {
  __shared__ TileStage<T> stage;
  __shared__ float sm[Codec::kSmemFloats];
  Codec::initShared(sm);
  __syncthreads();
  const ChunkLayout L = makeChunkLayout(a.codec, a.count, 4);
  const long tiles = (a.count + kTileElems - 1) / kTileElems;
  const uint8_t* enc = reinterpret_cast<const uint8_t*>(a.in);
  for (long it = blockIdx.x; it < tiles * a.chunks; it += gridDim.x) {
    const long ch = it / tiles, t = it % tiles;
    T* dst = reinterpret_cast<T*>(a.out) + ch * a.rawPitch;
    const long e0 = t * kTileElems;
    const long e = e0 + (long)threadIdx.x * kElemsPerThread;
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    decodeSum<Codec>(enc + ch * a.encStrideIn, a.chunks * a.encStrideIn, (int)a.reduce, L, a.codec, e,
                     Codec::finishScale(a.codec), acc, sm);
    Codec::finish(acc, a.codec);
    TileIO<T>::store(dst, L.count, e0, TileIO<T>::fastTile(dst, L.count, e0), stage, acc);
  }
}

// decode + reduce + re-encode without leaving registers
// (reference kernel: sdp4bit/quantization/dequant_reduce_quant.cu:14-179).
template <class Codec>
__global__ void __launch_bounds__(kTileThreads, Codec::kMinBlocks) decodeReduceEncodeKernel(const CodecArgs a) {
  __shared__ float sm[Codec::kSmemFloats];
  Codec::initShared(sm);
  __syncthreads();
  const ChunkLayout L = makeChunkLayout(a.codec, a.count, 4);
  const long tiles = (a.count + kTileElems - 1) / kTileElems;
  const uint8_t* enc = reinterpret_cast<const uint8_t*>(a.in);
  for (long it = blockIdx.x; it < tiles * a.chunks; it += gridDim.x) {
    const long ch = it / tiles, t = it % tiles;
    const long e = t * kTileElems + (long)threadIdx.x * kElemsPerThread;
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    decodeSum<Codec>(enc + ch * a.encStrideIn, a.chunks * a.encStrideIn, (int)a.reduce, L, a.codec, e, 1.f, acc, sm);
    const typename Codec::Enc o = Codec::encode(acc, a.codec, false, sm, ((uint64_t)(0x40 + ch) << 40) + (uint64_t)e);
    Codec::store(o, reinterpret_cast<uint8_t*>(a.out) + ch * a.encStrideOut, L, a.codec, e);
  }
}

}  // namespace coccl
