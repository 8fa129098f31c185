// libans.so: lossless byte-wise rANS entropy coder as a FRAMED compressor plugin (variable-length output).
//
// Option (reference: dietgpu/dietgpu_plugin.cu:18-20,193-202): probBits 9|10|11 (10).
// One frame per chunk in a fixed slot; the frame metadata says Encoded or Raw, and a chunk whose coded frame
// would not be smaller than its bytes is stored raw, as the reference's finalizeFrames does
// (dietgpu_plugin.cu:138-164,257-297). Any datatype is accepted: the coder sees bytes (kBytewiseLossless).
// Coder and frame layout: oracle/rans.h.
//
// Kernels per call: byte histogram -> probability table -> one warp per 4096-byte block codes into a candidate
// slot (32 interleaved lanes, words of a step appended in lane order through a warp ballot) -> per-chunk
// finalise (scan of the block sizes, compaction into the frame, Encoded/Raw decision, metadata). Decode: one
// warp per block walks the steps backwards. Nothing synchronises the host; sizes are published on the device.
#include "compressor_plugin/coccl_compressor_plugin.h"
#include "kernels/common.cuh"
#include "oracle/rans.h"

namespace {
using coccl::Status;
using namespace coccl;
using namespace coccl::rans;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
enum : uint32_t { kEncodingRaw = 0, kEncodingRans = 1 };

struct AnsConfig { int probBits = 10; };

struct AnsArgs {
  const uint8_t* raw;        // encode input / decode output base
  uint8_t* frames;           // frame slots
  cocclCompressorFrameMetadata* meta;
  uint32_t* hist;            // [chunks][256]
  uint16_t* cand;            // [chunks][numBlocks][kMaxBlockWords]
  long chunkBytes, frameStride, chunks;
  int probBits;
};

__device__ __forceinline__ uint16_t* pdfOf(uint8_t* frame) { return reinterpret_cast<uint16_t*>(frame + 32); }
__device__ __forceinline__ uint32_t* statesOf(uint8_t* frame) { return reinterpret_cast<uint32_t*>(frame + 32 + 512); }
__device__ __forceinline__ uint32_t* wordsOf(uint8_t* frame, uint32_t nb) { return statesOf(frame) + (size_t)nb * kLanes; }
__device__ __forceinline__ uint32_t* startsOf(uint8_t* frame, uint32_t nb) { return wordsOf(frame, nb) + nb; }

__global__ void __launch_bounds__(kThreads) ansHistKernel(const AnsArgs a) {
  __shared__ uint32_t h[256];
  const long ch = blockIdx.y;
  h[threadIdx.x] = 0;
  __syncthreads();
  const uint8_t* src = a.raw + ch * a.chunkBytes;
  const long vecs = a.chunkBytes / 4;
  for (long i = (long)blockIdx.x * kThreads + threadIdx.x; i < vecs; i += (long)gridDim.x * kThreads) {
    const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(src) + i);
    atomicAdd(&h[w & 0xff], 1u);
    atomicAdd(&h[(w >> 8) & 0xff], 1u);
    atomicAdd(&h[(w >> 16) & 0xff], 1u);
    atomicAdd(&h[w >> 24], 1u);
  }
  if (blockIdx.x == 0 && threadIdx.x < (a.chunkBytes & 3)) atomicAdd(&h[src[vecs * 4 + threadIdx.x]], 1u);
  __syncthreads();
  if (h[threadIdx.x]) atomicAdd(&a.hist[ch * 256 + threadIdx.x], h[threadIdx.x]);
}

__global__ void ansTableKernel(const AnsArgs a) {
  const long ch = blockIdx.x;
  if (threadIdx.x == 0) normalise(a.hist + ch * 256, (uint32_t)a.chunkBytes, a.probBits, pdfOf(a.frames + ch * a.frameStride));
}

__global__ void __launch_bounds__(kThreads) ansEncodeKernel(const AnsArgs a) {
  __shared__ uint16_t pdf[256], cdf[256];
  __shared__ __align__(16) uint8_t blk[kWarps][kBlockBytes];
  const long ch = blockIdx.y;
  uint8_t* frame = a.frames + ch * a.frameStride;
  const uint8_t* src = a.raw + ch * a.chunkBytes;
  const uint32_t nb = numBlocks((uint32_t)a.chunkBytes);
  pdf[threadIdx.x] = pdfOf(frame)[threadIdx.x];
  __syncthreads();
  if (threadIdx.x == 0) { uint32_t run = 0; for (int i = 0; i < 256; ++i) { cdf[i] = (uint16_t)run; run += pdf[i]; } }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint32_t b = blockIdx.x * kWarps + warp; b < nb; b += gridDim.x * kWarps) {
    const long off = (long)b * kBlockBytes;
    const int n = (int)min((long)kBlockBytes, a.chunkBytes - off);
    for (int i = lane; i < kBlockBytes; i += 32) blk[warp][i] = i < n ? src[off + i] : 0;
    __syncwarp();
    uint16_t* out = a.cand + ((size_t)ch * nb + b) * kMaxBlockWords;
    uint32_t state = kLower, written = 0;
    const int steps = (n + kLanes - 1) / kLanes;
    for (int j = 0; j < steps; ++j) {
      const bool active = j * kLanes + lane < n;
      bool emit = false;
      uint16_t word = 0;
      if (active) {
        const uint32_t s = blk[warp][j * kLanes + lane];
        emit = encodeStep(state, pdf[s], cdf[s], a.probBits, word);
      }
      const unsigned m = __ballot_sync(0xffffffffu, emit);
      if (emit) out[written + __popc(m & ((1u << lane) - 1))] = word;
      written += __popc(m);
    }
    statesOf(frame)[(size_t)b * kLanes + lane] = state;
    if (lane == 0) wordsOf(frame, nb)[b] = written;
    __syncwarp();
  }
}

// One CTA per chunk: place the block streams (8-word aligned), decide Encoded / Raw, write header and metadata.
__global__ void __launch_bounds__(1024) ansFinalizeKernel(const AnsArgs a) {
  __shared__ uint32_t part[1024];
  __shared__ uint32_t sTotal;
  const long ch = blockIdx.x;
  uint8_t* frame = a.frames + ch * a.frameStride;
  const uint32_t nb = numBlocks((uint32_t)a.chunkBytes);
  uint32_t* words = wordsOf(frame, nb);
  uint32_t* starts = startsOf(frame, nb);
  const uint32_t per = (nb + 1023) / 1024;
  const uint32_t b0 = threadIdx.x * per, b1 = min(nb, b0 + per);
  uint32_t sum = 0;
  for (uint32_t b = b0; b < b1; ++b) sum += (words[b] + 7) & ~7u;
  part[threadIdx.x] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t run = 0;
    for (int i = 0; i < 1024; ++i) { const uint32_t c = part[i]; part[i] = run; run += c; }
    sTotal = run;
  }
  __syncthreads();
  const uint32_t hdr = headerBytes(nb);
  const uint64_t coded = (uint64_t)hdr + (uint64_t)sTotal * 2;
  const bool useRans = coded < (uint64_t)a.chunkBytes && coded <= (uint64_t)a.frameStride;
  if (useRans) {
    uint32_t run = part[threadIdx.x];
    for (uint32_t b = b0; b < b1; ++b) { starts[b] = run; run += (words[b] + 7) & ~7u; }
    __syncthreads();
    uint16_t* streams = reinterpret_cast<uint16_t*>(frame + hdr);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t b = warp; b < nb; b += 32) {
      const uint16_t* src = a.cand + ((size_t)ch * nb + b) * kMaxBlockWords;
      uint16_t* dst = streams + starts[b];
      const uint32_t n = words[b];
      for (uint32_t i = lane; i < n; i += 32) dst[i] = src[i];
    }
    if (threadIdx.x == 0) {
      FrameHeader h{kMagic, nb, (uint32_t)a.chunkBytes, sTotal, (uint32_t)a.probBits, {0, 0, 0}};
      *reinterpret_cast<FrameHeader*>(frame) = h;
      a.meta[ch].payloadBytes = coded;
      a.meta[ch].encoding = kEncodingRans;
      a.meta[ch].reserved = 0;
    }
  } else {
    const uint8_t* src = a.raw + ch * a.chunkBytes;
    for (long i = threadIdx.x; i < a.chunkBytes; i += blockDim.x) frame[i] = src[i];
    if (threadIdx.x == 0) {
      a.meta[ch].payloadBytes = (uint64_t)a.chunkBytes;
      a.meta[ch].encoding = kEncodingRaw;
      a.meta[ch].reserved = 0;
    }
  }
}

__global__ void __launch_bounds__(kThreads) ansDecodeKernel(const AnsArgs a) {
  __shared__ uint16_t pdf[256], cdf[256];
  __shared__ uint8_t lookup[1 << 11];
  __shared__ __align__(16) uint8_t blk[kWarps][kBlockBytes];
  const long ch = blockIdx.y;
  uint8_t* frame = a.frames + ch * a.frameStride;
  uint8_t* dst = const_cast<uint8_t*>(a.raw) + ch * a.chunkBytes;
  if (a.meta[ch].encoding == kEncodingRaw) {
    for (long i = (long)blockIdx.x * kThreads + threadIdx.x; i < a.chunkBytes; i += (long)gridDim.x * kThreads) dst[i] = frame[i];
    return;
  }
  const FrameHeader h = *reinterpret_cast<const FrameHeader*>(frame);
  if (h.magic != kMagic || h.rawBytes != (uint32_t)a.chunkBytes || h.probBits < 9 || h.probBits > 11) return;  // not a frame of ours
  const uint32_t nb = h.numBlocks;
  const int pb = (int)h.probBits;
  pdf[threadIdx.x] = pdfOf(frame)[threadIdx.x];
  __syncthreads();
  if (threadIdx.x == 0) { uint32_t run = 0; for (int i = 0; i < 256; ++i) { cdf[i] = (uint16_t)run; run += pdf[i]; } }
  __syncthreads();
  {
    const uint32_t lo = cdf[threadIdx.x], hi = lo + pdf[threadIdx.x];
    for (uint32_t s = lo; s < hi && s < (1u << pb); ++s) lookup[s] = (uint8_t)threadIdx.x;
  }
  __syncthreads();
  const uint16_t* streams = reinterpret_cast<const uint16_t*>(frame + headerBytes(nb));
  const uint32_t mask = (1u << pb) - 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint32_t b = blockIdx.x * kWarps + warp; b < nb; b += gridDim.x * kWarps) {
    const long off = (long)b * kBlockBytes;
    const int n = (int)min((long)kBlockBytes, a.chunkBytes - off);
    const uint16_t* in = streams + startsOf(frame, nb)[b];
    uint32_t avail = wordsOf(frame, nb)[b];
    uint32_t state = statesOf(frame)[(size_t)b * kLanes + lane];
    const int steps = (n + kLanes - 1) / kLanes;
    for (int j = steps - 1; j >= 0; --j) {
      const bool active = j * kLanes + lane < n;
      bool need = false;
      if (active) {
        const uint32_t s = lookup[state & mask];
        blk[warp][j * kLanes + lane] = (uint8_t)s;
        need = decodeStep(state, pdf[s], cdf[s], pb);
      }
      const unsigned m = __ballot_sync(0xffffffffu, need);
      const uint32_t cnt = __popc(m);
      avail = avail >= cnt ? avail - cnt : 0;  // a damaged frame must not read before its stream
      if (need) state = (state << 16) | in[avail + __popc(m & ((1u << lane) - 1))];
    }
    __syncwarp();
    for (int i = lane; i < n; i += 32) dst[off + i] = blk[warp][i];
    __syncwarp();
  }
}

int smCount() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

struct Ans {
  using Config = AnsConfig;
  static constexpr bool kFramed = true;
  static constexpr bool kBytewiseLossless = true;

  static Status configure(coccl::ConfigReader& r, Config& c, const coccl::ConfigContext&) {
    r.get("probBits", c.probBits, 9, 11);
    return r.ok() ? ncclSuccess : ncclInvalidArgument;
  }

  static bool shapeOk(size_t bytes, size_t chunks) {
    return chunks > 0 && chunks <= 65535 && bytes % chunks == 0 && (bytes / chunks) % 4 == 0 && bytes / chunks <= (1ull << 30);
  }

  static Status encodedSizeBound(const coccl::Shape& s, size_t* bytes, const coccl::SizeContext&) {
    const size_t raw = s.elements() * coccl::dataTypeSize(s.datatype());
    if (!shapeOk(raw, s.chunks())) return ncclInvalidUsage;
    *bytes = (size_t)frameBound(raw / s.chunks()) * s.chunks();
    return ncclSuccess;
  }

  static Status compress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    if (!shapeOk(in.bytes(), in.chunks()) || !out.framed()) return ncclInvalidArgument;
    AnsArgs a{};
    a.chunks = (long)in.chunks();
    a.chunkBytes = (long)(in.bytes() / in.chunks());
    a.frameStride = (long)out.frameStrideBytes();
    a.probBits = ctx.config<Config>().probBits;
    if ((uint64_t)a.frameStride < frameBound((uint64_t)a.chunkBytes) && a.frameStride < a.chunkBytes) return ncclInvalidArgument;
    const uint32_t nb = numBlocks((uint32_t)a.chunkBytes);
    if ((uint64_t)a.frameStride < headerBytes(nb)) return ncclInvalidArgument;
    coccl::Buffer hist, cand;
    Status s = ctx.scratch((size_t)a.chunks * 256 * 4, &hist);
    if (s != ncclSuccess) return s;
    s = ctx.scratch((size_t)a.chunks * nb * kMaxBlockWords * 2, &cand);
    if (s != ncclSuccess) return s;
    a.raw = static_cast<const uint8_t*>(in.data());
    a.frames = static_cast<uint8_t*>(out.data());
    a.meta = out.frameMetadata();
    a.hist = hist.dataAs<uint32_t>();
    a.cand = cand.dataAs<uint16_t>();
    cudaStream_t st = ctx.stream();
    if (cudaMemsetAsync(a.hist, 0, (size_t)a.chunks * 256 * 4, st) != cudaSuccess) return ncclUnhandledCudaError;
    const int perChunk = (int)std::max<long>(1, std::min<long>((long)smCount() * 4 / a.chunks, (a.chunkBytes / 4 + kThreads - 1) / kThreads));
    ansHistKernel<<<dim3(perChunk, (unsigned)a.chunks), kThreads, 0, st>>>(a);
    ansTableKernel<<<(unsigned)a.chunks, 32, 0, st>>>(a);
    const int encCtas = (int)std::max<long>(1, std::min<long>((nb + kWarps - 1) / kWarps, (long)smCount() * 4 / a.chunks + 1));
    ansEncodeKernel<<<dim3(encCtas, (unsigned)a.chunks), kThreads, 0, st>>>(a);
    ansFinalizeKernel<<<(unsigned)a.chunks, 1024, 0, st>>>(a);
    if (cudaGetLastError() != cudaSuccess) return ncclUnhandledCudaError;
    return out.commitFrames();
  }

  static Status decompress(const coccl::Input& in, coccl::Output& out, coccl::Context& ctx) {
    const size_t raw = out.elements() * coccl::dataTypeSize(out.datatype());
    if (coccl::isPassthrough(in)) {
      if (in.bytes() != raw) return ncclInvalidArgument;
      if (in.data() != out.data() &&
          cudaMemcpyAsync(out.data(), in.data(), in.bytes(), cudaMemcpyDeviceToDevice, ctx.stream()) != cudaSuccess)
        return ncclUnhandledCudaError;
      return out.commitPlanned();
    }
    if (!in.framed() || !shapeOk(raw, out.chunks()) || in.chunks() != out.chunks()) return ncclInvalidArgument;
    AnsArgs a{};
    a.chunks = (long)out.chunks();
    a.chunkBytes = (long)(raw / out.chunks());
    a.frameStride = (long)in.frameStrideBytes();
    a.probBits = ctx.config<Config>().probBits;
    a.raw = static_cast<const uint8_t*>(out.data());
    a.frames = static_cast<uint8_t*>(const_cast<void*>(in.data()));
    a.meta = const_cast<cocclCompressorFrameMetadata*>(in.frameMetadata());
    const uint32_t nb = numBlocks((uint32_t)a.chunkBytes);
    const int ctas = (int)std::max<long>(1, std::min<long>((nb + kWarps - 1) / kWarps, (long)smCount() * 4 / a.chunks + 1));
    ansDecodeKernel<<<dim3(ctas, (unsigned)a.chunks), kThreads, 0, ctx.stream()>>>(a);
    if (cudaGetLastError() != cudaSuccess) return ncclUnhandledCudaError;
    return out.commitPlanned();
  }
};
}  // namespace

COCCL_REGISTER_COMPRESSOR("ans", Ans)
