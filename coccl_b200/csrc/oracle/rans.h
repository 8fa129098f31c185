// Byte-wise rANS with 32 interleaved lanes per 4096-byte block: constants and the scalar steps shared by the
// device kernels of the ans plugin and the CPU oracle.
//
// Behavioural model: the reference's dietGPU codec (dietgpu/vendor/dietgpu/dietgpu/ans/GpuANSEncode.cuh:49-92,
// GpuANSUtils.cuh:67-228): 31-bit state, 16-bit renormalisation words, probabilities quantised to
// 2^probBits, one frame per chunk that stays decodable on its own. The frame layout here is this library's own:
//   FrameHeader (32 B) | u16 pdf[256] | u32 finalState[numBlocks][32] | u32 blockWords[numBlocks] |
//   u32 blockStart[numBlocks] (in u16 words, multiple of 8) | u16 streams...
// Lane l of a block codes bytes l, l+32, l+64, ... in order; at step j the lanes that renormalise append their
// 16-bit words in lane order. The decoder walks the steps backwards and pops the same words from the end.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define COCCL_RANS_HD __host__ __device__ __forceinline__
#else
#define COCCL_RANS_HD inline
#endif

namespace coccl {
namespace rans {

constexpr uint32_t kMagic = 0xC0CCA115u;
constexpr int kBlockBytes = 4096;
constexpr int kLanes = 32;
constexpr int kStepsPerBlock = kBlockBytes / kLanes;
constexpr uint32_t kLower = 1u << 15;  // state stays in [2^15, 2^31)
constexpr int kMaxBlockWords = kBlockBytes / 2 + kBlockBytes / 8;  // candidate slot per block (u16 words)

struct FrameHeader {
  uint32_t magic;
  uint32_t numBlocks;
  uint32_t rawBytes;
  uint32_t totalWords;   // u16 words in all block streams (with alignment padding)
  uint32_t probBits;
  uint32_t reserved[3];
};
static_assert(sizeof(FrameHeader) == 32, "frame header is a 32-byte wire contract");

COCCL_RANS_HD uint32_t numBlocks(uint32_t rawBytes) { return (rawBytes + kBlockBytes - 1) / kBlockBytes; }
// bytes before the first stream word
COCCL_RANS_HD uint32_t headerBytes(uint32_t blocks) {
  const uint32_t b = 32 + 512 + blocks * (kLanes * 4 + 8);
  return (b + 15) & ~15u;
}
// worst-case encoded frame (the plugin falls back to raw bytes when the coded frame is not smaller)
COCCL_RANS_HD uint64_t frameBound(uint64_t rawBytes) {
  const uint64_t blocks = (rawBytes + kBlockBytes - 1) / kBlockBytes;
  return ((uint64_t)headerBytes((uint32_t)blocks) + blocks * kMaxBlockWords * 2 + 31) & ~31ull;
}

// Encoder step for a symbol with frequency f and cumulative start c. Returns true when `word` must be emitted.
COCCL_RANS_HD bool encodeStep(uint32_t& state, uint32_t f, uint32_t c, int probBits, uint16_t& word) {
  bool emit = false;
  if (state >= (f << (31 - probBits))) {
    word = (uint16_t)(state & 0xffffu);
    state >>= 16;
    emit = true;
  }
  state = ((state / f) << probBits) + (state % f) + c;
  return emit;
}
// Decoder step, first half: undo the state update for the symbol found at slot = state & mask.
COCCL_RANS_HD bool decodeStep(uint32_t& state, uint32_t f, uint32_t c, int probBits) {
  const uint32_t mask = (1u << probBits) - 1;
  state = f * (state >> probBits) + (state & mask) - c;
  return state < kLower;  // true: the encoder renormalised here, the caller must pop a word
}

// Quantise a byte histogram to frequencies that sum to 2^probBits, every present symbol >= 1.
COCCL_RANS_HD void normalise(const uint32_t* hist, uint32_t total, int probBits, uint16_t* pdf) {
  const uint32_t target = 1u << probBits;
  uint32_t sum = 0;
  int best = 0;
  for (int i = 0; i < 256; ++i) {
    uint32_t f = 0;
    if (hist[i]) {
      f = (uint32_t)(((uint64_t)hist[i] * target) / (total ? total : 1));
      if (f == 0) f = 1;
    }
    pdf[i] = (uint16_t)f;
    sum += f;
    if (hist[i] > hist[best]) best = i;
  }
  if (total == 0) { pdf[0] = (uint16_t)target; return; }
  // settle the rounding on the largest entries
  while (sum != target) {
    if (sum < target) { pdf[best] = (uint16_t)(pdf[best] + (target - sum)); sum = target; }
    else {
      int big = 0;
      for (int i = 1; i < 256; ++i) if (pdf[i] > pdf[big]) big = i;
      const uint32_t take = (sum - target) < (uint32_t)(pdf[big] - 1) ? (sum - target) : (uint32_t)(pdf[big] - 1);
      if (take == 0) break;
      pdf[big] = (uint16_t)(pdf[big] - take);
      sum -= take;
    }
  }
}

}  // namespace rans
}  // namespace coccl
