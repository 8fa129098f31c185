// Tile-level codecs shared by the standalone codec kernels, the plugin
// adapters and the fused collective kernels.
//
// A CTA of 256 threads owns a tile of 2048 consecutive elements of one chunk;
// every thread owns 8 consecutive elements in registers. A codec turns those
// registers into an `Enc` (packed payload words + the group parameters held by
// the group's first lane) that can be stored to any number of destinations
// (local scratch or a peer's receive slot), and back.
//
// Numerics follow the reference codecs:
//  * SDP4Bit group quantisation: symmetric scale=(2^(b-1)-1)/absmax, stored
//    parameter 1/scale, clamp to [-2^(b-1), 2^(b-1)-1]; asymmetric
//    scale=2^b/(max-min), offset=(max+min)/2
//    (sdp4bit/includes/quantization_utils.h:126-272), int4 pairs packed
//    low nibble first (sdp4bit/includes/quantization.h:18-21), optional
//    unnormalised 32-point Walsh-Hadamard on every aligned run of 32 elements,
//    undone by a second transform and a 1/32 factor
//    (sdp4bit/includes/fast_hadamard_transform_common.h:248-264).
//  * Stochastic rounding uses a counter-based hash keyed by (seed, element)
//    instead of the reference's per-element curand_init(clock())
//    (quantization_utils.h:153-174); only the error statistics are comparable.
//  * MX-FP8 (no counterpart in the reference; TACO, taco/taco.cu:89-295, is its
//    behavioural model): 32-element blocks, UE8M0 power-of-two scale chosen so
//    that the block maximum does not saturate, E4M3 payload.
//
// Encoded chunk layout (all codecs): [payload bytes of every group][parameters
// of every group]; the chunk is padded to whole groups in the encoded stream
// only. Encoded sizes equal the reference's (544 B for 1024 fp32 elements in
// 4 chunks at g128/q4, 576 B for 16-bit inputs;
// tests/coccl-tests/src/coccl_fixed_compressor_test.cc:97-105).
#pragma once
#include "common.cuh"
#include <cuda_fp8.h>

namespace coccl {

enum CodecKind : int { kCodecSdp4bit = 0, kCodecMxfp8 = 1, kCodecRaw = 2 };

struct CodecCfg {
  int kind;        // CodecKind
  int bits;        // 4 | 8 (sdp4bit); 8 (mxfp8)
  int group;       // elements per group; power of two in [8, 2048] for tile kernels
  int asym;        // sdp4bit: 1 = asymmetric
  int hadamard;    // sdp4bit: 1 = H32 rotation
  int stochastic;  // 1 = stochastic rounding, 0 = round to nearest even
  int paramBytes;  // bytes of parameters per group (4 | 8 sdp4bit, 1 mxfp8)
  uint32_t seed;
};

struct ChunkLayout {
  long count;         // elements in the chunk
  long groups;        // ceil(count / group)
  long payloadBytes;  // groups * group * bits / 8
  long totalBytes;    // payload + parameters (exact)
  long stride;        // distance between consecutive chunks (>= totalBytes)
};

__host__ __device__ inline long alignUp(long x, long a) { return (x + a - 1) / a * a; }

__host__ __device__ inline ChunkLayout makeChunkLayout(const CodecCfg& c, long count, long strideAlign) {
  ChunkLayout L;
  L.count = count;
  L.groups = (count + c.group - 1) / c.group;
  L.payloadBytes = L.groups * (long)c.group * c.bits / 8;
  L.totalBytes = alignUp(L.payloadBytes + L.groups * c.paramBytes, 4);
  L.stride = alignUp(L.totalBytes, strideAlign);
  return L;
}

struct Enc {
  uint32_t w[2];  // payload: 4-bit -> w[0]; 8-bit / fp8 -> w[0..1]
  float p0, p1;   // group parameters (valid on the group's first lane)
};

// ------------------------------------------------------------------ helpers
__device__ __forceinline__ void hadamard8(float (&v)[8]) {
#pragma unroll
  for (int s = 1; s < 8; s <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if ((i & s) == 0) {
        float a = v[i], b = v[i | s];
        v[i] = a + b;
        v[i | s] = a - b;
      }
    }
  }
}
// 32-point unnormalised WHT over 4 adjacent lanes x 8 registers.
__device__ __forceinline__ void hadamard32(float (&v)[8]) {
  hadamard8(v);
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int s = 1; s <= 2; s <<= 1) {
    const bool upper = (lane & s) != 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float o = __shfl_xor_sync(0xffffffffu, v[i], s);
      v[i] = upper ? (o - v[i]) : (v[i] + o);
    }
  }
}

// Reduce over the `lpg` consecutive threads that share a group (lpg = group/8,
// a power of two <= 256). For lpg > 32 the CTA cooperates through `sm` (needs
// 2*8 floats) and every thread of the CTA must call this.
struct MaxOp { static __device__ __forceinline__ float f(float a, float b) { return fmaxf(a, b); } };
struct MinOp { static __device__ __forceinline__ float f(float a, float b) { return fminf(a, b); } };

template <class Op>
__device__ __forceinline__ float groupReduce(float x, int lpg, float* sm) {
  const int w = lpg < 32 ? lpg : 32;
  for (int o = 1; o < w; o <<= 1) x = Op::f(x, __shfl_xor_sync(0xffffffffu, x, o));
  if (lpg > 32) {
    const int warp = threadIdx.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sm[warp] = x;
    __syncthreads();
    const int wpg = lpg >> 5;
    const int base = warp / wpg * wpg;
    x = sm[base];
    for (int i = 1; i < wpg; ++i) x = Op::f(x, sm[base + i]);
  }
  return x;
}

__device__ __forceinline__ int quantRound(float y, bool stochastic, uint32_t word, int k) {
  if (stochastic) return (int)floorf(y + rngUnit(word, k));
  return __float2int_rn(y);
}

// ------------------------------------------------------------------ SDP4Bit
template <int BITS, bool ASYM, bool HAD>
struct SdpCodec {
  static constexpr int kBits = BITS;
  static constexpr int kWords = BITS / 4;  // u32 payload words per thread
  static constexpr bool kRotated = HAD;

  // v: 8 values of this thread (zero beyond the chunk). elem = chunk-relative
  // index of v[0]. `rotate=false` when v is already in the rotated domain.
  // rngElem = message-wide element index of v[0] (keys the rounding RNG).
  static __device__ __forceinline__ Enc encode(float (&v)[8], const CodecCfg& c, long elem,
                                               bool rotate, float* sm, uint64_t rngElem) {
    if (HAD && rotate) hadamard32(v);
    const int lpg = c.group >> 3;
    Enc e;
    float scale, offset = 0.f;
    constexpr float qmax = (float)((1 << (BITS - 1)) - 1);
    constexpr int qlo = -(1 << (BITS - 1)), qhi = (1 << (BITS - 1)) - 1;
    if (!ASYM) {
      float m = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
      m = groupReduce<MaxOp>(m, lpg, sm);
      scale = (m == 0.f) ? 1.f : qmax / m;
      e.p0 = 1.f / scale;
      e.p1 = 0.f;
    } else {
      float mx = v[0], mn = v[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) { mx = fmaxf(mx, v[i]); mn = fminf(mn, v[i]); }
      mx = groupReduce<MaxOp>(mx, lpg, sm);
      mn = groupReduce<MinOp>(mn, lpg, sm + 8);
      const float range = mx - mn;
      scale = (range == 0.f) ? 1.f : (float)(1 << BITS) / range;
      offset = 0.5f * (mx + mn);
      e.p0 = 1.f / scale;
      e.p1 = offset;
    }
    int q[8];
    const bool st = c.stochastic != 0;
    uint32_t r0 = 0, r1 = 0;
    if (st) {
      r0 = rngWord(c.seed, rngElem >> 2);
      r1 = rngWord(c.seed, (rngElem >> 2) + 1);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int t = quantRound((v[i] - offset) * scale, st, i < 4 ? r0 : r1, i & 3);
      q[i] = max(qlo, min(qhi, t));
    }
    if (BITS == 4) {
      uint32_t w = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) w |= ((uint32_t)(q[i] & 0xf)) << (4 * i);
      e.w[0] = w; e.w[1] = 0;
    } else {
      e.w[0] = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
      e.w[1] = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    }
    return e;
  }

  static __device__ __forceinline__ void store(const Enc& e, uint8_t* chunk, const ChunkLayout& L,
                                               const CodecCfg& c, long elem) {
    if (elem >= L.groups * c.group) return;
    uint32_t* pw = reinterpret_cast<uint32_t*>(chunk + elem * BITS / 8);
    pw[0] = e.w[0];
    if (BITS == 8) pw[1] = e.w[1];
    if ((elem & (c.group - 1)) == 0) {
      float* pp = reinterpret_cast<float*>(chunk + L.payloadBytes + (elem / c.group) * c.paramBytes);
      pp[0] = e.p0;
      if (c.paramBytes == 8) pp[1] = e.p1;
    }
  }

  // Dequantise 8 values (still rotated when HAD) and ADD them into acc.
  static __device__ __forceinline__ void loadAdd(const uint8_t* chunk, const ChunkLayout& L,
                                                 const CodecCfg& c, long elem, float (&acc)[8]) {
    if (elem >= L.groups * c.group) return;
    const uint32_t* pw = reinterpret_cast<const uint32_t*>(chunk + elem * BITS / 8);
    const float* pp = reinterpret_cast<const float*>(chunk + L.payloadBytes + (elem / c.group) * c.paramBytes);
    // __ldcg: the bytes may have been written by a peer GPU during this launch
    const float inv = __ldcg(pp);
    const float off = ASYM ? __ldcg(pp + 1) : 0.f;
    if (BITS == 4) {
      const uint32_t w = __ldcg(pw);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        int q = (int)(w << (28 - 4 * i)) >> 28;
        acc[i] += (float)q * inv + off;
      }
    } else {
      const uint32_t w0 = __ldcg(pw), w1 = __ldcg(pw + 1);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[i] += (float)((int)(w0 << (24 - 8 * i)) >> 24) * inv + off;
        acc[4 + i] += (float)((int)(w1 << (24 - 8 * i)) >> 24) * inv + off;
      }
    }
  }

  // Leave the rotated domain (after any reduction: the transform is linear).
  static __device__ __forceinline__ void finish(float (&v)[8]) {
    if (HAD) {
      hadamard32(v);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] *= (1.f / 32.f);
    }
  }
};

// ------------------------------------------------------------------ MX-FP8
struct MxFp8Codec {
  static constexpr int kBits = 8;
  static constexpr int kWords = 2;
  static constexpr bool kRotated = false;

  static __device__ __forceinline__ Enc encode(float (&v)[8], const CodecCfg& c, long elem,
                                               bool /*rotate*/, float* /*sm*/, uint64_t /*rngElem*/) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    // UE8M0: smallest power of two s with m / s <= 448.
    int biased = 0;
    if (m > 0.f && m < INFINITY) {
      const float r = m * (1.f / 448.f);
      const uint32_t rb = __float_as_uint(r);
      int ex = (int)((rb >> 23) & 0xff);
      if (rb & 0x7fffffu) ex += 1;
      biased = max(0, min(254, ex));
    }
    // 2^-(biased-127) as a float: exponent field 254 - biased (denormal-safe for biased in [1,253]).
    const int invExp = 254 - biased;
    const float inv = invExp > 0 ? __uint_as_float((uint32_t)invExp << 23)
                                 : __uint_as_float(0x00400000u);  // 2^-127
    Enc e;
    uint16_t h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      h[i] = __nv_cvt_float2_to_fp8x2(make_float2(v[2 * i] * inv, v[2 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    e.w[0] = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
    e.w[1] = (uint32_t)h[2] | ((uint32_t)h[3] << 16);
    e.p0 = __uint_as_float((uint32_t)biased);  // carries the scale byte
    e.p1 = 0.f;
    return e;
  }

  // Every lane of the warp must call this (it shuffles), valid or not.
  static __device__ __forceinline__ void store(const Enc& e, uint8_t* chunk, const ChunkLayout& L,
                                               const CodecCfg& c, long elem) {
    const bool valid = elem < L.groups * 32;
    if (valid) {
      uint32_t* pw = reinterpret_cast<uint32_t*>(chunk + elem);
      pw[0] = e.w[0];
      pw[1] = e.w[1];
    }
    // Gather the 8 scale bytes of this warp's 8 blocks (lanes 0,4,..,28) into
    // lane 0 and write them with one 8-byte-aligned store when possible.
    uint32_t b = __float_as_uint(e.p0) & 0xffu;
    uint32_t t = b | (__shfl_down_sync(0xffffffffu, b, 4) << 8);
    t = t | (__shfl_down_sync(0xffffffffu, t, 8) << 16);
    uint32_t hi = __shfl_down_sync(0xffffffffu, t, 16);
    if ((threadIdx.x & 31) == 0 && valid) {
      uint8_t* ps = chunk + L.payloadBytes + elem / 32;
      const long left = L.groups - elem / 32;
      if (left >= 8 && ((reinterpret_cast<uintptr_t>(ps) & 7u) == 0)) {
        *reinterpret_cast<uint2*>(ps) = make_uint2(t, hi);
      } else {
        for (int i = 0; i < 8 && i < left; ++i) ps[i] = (uint8_t)((i < 4 ? t >> (8 * i) : hi >> (8 * (i - 4))) & 0xff);
      }
    }
  }

  static __device__ __forceinline__ void loadAdd(const uint8_t* chunk, const ChunkLayout& L,
                                                 const CodecCfg& c, long elem, float (&acc)[8]) {
    if (elem >= L.groups * 32) return;
    const uint32_t* pw = reinterpret_cast<const uint32_t*>(chunk + elem);
    const uint32_t w[2] = {__ldcg(pw), __ldcg(pw + 1)};
    const uint32_t biased = __ldcg(chunk + L.payloadBytes + elem / 32);
    const float scale = biased > 0 ? __uint_as_float(biased << 23) : __uint_as_float(0x00400000u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint16_t pair = (uint16_t)(w[i >> 1] >> (16 * (i & 1)));
      __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
      float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
      acc[2 * i] += f.x * scale;
      acc[2 * i + 1] += f.y * scale;
    }
  }

  static __device__ __forceinline__ void finish(float (&)[8]) {}
};

// Dispatch a generic lambda on the runtime codec configuration. The functor
// receives a codec type tag; unsupported configurations return false.
template <class F>
inline bool dispatchCodec(const CodecCfg& c, F&& f) {
  if (c.kind == kCodecMxfp8) { f(MxFp8Codec{}); return true; }
  if (c.kind != kCodecSdp4bit) return false;
#define COCCL_SDP_CASE(B, A, H) \
  if (c.bits == B && (c.asym != 0) == A && (c.hadamard != 0) == H) { f(SdpCodec<B, A, H>{}); return true; }
  COCCL_SDP_CASE(4, false, true)
  COCCL_SDP_CASE(4, false, false)
  COCCL_SDP_CASE(8, false, true)
  COCCL_SDP_CASE(8, false, false)
  COCCL_SDP_CASE(4, true, true)
  COCCL_SDP_CASE(4, true, false)
  COCCL_SDP_CASE(8, true, true)
  COCCL_SDP_CASE(8, true, false)
#undef COCCL_SDP_CASE
  return false;
}

inline bool tileCodecSupported(const CodecCfg& c) {
  if (c.kind == kCodecMxfp8) return c.group == 32;
  if (c.kind != kCodecSdp4bit) return false;
  if (c.group < 8 || c.group > 2048 || (c.group & (c.group - 1))) return false;
  if (c.hadamard && c.group < 32) return false;
  return c.bits == 4 || c.bits == 8;
}

}  // namespace coccl
