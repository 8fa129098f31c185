// Tile-level codecs shared by the standalone codec kernels, the plugin adapters and the fused
// collective kernels.
//
// A CTA of 256 threads owns a tile of 8192 consecutive elements of one chunk; every thread owns one
// aligned run of 32 elements in registers (tile_io.cuh). A codec turns a run into an `Enc` (packed payload
// words + the parameters of the groups that start in the run) that can be stored to any number of
// destinations (local scratch or a peer's receive slot), and back.
//
// Numerics follow the reference codecs:
//  * SDP4Bit group quantisation: symmetric scale=(2^(b-1)-1)/absmax, stored parameter 1/scale, clamp to
//    [-2^(b-1), 2^(b-1)-1]; asymmetric scale=2^b/(max-min), offset=(max+min)/2
//    (sdp4bit/includes/quantization_utils.h:126-272), int4 pairs packed low nibble first
//    (sdp4bit/includes/quantization.h:18-21), optional unnormalised 32-point Walsh-Hadamard on every
//    aligned run of 32 elements, undone by a second transform and a 1/32 factor
//    (sdp4bit/includes/fast_hadamard_transform_common.h:248-264).
//  * Stochastic rounding uses a counter-based hash keyed by (seed, element) instead of the reference's
//    per-element curand_init(clock()) (quantization_utils.h:153-174); only the error statistics are
//    comparable.
//  * MX-FP8 (no counterpart in the reference; TACO, taco/taco.cu:89-295, is its behavioural model):
//    32-element blocks, UE8M0 power-of-two scale chosen so that the block maximum does not saturate, E4M3
//    payload.
//
// Float <-> integer conversions go through the mantissa ("magic number") instead of the conversion unit:
// adding 1.5 * 2^23 to y leaves round-to-nearest-even(y) in the low mantissa bits, and OR-ing an integer
// n < 2^23 into the bits of 2^23 gives the float 2^23 + n. Packing eight 4-bit values is then one
// multiply-add chain over the raw float bits: sum(bits_i * 16^i) = C + sum(q_i * 16^i), and adding
// 0x88888888 turns the signed digits into offset-binary nibbles, which differ from two's-complement nibbles
// by the XOR 0x88888888.
//
// Encoded chunk layout (all codecs): [payload bytes of every group][parameters of every group]; the chunk is
// padded to whole groups in the encoded stream only. Encoded sizes equal the reference's (544 B for 1024
// fp32 elements in 4 chunks at g128/q4, 576 B for 16-bit inputs;
// tests/coccl-tests/src/coccl_fixed_compressor_test.cc:97-105).
#pragma once
#include "common.cuh"
#include "oracle/zfp1d.h"
#include <cuda_fp8.h>

namespace coccl {

enum CodecKind : int { kCodecSdp4bit = 0, kCodecMxfp8 = 1, kCodecRaw = 2, kCodecTaco = 3, kCodecZfp = 4 };

struct CodecCfg {
  int kind;        // CodecKind
  int bits;        // 4 | 8 (sdp4bit); 8 (mxfp8)
  int group;       // elements per group; power of two in [8, 2048] for tile kernels
  int asym;        // sdp4bit: 1 = asymmetric
  int hadamard;    // sdp4bit: 1 = H32 rotation
  int stochastic;  // 1 = stochastic rounding, 0 = round to nearest even
  int paramBytes;  // bytes of parameters per group (4 | 8 sdp4bit, 1 mxfp8, 8 taco, 0 zfp)
  uint32_t seed;
  int aux;         // taco: bit 0 = E5M2 payload, bit 1 = saturating conversion
  float f0, f1, f2;  // taco: targetRange, lambda, fp8 maximum
};
// taco: bits = 8, group = 32..512. zfp: bits = rate (bits per value), group = 4 (one block).

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

// ------------------------------------------------------------------ bounds-checked build
// With -DCOCCL_BOUNDS_CHECK (libcoccl_checked.so) every access of a codec to an encoded chunk is preceded by a check
// of the byte ranges it is about to touch against the chunk's layout: the payload part must end inside the payload,
// the parameter part inside the chunk. A violation records {site, element, offending end, limit} once in a device
// word that the host reads (cocclkBoundsWord) and the access is SKIPPED, so a wrong index shows up as an error word
// and wrong numbers, never as a fault. The normal build compiles the checks away.
#ifdef COCCL_BOUNDS_CHECK
static __device__ unsigned int gBoundsWord[8];   // one per translation unit; each checked unit exports a reader
__device__ __forceinline__ bool chunkRangeOk(const ChunkLayout& L, long elem, long payloadEnd, long totalEnd, int site) {
  if (elem >= 0 && payloadEnd <= L.payloadBytes && totalEnd <= L.totalBytes && L.totalBytes <= L.stride) return true;
  if (atomicCAS(&gBoundsWord[0], 0u, 0x80000000u | (unsigned)site) == 0u) {
    gBoundsWord[1] = (unsigned)elem; gBoundsWord[2] = (unsigned)((unsigned long long)elem >> 32);
    gBoundsWord[3] = (unsigned)payloadEnd; gBoundsWord[4] = (unsigned)L.payloadBytes;
    gBoundsWord[5] = (unsigned)totalEnd; gBoundsWord[6] = (unsigned)L.totalBytes;
  }
  return false;
}
#define COCCL_CHUNK_RANGE_OK(Codec, L, c, elem, site) \
  ([&] { long pe_, te_; Codec::touched(L, c, elem, &pe_, &te_); return chunkRangeOk(L, elem, pe_, te_, site); }())
#else
#define COCCL_CHUNK_RANGE_OK(Codec, L, c, elem, site) true
#endif

// ------------------------------------------------------------------ helpers
// Unnormalised 32-point Walsh-Hadamard transform of one run, entirely in registers.
__device__ __forceinline__ void hadamard32(float (&v)[32]) {
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if ((i & s) == 0) {
        const float a = v[i], b = v[i | s];
        v[i] = a + b;
        v[i | s] = a - b;
      }
    }
  }
}

// Reduce over the `lpg` consecutive threads that share a group (lpg = group/32, a power of two <= 64).
// For lpg > 32 the CTA cooperates through `sm` (8 floats) and every thread of the CTA must call this.
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
    x = Op::f(sm[warp & ~1], sm[warp | 1]);
  }
  return x;
}

constexpr float kRoundMagic = 12582912.f;          // 1.5 * 2^23
constexpr uint32_t kRoundMagicBits = 0x4B400000u;  // its bit pattern
constexpr uint32_t kIntMagicBits = 0x4B000000u;    // 2^23: OR an integer < 2^23 into the mantissa

// (u - 0.5) for the k-th byte of a random word, u = (byte + 0.5) / 256, built in the mantissa of [1, 2).
__device__ __forceinline__ float rngCentered(uint32_t word, int k) {
  const uint32_t b = (word >> (8 * k)) & 0xffu;
  return __uint_as_float(0x3F800000u | (b << 15)) - 1.498046875f;
}

// ------------------------------------------------------------------ SDP4Bit
// SMALLG: groups of 8 or 16 elements (several per run, no rotation); otherwise group >= 32.
template <int BITS, bool ASYM, bool HAD, bool SMALLG>
struct SdpCodec {
  static_assert(!(HAD && SMALLG), "the rotation needs groups of at least one run");
  static constexpr int kBits = BITS;
  static constexpr int kWords = BITS;          // payload words per run
  static constexpr int kPerWord = 32 / BITS;   // elements per payload word
  static constexpr int kParams = SMALLG ? 4 : 1;
  static constexpr bool kRotated = HAD;
  static constexpr int kMinBlocks = 3;  // resident CTAs per SM the fused kernels are compiled for
  static constexpr int kSmemFloats = 8; // shared scratch every kernel passes as `sm` (group reductions wider than a warp)
  static __device__ __forceinline__ void initShared(float*) {}
  static constexpr uint32_t kSignBits = BITS == 4 ? 0x88888888u : 0x80808080u;
  static constexpr uint32_t kPackFix = kSignBits - kRoundMagicBits * (BITS == 4 ? 0x11111111u : 0x01010101u);

  struct Enc {
    uint32_t w[kWords];
    float p0[kParams], p1[kParams];
  };

  template <bool ST>
  static __device__ __forceinline__ void quantise(const float (&v)[32], const float (&scale)[kParams],
                                                  const float (&offset)[kParams], const CodecCfg& c,
                                                  uint64_t rngElem, Enc& e) {
    constexpr float qlo = (float)(-(1 << (BITS - 1))), qhi = (float)((1 << (BITS - 1)) - 1);
    uint32_t rw[8];
    if (ST) {
#pragma unroll
      for (int k = 0; k < 8; ++k) rw[k] = rngWord(c.seed, (rngElem >> 2) + k);
    }
#pragma unroll
    for (int k = 0; k < kWords; ++k) {
      uint32_t acc = 0;
#pragma unroll
      for (int i = kPerWord - 1; i >= 0; --i) {
        const int idx = k * kPerWord + i;
        const int pj = SMALLG ? idx / 8 : 0;
        // the product is rounded to fp32 before the rounding to an integer, as in the reference (no fma)
        float y = __fmul_rn(ASYM ? v[idx] - offset[pj] : v[idx], scale[pj]);
        if (ST) y = __fadd_rn(y, rngCentered(rw[idx >> 2], idx & 3));
        // symmetric: |y| <= 2^(b-1)-1 by construction; asymmetric: the top of the range rounds to 2^(b-1)
        if (ASYM) y = fminf(fmaxf(y, qlo), qhi);
        const uint32_t b = __float_as_uint(__fadd_rn(y, kRoundMagic));
        acc = (i == kPerWord - 1) ? b : acc * (1u << BITS) + b;
      }
      e.w[k] = (acc + kPackFix) ^ kSignBits;
    }
  }

  static __device__ __forceinline__ void params(float mx, float mn, float& scale, float& offset, float& p0, float& p1) {
    constexpr float qmax = (float)((1 << (BITS - 1)) - 1);
    if (!ASYM) {
      scale = (mx == 0.f) ? 1.f : qmax / mx;
      offset = 0.f;
    } else {
      const float range = mx - mn;
      scale = (range == 0.f) ? 1.f : (float)(1 << BITS) / range;
      offset = 0.5f * (mx + mn);
    }
    p0 = 1.f / scale;
    p1 = offset;
  }

  // v: the run of this thread (zero beyond the chunk). `rotate=false` when v is already in the rotated
  // domain. rngElem = message-wide element index of v[0] (keys the rounding RNG).
  static __device__ __forceinline__ Enc encode(float (&v)[32], const CodecCfg& c, bool rotate, float* sm,
                                               uint64_t rngElem) {
    if (HAD && rotate) hadamard32(v);
    Enc e;
    float scale[kParams], offset[kParams];
    if (!SMALLG) {
      float mx, mn = 0.f;
      if (!ASYM) {
        mx = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fabsf(v[i]));
        mx = groupReduce<MaxOp>(mx, c.group >> 5, sm);
      } else {
        mx = v[0]; mn = v[0];
#pragma unroll
        for (int i = 1; i < 32; ++i) { mx = fmaxf(mx, v[i]); mn = fminf(mn, v[i]); }
        mx = groupReduce<MaxOp>(mx, c.group >> 5, sm);
        mn = groupReduce<MinOp>(mn, c.group >> 5, sm);
      }
      params(mx, mn, scale[0], offset[0], e.p0[0], e.p1[0]);
    } else {
      float mx[4], mn[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (!ASYM) {
          mx[j] = 0.f; mn[j] = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) mx[j] = fmaxf(mx[j], fabsf(v[8 * j + i]));
        } else {
          mx[j] = v[8 * j]; mn[j] = v[8 * j];
#pragma unroll
          for (int i = 1; i < 8; ++i) { mx[j] = fmaxf(mx[j], v[8 * j + i]); mn[j] = fminf(mn[j], v[8 * j + i]); }
        }
      }
      if (c.group == 16) {
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
          mx[j] = mx[j + 1] = fmaxf(mx[j], mx[j + 1]);
          mn[j] = mn[j + 1] = fminf(mn[j], mn[j + 1]);
        }
      }
#pragma unroll
      for (int j = 0; j < kParams; ++j) params(mx[j], mn[j], scale[j], offset[j], e.p0[j], e.p1[j]);
    }
    if (c.stochastic) quantise<true>(v, scale, offset, c, rngElem, e);
    else quantise<false>(v, scale, offset, c, rngElem, e);
    return e;
  }

  // Exclusive ends of the payload bytes and of the parameter bytes that store / fetch touch for the run at `elem`
  // (0 when the run lies in the padding and nothing is touched); used by the bounds-checked build.
  static __device__ __forceinline__ void touched(const ChunkLayout& L, const CodecCfg& c, long elem, long* payloadEnd, long* totalEnd) {
    const int gs = 31 - __clz(c.group);
    const long padded = L.groups << gs;
    if (elem >= padded) { *payloadEnd = 0; *totalEnd = 0; return; }
    const long last = elem + 32 < padded ? elem + 32 : padded;
    *payloadEnd = last * BITS / 8;
    long g = (last - 1) >> gs;
    if (g >= L.groups) g = L.groups - 1;
    *totalEnd = L.payloadBytes + (g + 1) * c.paramBytes;
  }

  // elem = chunk-relative index of the run's first element
  static __device__ __forceinline__ void store(const Enc& e, uint8_t* chunk, const ChunkLayout& L,
                                               const CodecCfg& c, long elem) {
    const int gs = 31 - __clz(c.group);  // the group size is a power of two
    const long padded = L.groups << gs;
    if (elem >= padded) return;
    uint8_t* pw = chunk + elem * BITS / 8;
    if (elem + 32 <= padded && aligned16(pw)) {
#pragma unroll
      for (int q = 0; q < kWords / 4; ++q)
        reinterpret_cast<uint4*>(pw)[q] = make_uint4(e.w[4 * q], e.w[4 * q + 1], e.w[4 * q + 2], e.w[4 * q + 3]);
    } else {
#pragma unroll
      for (int k = 0; k < kWords; ++k)
        if (elem + k * kPerWord < padded) reinterpret_cast<uint32_t*>(pw)[k] = e.w[k];
    }
    uint8_t* pbase = chunk + L.payloadBytes;
    if (!SMALLG) {
      if ((elem & (c.group - 1)) == 0) {
        float* pp = reinterpret_cast<float*>(pbase + (elem >> gs) * c.paramBytes);
        pp[0] = e.p0[0];
        if (c.paramBytes == 8) pp[1] = e.p1[0];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long ge = elem + 8 * j;
        if ((ge & (c.group - 1)) == 0 && ge < padded) {
          float* pp = reinterpret_cast<float*>(pbase + (ge >> gs) * c.paramBytes);
          pp[0] = e.p0[j];
          if (c.paramBytes == 8) pp[1] = e.p1[j];
        }
      }
    }
  }

  // Encoded run as fetched from memory; `accumulate` dequantises it. Splitting the two lets a reduction
  // keep the loads of several sources in flight.
  struct Raw {
    uint32_t w[kWords];
    float inv[kParams], off[kParams];
    bool valid;
  };
  static constexpr int kBatch = 2;

  // `mul` scales the dequantised values (a power of two: exact); decoders that leave the rotated domain
  // right afterwards pass 1/32 here instead of multiplying all 32 outputs.
  static __device__ __forceinline__ Raw fetch(const uint8_t* chunk, const ChunkLayout& L, const CodecCfg& c, long elem,
                                              float mul, const float* /*sm*/ = nullptr) {
    Raw r;
    const int gs = 31 - __clz(c.group);
    const long padded = L.groups << gs;
    r.valid = elem < padded;
    if (!r.valid) return r;
    // __ldcg: the bytes may have been written by a peer GPU during this launch
    const uint8_t* pw = chunk + elem * BITS / 8;
    if (elem + 32 <= padded && aligned16(pw)) {
#pragma unroll
      for (int q = 0; q < kWords / 4; ++q) {
        const uint4 t = __ldcg(reinterpret_cast<const uint4*>(pw) + q);
        r.w[4 * q] = t.x; r.w[4 * q + 1] = t.y; r.w[4 * q + 2] = t.z; r.w[4 * q + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int k = 0; k < kWords; ++k)
        r.w[k] = (elem + k * kPerWord < padded) ? __ldcg(reinterpret_cast<const uint32_t*>(pw) + k) : 0u;
    }
    const uint8_t* pbase = chunk + L.payloadBytes;
#pragma unroll
    for (int j = 0; j < kParams; ++j) {
      long g = (elem + 8 * j) >> gs;
      if (g >= L.groups) g = L.groups - 1;
      const float* pp = reinterpret_cast<const float*>(pbase + g * c.paramBytes);
      r.inv[j] = __ldcg(pp) * mul;
      r.off[j] = ASYM ? __ldcg(pp + 1) * mul : 0.f;
    }
    return r;
  }

  // Dequantise the run (still rotated when HAD) and ADD it into acc.
  static __device__ __forceinline__ void accumulate(const Raw& r, float (&acc)[32]) {
    if (!r.valid) return;
#pragma unroll
    for (int k = 0; k < kWords; ++k) {
      const uint32_t x = r.w[k] ^ kSignBits;  // offset-binary digits: q + 2^(b-1)
#pragma unroll
      for (int i = 0; i < kPerWord; ++i) {
        const int idx = k * kPerWord + i;
        const int pj = SMALLG ? idx / 8 : 0;
        float f;
        if (BITS == 4) {
          const uint32_t m = ((x >> (4 * i)) & 0xfu) | kIntMagicBits;
          f = __uint_as_float(m) - 8388616.f;  // 2^23 + 8
        } else {
          const uint32_t m = __byte_perm(x, kIntMagicBits, 0x7650 + i);
          f = __uint_as_float(m) - 8388736.f;  // 2^23 + 128
        }
        if (ASYM) acc[idx] += fmaf(f, r.inv[pj], r.off[pj]);
        else acc[idx] = fmaf(f, r.inv[pj], acc[idx]);
      }
    }
  }

  // Leave the rotated domain (after any reduction: the transform is linear). The 1/32 of the inverse
  // transform was applied by fetch (kFinishScale).
  static __device__ __forceinline__ float finishScale(const CodecCfg&) { return HAD ? 1.f / 32.f : 1.f; }
  static __device__ __forceinline__ void finish(float (&v)[32], const CodecCfg&) {
    if (HAD) hadamard32(v);
  }
};

// ------------------------------------------------------------------ MX-FP8
// One 32-element block per run: the scale needs no cross-lane traffic at all.
struct MxFp8Codec {
  static constexpr int kBits = 8;
  static constexpr int kWords = 8;
  static constexpr bool kRotated = false;
  static constexpr int kMinBlocks = 3;
  static constexpr int kSmemFloats = 8;
  static __device__ __forceinline__ void initShared(float*) {}

  struct Enc {
    uint32_t w[8];
    uint32_t scaleByte;
  };

  static __device__ __forceinline__ Enc encode(float (&v)[32], const CodecCfg& /*c*/, bool /*rotate*/, float* /*sm*/,
                                               uint64_t /*rngElem*/) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) m = fmaxf(m, fabsf(v[i]));
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
    const float inv = invExp > 0 ? __uint_as_float((uint32_t)invExp << 23) : __uint_as_float(0x00400000u);  // 2^-127
    Enc e;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * k] * inv, v[4 * k + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * k + 2] * inv, v[4 * k + 3] * inv), __NV_SATFINITE, __NV_E4M3);
      e.w[k] = lo | (hi << 16);
    }
    e.scaleByte = (uint32_t)biased;
    return e;
  }

  static __device__ __forceinline__ void touched(const ChunkLayout& L, const CodecCfg&, long elem, long* payloadEnd, long* totalEnd) {
    if (elem >= L.groups * 32) { *payloadEnd = 0; *totalEnd = 0; return; }
    *payloadEnd = elem + 32;
    *totalEnd = L.payloadBytes + elem / 32 + 1;
  }

  static __device__ __forceinline__ void store(const Enc& e, uint8_t* chunk, const ChunkLayout& L, const CodecCfg& /*c*/,
                                               long elem) {
    if (elem >= L.groups * 32) return;
    uint8_t* pw = chunk + elem;
    if (aligned16(pw)) {
      reinterpret_cast<uint4*>(pw)[0] = make_uint4(e.w[0], e.w[1], e.w[2], e.w[3]);
      reinterpret_cast<uint4*>(pw)[1] = make_uint4(e.w[4], e.w[5], e.w[6], e.w[7]);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) reinterpret_cast<uint32_t*>(pw)[k] = e.w[k];
    }
    chunk[L.payloadBytes + elem / 32] = (uint8_t)e.scaleByte;
  }

  struct Raw {
    uint32_t w[8];
    uint32_t biased;
    bool valid;
  };
  static constexpr int kBatch = 2;

  static __device__ __forceinline__ Raw fetch(const uint8_t* chunk, const ChunkLayout& L, const CodecCfg& /*c*/, long elem,
                                              float /*mul*/, const float* /*sm*/ = nullptr) {
    Raw r;
    r.valid = elem < L.groups * 32;
    if (!r.valid) return r;
    const uint8_t* pw = chunk + elem;
    if (aligned16(pw)) {
      const uint4 a = __ldcg(reinterpret_cast<const uint4*>(pw)), b = __ldcg(reinterpret_cast<const uint4*>(pw) + 1);
      r.w[0] = a.x; r.w[1] = a.y; r.w[2] = a.z; r.w[3] = a.w; r.w[4] = b.x; r.w[5] = b.y; r.w[6] = b.z; r.w[7] = b.w;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) r.w[k] = __ldcg(reinterpret_cast<const uint32_t*>(pw) + k);
    }
    r.biased = __ldcg(chunk + L.payloadBytes + elem / 32);
    return r;
  }

  static __device__ __forceinline__ void accumulate(const Raw& r, float (&acc)[32]) {
    if (!r.valid) return;
    const float scale = r.biased > 0 ? __uint_as_float(r.biased << 23) : __uint_as_float(0x00400000u);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint16_t pair = (uint16_t)(r.w[k] >> (16 * h));
        __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
        acc[4 * k + 2 * h] = fmaf(f.x, scale, acc[4 * k + 2 * h]);
        acc[4 * k + 2 * h + 1] = fmaf(f.y, scale, acc[4 * k + 2 * h + 1]);
      }
    }
  }

  static __device__ __forceinline__ float finishScale(const CodecCfg&) { return 1.f; }
  static __device__ __forceinline__ void finish(float (&)[32], const CodecCfg&) {}
};

// ------------------------------------------------------------------ TACO
// Adaptive FP8 with a Walsh-Hadamard transform over the whole group (reference numerics: taco/taco.cu:118-218):
//   ada = clamp(fp8max * rsqrt(mean(x^2) + lambda), 1e-3, 1e3);  y = H_G(x * ada) / sqrt(G);
//   qs = clamp(max|y| / targetRange, 1e-12, 1e6);  code = fp8(clamp(y / qs, +-448));  x^ = H_G(code * qs) / sqrt(G) / ada
// Chunk layout as the reference's: [one fp8 byte per value of every (padded) group][groups x f32 qs][groups x f32 ada].
// A group is G/32 consecutive runs, i.e. G/32 adjacent lanes of one warp: the first five butterfly stages are
// register work, the rest and the group statistics are warp shuffles, so every lane of the warp must call
// encode() and finish() together. "Rotated domain" here is y / ada = H_G(x) / sqrt(G): independent of the
// sender's ada, so copies from different ranks add up there and one inverse transform serves the sum; the
// transform is orthonormal, so mean(x^2) for a re-encode is available without leaving the domain.
struct TacoCodec {
  static constexpr int kBits = 8;
  static constexpr int kWords = 8;
  static constexpr bool kRotated = true;
  static constexpr int kMinBlocks = 2;  // the lane butterflies keep two copies of a run live: 128 registers, no spills
  static constexpr int kSmemFloats = 8;
  static __device__ __forceinline__ void initShared(float*) {}

  struct Enc {
    uint32_t w[8];
    float qs, ada;
  };

  static __device__ __forceinline__ void lanes(float (&v)[32], int lpg) {
    const int lane = threadIdx.x & 31;
    for (int s = 1; s < lpg; s <<= 1) {
      const bool upper = (lane & s) != 0;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float o = __shfl_xor_sync(0xffffffffu, v[i], s);
        v[i] = upper ? o - v[i] : v[i] + o;
      }
    }
  }

  static __device__ __forceinline__ Enc encode(float (&v)[32], const CodecCfg& c, bool rotate, float* /*sm*/,
                                               uint64_t /*rngElem*/) {
    const int lpg = c.group >> 5;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) ss = fmaf(v[i], v[i], ss);
    for (int o = 1; o < lpg; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    Enc e;
    e.ada = fminf(fmaxf(c.f2 * rsqrtf(ss / (float)c.group + c.f1), 1e-3f), 1e3f);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= e.ada;
    if (rotate) {
      hadamard32(v);
      lanes(v, lpg);
      const float rsG = rsqrtf((float)c.group);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= rsG;
    }
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) m = fmaxf(m, fabsf(v[i]));
    for (int o = 1; o < lpg; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    e.qs = fminf(fmaxf(m / c.f0, 1e-12f), 1e6f);
    const float inv = 1.f / e.qs;
    const __nv_fp8_interpretation_t fmt = (c.aux & 1) ? __NV_E5M2 : __NV_E4M3;
    const __nv_saturation_t sat = (c.aux & 2) ? __NV_SATFINITE : __NV_NOSAT;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float q[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = fminf(fmaxf(v[4 * k + i] * inv, -448.f), 448.f);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q[0], q[1]), sat, fmt);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q[2], q[3]), sat, fmt);
      e.w[k] = lo | (hi << 16);
    }
    return e;
  }

  static __device__ __forceinline__ void touched(const ChunkLayout& L, const CodecCfg& c, long elem, long* payloadEnd, long* totalEnd) {
    if (elem >= L.payloadBytes) { *payloadEnd = 0; *totalEnd = 0; return; }
    *payloadEnd = elem + 32;
    *totalEnd = L.payloadBytes + (L.groups + elem / c.group + 1) * 4;   // the group's scale, then its adaptive factor
  }

  static __device__ __forceinline__ void store(const Enc& e, uint8_t* chunk, const ChunkLayout& L, const CodecCfg& c,
                                               long elem) {
    if (elem >= L.payloadBytes) return;  // runs of the padded last group are part of the stream
    uint8_t* pw = chunk + elem;
    if (aligned16(pw)) {
      reinterpret_cast<uint4*>(pw)[0] = make_uint4(e.w[0], e.w[1], e.w[2], e.w[3]);
      reinterpret_cast<uint4*>(pw)[1] = make_uint4(e.w[4], e.w[5], e.w[6], e.w[7]);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) reinterpret_cast<uint32_t*>(pw)[k] = e.w[k];
    }
    if ((elem & (c.group - 1)) == 0) {
      float* ps = reinterpret_cast<float*>(chunk + L.payloadBytes);
      const long g = elem / c.group;
      ps[g] = e.qs;
      ps[L.groups + g] = e.ada;
    }
  }

  struct Raw {
    uint32_t w[8];
    float scale;  // qs / ada (* mul)
    int e5m2;
    bool valid;
  };
  static constexpr int kBatch = 2;

  static __device__ __forceinline__ Raw fetch(const uint8_t* chunk, const ChunkLayout& L, const CodecCfg& c, long elem,
                                              float mul, const float* /*sm*/ = nullptr) {
    Raw r;
    r.valid = elem < L.payloadBytes;
    r.e5m2 = c.aux & 1;
    if (!r.valid) return r;
    const uint8_t* pw = chunk + elem;
    if (aligned16(pw)) {
      const uint4 a = __ldcg(reinterpret_cast<const uint4*>(pw)), b = __ldcg(reinterpret_cast<const uint4*>(pw) + 1);
      r.w[0] = a.x; r.w[1] = a.y; r.w[2] = a.z; r.w[3] = a.w; r.w[4] = b.x; r.w[5] = b.y; r.w[6] = b.z; r.w[7] = b.w;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) r.w[k] = __ldcg(reinterpret_cast<const uint32_t*>(pw) + k);
    }
    const float* ps = reinterpret_cast<const float*>(chunk + L.payloadBytes);
    const long g = elem / c.group;
    r.scale = __ldcg(ps + g) / __ldcg(ps + L.groups + g) * mul;
    return r;
  }

  static __device__ __forceinline__ void accumulate(const Raw& r, float (&acc)[32]) {
    if (!r.valid) return;
    const __nv_fp8_interpretation_t fmt = r.e5m2 ? __NV_E5M2 : __NV_E4M3;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(r.w[k] >> (16 * h)), fmt);
        const float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
        acc[4 * k + 2 * h] = fmaf(f.x, r.scale, acc[4 * k + 2 * h]);
        acc[4 * k + 2 * h + 1] = fmaf(f.y, r.scale, acc[4 * k + 2 * h + 1]);
      }
    }
  }

  static __device__ __forceinline__ float finishScale(const CodecCfg& c) { return rsqrtf((float)c.group); }
  static __device__ __forceinline__ void finish(float (&v)[32], const CodecCfg& c) {
    hadamard32(v);
    lanes(v, c.group >> 5);
  }
};

// ------------------------------------------------------------------ ZFP fixed rate, 1-D
// A run of 32 values is eight ZFP blocks of four; at RATE bits per value a block takes 4 * RATE bits
// (zfp/src/zfp.c:773-803) and the run exactly RATE 32-bit words, so a thread writes whole words of the stream and
// nothing is assembled across threads (the reference's encoder ORs blocks into a zeroed stream with atomics,
// zfp/src/cuda_zfp/encode.cuh:224-231). Block i of a chunk sits at bit i * 4 * RATE, as in the reference stream;
// the block coder is oracle/zfp1d.h, shared with the CPU oracle. Lossy re-encoding (two-shot all-reduce) simply
// encodes the decoded sum again: there is no separate domain.
template <int RATE>
struct ZfpCodec {
  static_assert(RATE == 4 || RATE == 8 || RATE == 16, "fused rates: 4, 8, 16 bits per value");
  static constexpr int kBits = RATE;
  static constexpr int kWords = RATE;
  static constexpr bool kRotated = false;
  static constexpr int kMinBlocks = 2;
  static constexpr int kMaxBits = 4 * RATE;
  // the plane tables of oracle/zfp1d.h live in the kernel's shared scratch, behind its first 8 floats
  static constexpr int kSmemFloats = 8 + (zfp1d::kPlaneEncEntries + zfp1d::kPlaneDecEntries) / 2;
  static __device__ __forceinline__ uint16_t* encTab(float* sm) { return reinterpret_cast<uint16_t*>(sm + 8); }
  static __device__ __forceinline__ const uint16_t* decTab(const float* sm) {
    return reinterpret_cast<const uint16_t*>(sm + 8) + zfp1d::kPlaneEncEntries;
  }
  // Every thread of the CTA calls this once, followed by a __syncthreads(), before any encode or fetch.
  static __device__ __forceinline__ void initShared(float* sm) {
    uint16_t* t = encTab(sm);
    for (int i = threadIdx.x; i < zfp1d::kPlaneEncEntries + zfp1d::kPlaneDecEntries; i += blockDim.x) {
      if (i < zfp1d::kPlaneEncEntries) t[i] = zfp1d::planeCode(i >> 4, (uint32_t)(i & 15));
      else t[i] = zfp1d::planeDecode((i - zfp1d::kPlaneEncEntries) >> 7, (uint32_t)((i - zfp1d::kPlaneEncEntries) & 127));
    }
  }

  struct Enc { uint32_t w[RATE]; };

  static __device__ __forceinline__ Enc encode(float (&v)[32], const CodecCfg& /*c*/, bool /*rotate*/, float* sm,
                                               uint64_t /*rngElem*/) {
    Enc e;
    const uint16_t* tab = encTab(sm);
    if (RATE == 4) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t lo = (uint32_t)zfp1d::encodeBlock64T(&v[8 * k], kMaxBits, tab);
        const uint32_t hi = (uint32_t)zfp1d::encodeBlock64T(&v[8 * k + 4], kMaxBits, tab);
        e.w[k] = lo | (hi << 16);
      }
    } else {
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        const uint64_t s = zfp1d::encodeBlock64T(&v[4 * b], kMaxBits, tab);
        if (RATE == 8) e.w[b] = (uint32_t)s;
        else { e.w[(2 * b) % RATE] = (uint32_t)s; e.w[(2 * b + 1) % RATE] = (uint32_t)(s >> 32); }
      }
    }
    return e;
  }

  static __device__ __forceinline__ void touched(const ChunkLayout& L, const CodecCfg&, long elem, long* payloadEnd, long* totalEnd) {
    const long off = (elem >> 5) * (4 * RATE);
    if (off >= L.totalBytes) { *payloadEnd = 0; *totalEnd = 0; return; }
    long end = off + 4 * RATE;
    if (end > L.totalBytes) end = L.totalBytes / 4 * 4;   // the tail is written word by word, whole words only
    *payloadEnd = end < L.payloadBytes ? end : L.payloadBytes;   // a ZFP chunk has no parameter part
    *totalEnd = end;
  }

  static __device__ __forceinline__ void store(const Enc& e, uint8_t* chunk, const ChunkLayout& L, const CodecCfg& /*c*/,
                                               long elem) {
    const long off = (elem >> 5) * (4 * RATE);
    if (off >= L.totalBytes) return;
    uint8_t* pw = chunk + off;
    if (off + 4 * RATE <= L.totalBytes && aligned16(pw)) {
#pragma unroll
      for (int q = 0; q < RATE / 4; ++q)
        reinterpret_cast<uint4*>(pw)[q] = make_uint4(e.w[4 * q], e.w[4 * q + 1], e.w[4 * q + 2], e.w[4 * q + 3]);
    } else {
#pragma unroll
      for (int k = 0; k < RATE; ++k)
        if (off + 4 * k + 4 <= L.totalBytes) reinterpret_cast<uint32_t*>(pw)[k] = e.w[k];
    }
  }

  struct Raw {
    uint32_t w[RATE];
    const uint16_t* tab;
    bool valid;
  };
  static constexpr int kBatch = 1;

  static __device__ __forceinline__ Raw fetch(const uint8_t* chunk, const ChunkLayout& L, const CodecCfg& /*c*/, long elem,
                                              float /*mul*/, const float* sm) {
    Raw r;
    r.tab = decTab(sm);
    const long off = (elem >> 5) * (4 * RATE);
    r.valid = off < L.totalBytes;
    if (!r.valid) return r;
    const uint8_t* pw = chunk + off;
    if (off + 4 * RATE <= L.totalBytes && aligned16(pw)) {
#pragma unroll
      for (int q = 0; q < RATE / 4; ++q) {
        const uint4 t = __ldcg(reinterpret_cast<const uint4*>(pw) + q);
        r.w[4 * q] = t.x; r.w[4 * q + 1] = t.y; r.w[4 * q + 2] = t.z; r.w[4 * q + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int k = 0; k < RATE; ++k)
        r.w[k] = (off + 4 * k + 4 <= L.totalBytes) ? __ldcg(reinterpret_cast<const uint32_t*>(pw) + k) : 0u;
    }
    return r;
  }

  static __device__ __forceinline__ void accumulate(const Raw& r, float (&acc)[32]) {
    if (!r.valid) return;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      uint64_t s;
      if (RATE == 4) s = (r.w[b >> 1] >> (16 * (b & 1))) & 0xffffu;
      else if (RATE == 8) s = r.w[b % RATE];
      else s = (uint64_t)r.w[(2 * b) % RATE] | ((uint64_t)r.w[(2 * b + 1) % RATE] << 32);
      float x[4];
      zfp1d::decodeBlock64T(s, kMaxBits, r.tab, x);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[4 * b + i] += x[i];
    }
  }

  static __device__ __forceinline__ float finishScale(const CodecCfg&) { return 1.f; }
  static __device__ __forceinline__ void finish(float (&)[32], const CodecCfg&) {}
};

// acc += mul * sum over n encoded copies of the run at `elem`, copy i at base + i * stride. The loads of
// Codec::kBatch copies are issued before any of them is unpacked.
// `sm`: the kernel's shared scratch (Codec::kSmemFloats floats, Codec::initShared called).
template <class Codec>
__device__ __forceinline__ void decodeSum(const uint8_t* base, long stride, int n, const ChunkLayout& L,
                                          const CodecCfg& c, long elem, float mul, float (&acc)[32], const float* sm) {
  for (int q = 0; q < n; q += Codec::kBatch) {
    typename Codec::Raw r[Codec::kBatch];
#pragma unroll
    for (int j = 0; j < Codec::kBatch; ++j) {
      if (q + j < n && COCCL_CHUNK_RANGE_OK(Codec, L, c, elem, 2)) r[j] = Codec::fetch(base + (long)(q + j) * stride, L, c, elem, mul, sm);
      else r[j].valid = false;
    }
#pragma unroll
    for (int j = 0; j < Codec::kBatch; ++j) Codec::accumulate(r[j], acc);
  }
}

// Dispatch a generic lambda on the runtime codec configuration. The functor receives a codec type tag;
// unsupported configurations return false.
template <class F>
inline bool dispatchCodec(const CodecCfg& c, F&& f) {
  if (c.kind == kCodecMxfp8) { f(MxFp8Codec{}); return true; }
  if (c.kind == kCodecTaco) { f(TacoCodec{}); return true; }
  if (c.kind == kCodecZfp) {
    if (c.bits == 4) { f(ZfpCodec<4>{}); return true; }
    if (c.bits == 8) { f(ZfpCodec<8>{}); return true; }
    if (c.bits == 16) { f(ZfpCodec<16>{}); return true; }
    return false;
  }
  if (c.kind != kCodecSdp4bit) return false;
  const bool small = c.group < 32;
#define COCCL_SDP_CASE(B, A, H, S) \
  if (c.bits == B && (c.asym != 0) == A && (c.hadamard != 0) == H && small == S) { f(SdpCodec<B, A, H, S>{}); return true; }
  COCCL_SDP_CASE(4, false, true, false)
  COCCL_SDP_CASE(4, false, false, false)
  COCCL_SDP_CASE(8, false, true, false)
  COCCL_SDP_CASE(8, false, false, false)
  COCCL_SDP_CASE(4, true, true, false)
  COCCL_SDP_CASE(4, true, false, false)
  COCCL_SDP_CASE(8, true, true, false)
  COCCL_SDP_CASE(8, true, false, false)
  COCCL_SDP_CASE(4, false, false, true)
  COCCL_SDP_CASE(8, false, false, true)
  COCCL_SDP_CASE(4, true, false, true)
  COCCL_SDP_CASE(8, true, false, true)
#undef COCCL_SDP_CASE
  return false;
}

inline bool tileCodecSupported(const CodecCfg& c) {
  if (c.kind == kCodecMxfp8) return c.group == 32;
  if (c.kind == kCodecTaco)
    return c.bits == 8 && c.paramBytes == 8 && (c.group == 32 || c.group == 64 || c.group == 128 || c.group == 256 || c.group == 512);
  if (c.kind == kCodecZfp) return c.group == 4 && c.paramBytes == 0 && (c.bits == 4 || c.bits == 8 || c.bits == 16);
  if (c.kind != kCodecSdp4bit) return false;
  if (c.group < 8 || c.group > 2048 || (c.group & (c.group - 1))) return false;
  if (c.hadamard && c.group < 32) return false;
  return c.bits == 4 || c.bits == 8;
}

}  // namespace coccl
