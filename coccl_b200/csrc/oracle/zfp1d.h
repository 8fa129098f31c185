// ZFP fixed-rate coder for 1-D blocks of four floats, written once for host and device: the device kernels of
// the zfp plugin and the CPU oracle compile this same code, so their streams are bit-identical.
//
// Algorithm (public ZFP specification; reference files zfp/src/cuda_zfp/encode.cuh:73-231, decode.cuh,
// zfp/src/zfp.c:773-803): common exponent of the block (9 header bits: 1 "non-zero" bit + 8 exponent bits),
// block-floating-point conversion to int32 with 30 fraction bits, the reversible-up-to-rounding decorrelating
// lift, negabinary, then the bit planes from the most significant one down, each coded as "the bits of the
// values already known to be significant" + a unary run-length code of the rest, until the block's budget of
// maxbits = max(round(4 * rate), 9) bits is used up; short blocks are padded with zeros. Block i starts at
// bit i * maxbits of a stream of 32-bit little-endian words.
#pragma once
#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define COCCL_HD __host__ __device__ __forceinline__
#else
#define COCCL_HD inline
#endif

namespace coccl {
namespace zfp1d {

constexpr int kBlock = 4;
constexpr int kEbias = 127;
constexpr int kMaxWords = 6;  // rate <= 32: a block of up to 128 bits starting at any bit of a word spans 5 words; one spare

COCCL_HD int maxBits(int rate) {
  const int b = 4 * rate;
  return b < 9 ? 9 : b;
}

// Bits are appended LSB-first into a zero-initialised window of words, starting at bit `pos`.
struct BitWindow {
  uint32_t w[kMaxWords];
  int pos;
};

COCCL_HD void putBits(BitWindow& s, uint64_t v, int n) {
  for (int done = 0; done < n;) {
    const int word = s.pos >> 5, off = s.pos & 31;
    const int take = (32 - off) < (n - done) ? (32 - off) : (n - done);
    const uint32_t piece = (uint32_t)((v >> done) & ((take == 32) ? 0xffffffffull : ((1ull << take) - 1)));
    s.w[word] |= piece << off;
    s.pos += take;
    done += take;
  }
}
COCCL_HD uint64_t getBits(BitWindow& s, int n) {
  uint64_t v = 0;
  for (int done = 0; done < n;) {
    const int word = s.pos >> 5, off = s.pos & 31;
    const int take = (32 - off) < (n - done) ? (32 - off) : (n - done);
    const uint64_t piece = (s.w[word] >> off) & ((take == 32) ? 0xffffffffu : ((1u << take) - 1));
    v |= piece << done;
    s.pos += take;
    done += take;
  }
  return v;
}

COCCL_HD int blockExponent(const float* x) {
  float m = 0.f;
  for (int i = 0; i < kBlock; ++i) { const float a = fabsf(x[i]); if (a > m) m = a; }
  if (!(m > 0.f) || !(m < INFINITY)) return -kEbias;
  int e;
  frexpf(m, &e);            // m = f * 2^e, f in [0.5, 1)
  return e < 1 - kEbias ? 1 - kEbias : e;
}

COCCL_HD void forwardLift(int32_t* p) {
  int32_t x = p[0], y = p[1], z = p[2], w = p[3];
  x += w; x >>= 1; w -= x;
  z += y; z >>= 1; y -= z;
  x += z; x >>= 1; z -= x;
  w += y; w >>= 1; y -= w;
  w += y >> 1; y -= w >> 1;
  p[0] = x; p[1] = y; p[2] = z; p[3] = w;
}
COCCL_HD void inverseLift(int32_t* p) {
  int32_t x = p[0], y = p[1], z = p[2], w = p[3];
  y += w >> 1; w -= y >> 1;
  y += w; w <<= 1; w -= y;
  z += x; x <<= 1; x -= z;
  y += z; z <<= 1; z -= y;
  w += x; x <<= 1; x -= w;
  p[0] = x; p[1] = y; p[2] = z; p[3] = w;
}
COCCL_HD uint32_t toNegabinary(int32_t v) { return ((uint32_t)v + 0xaaaaaaaau) ^ 0xaaaaaaaau; }
COCCL_HD int32_t fromNegabinary(uint32_t v) { return (int32_t)((v ^ 0xaaaaaaaau) - 0xaaaaaaaau); }

// Encode one block into `s` (window zeroed by the caller, s.pos = first bit of the block).
COCCL_HD void encodeBlock(const float* x, int maxbits, BitWindow& s) {
  const int start = s.pos;
  const int emax = blockExponent(x);
  if (emax == -kEbias) {  // all zero (or not finite): a single 0 bit, the rest of the budget is padding
    s.pos = start + maxbits;
    return;
  }
  putBits(s, (uint64_t)(2 * (emax + kEbias) + 1), 9);
  int32_t q[kBlock];
  const float scale = ldexpf(1.f, 30 - emax);
  for (int i = 0; i < kBlock; ++i) q[i] = (int32_t)(x[i] * scale);
  forwardLift(q);
  uint32_t u[kBlock];
  for (int i = 0; i < kBlock; ++i) u[i] = toNegabinary(q[i]);
  int bits = maxbits - 9;
  int n = 0;
  for (int k = 32; bits && k-- > 0;) {
    uint32_t plane = 0;
    for (int i = 0; i < kBlock; ++i) plane |= ((u[i] >> k) & 1u) << i;
    const int m = n < bits ? n : bits;
    bits -= m;
    putBits(s, plane, m);
    plane >>= m;
    // unary run-length code of the values that are not yet significant
    while (n < kBlock && bits) {
      --bits;
      const uint32_t any = plane != 0;
      putBits(s, any, 1);
      if (!any) break;
      while (n < kBlock - 1 && bits) {
        --bits;
        const uint32_t bit = plane & 1u;
        putBits(s, bit, 1);
        if (bit) break;
        plane >>= 1;
        ++n;
      }
      plane >>= 1;
      ++n;
    }
  }
  s.pos = start + maxbits;
}

// Decode one block from `s` (s.pos = first bit of the block).
COCCL_HD void decodeBlock(BitWindow& s, int maxbits, float* x) {
  const int start = s.pos;
  if (getBits(s, 1) == 0) {
    for (int i = 0; i < kBlock; ++i) x[i] = 0.f;
    s.pos = start + maxbits;
    return;
  }
  const int emax = (int)getBits(s, 8) - kEbias;
  uint32_t u[kBlock] = {0, 0, 0, 0};
  int bits = maxbits - 9;
  int n = 0;
  for (int k = 32; bits && k-- > 0;) {
    const int m = n < bits ? n : bits;
    bits -= m;
    uint32_t plane = (uint32_t)getBits(s, m);
    while (n < kBlock && bits) {
      --bits;
      if (!getBits(s, 1)) break;
      while (n < kBlock - 1 && bits) {
        --bits;
        if (getBits(s, 1)) break;
        ++n;
      }
      plane |= 1u << n;
      ++n;
    }
    for (int i = 0; plane; ++i, plane >>= 1) u[i] |= (plane & 1u) << k;
  }
  int32_t q[kBlock];
  for (int i = 0; i < kBlock; ++i) q[i] = fromNegabinary(u[i]);
  inverseLift(q);
  const float scale = ldexpf(1.f, emax - 30);
  for (int i = 0; i < kBlock; ++i) x[i] = (float)q[i] * scale;
  s.pos = start + maxbits;
}


// ------------------------------------------------------------------ blocks of at most 64 bits
// The same coder with the block's bit stream held in ONE 64-bit register (maxbits <= 64, i.e. rate <= 16): no
// indexed window, so on the GPU nothing spills to local memory. Bit i of the result is bit i of the block's
// stream; the results are bit-identical to encodeBlock / decodeBlock.
COCCL_HD uint64_t encodeBlock64(const float* x, int maxbits) {
  const int emax = blockExponent(x);
  if (emax == -kEbias) return 0;
  uint64_t acc = (uint64_t)(2 * (emax + kEbias) + 1);
  int pos = 9;
  int32_t q[kBlock];
  const float scale = ldexpf(1.f, 30 - emax);
  for (int i = 0; i < kBlock; ++i) q[i] = (int32_t)(x[i] * scale);
  forwardLift(q);
  uint32_t u0 = toNegabinary(q[0]), u1 = toNegabinary(q[1]), u2 = toNegabinary(q[2]), u3 = toNegabinary(q[3]);
  int bits = maxbits - 9;
  int n = 0;
  for (int k = 32; bits && k-- > 0;) {
    uint32_t plane = ((u0 >> k) & 1u) | (((u1 >> k) & 1u) << 1) | (((u2 >> k) & 1u) << 2) | (((u3 >> k) & 1u) << 3);
    const int m = n < bits ? n : bits;
    bits -= m;
    acc |= (uint64_t)(plane & ((1u << m) - 1u)) << pos;
    pos += m;
    plane >>= m;
    while (n < kBlock && bits) {
      --bits;
      const uint32_t any = plane != 0;
      acc |= (uint64_t)any << pos;
      ++pos;
      if (!any) break;
      while (n < kBlock - 1 && bits) {
        --bits;
        const uint32_t bit = plane & 1u;
        acc |= (uint64_t)bit << pos;
        ++pos;
        if (bit) break;
        plane >>= 1;
        ++n;
      }
      plane >>= 1;
      ++n;
    }
  }
  return acc;
}

COCCL_HD void decodeBlock64(uint64_t s, int maxbits, float* x) {
  if ((s & 1u) == 0) {
    for (int i = 0; i < kBlock; ++i) x[i] = 0.f;
    return;
  }
  const int emax = (int)((s >> 1) & 0xffu) - kEbias;
  int pos = 9;
  uint32_t u0 = 0, u1 = 0, u2 = 0, u3 = 0;
  int bits = maxbits - 9;
  int n = 0;
  for (int k = 32; bits && k-- > 0;) {
    const int m = n < bits ? n : bits;
    bits -= m;
    uint32_t plane = (uint32_t)(s >> pos) & ((1u << m) - 1u);
    pos += m;
    while (n < kBlock && bits) {
      --bits;
      const uint32_t any = (uint32_t)(s >> pos) & 1u;
      ++pos;
      if (!any) break;
      while (n < kBlock - 1 && bits) {
        --bits;
        const uint32_t bit = (uint32_t)(s >> pos) & 1u;
        ++pos;
        if (bit) break;
        ++n;
      }
      plane |= 1u << n;
      ++n;
    }
    u0 |= (plane & 1u) << k;
    u1 |= ((plane >> 1) & 1u) << k;
    u2 |= ((plane >> 2) & 1u) << k;
    u3 |= ((plane >> 3) & 1u) << k;
  }
  int32_t q[kBlock] = {fromNegabinary(u0), fromNegabinary(u1), fromNegabinary(u2), fromNegabinary(u3)};
  inverseLift(q);
  const float scale = ldexpf(1.f, emax - 30);
  for (int i = 0; i < kBlock; ++i) x[i] = (float)q[i] * scale;
}

// ------------------------------------------------------------------ table-driven planes
// One bit plane of a block is the four bits x of the values at that plane plus the number n of values already
// known to be significant; what the coder emits for it (the n known bits verbatim, then the group test of the
// rest) depends on (n, x) only, is at most 7 bits long, and the codes of one n form a prefix code. The stream
// of a block is the concatenation of its plane codes cut off at the block's budget, so the encoder is one table
// look-up per plane, and the decoder one look-up on the next 7 stream bits per plane, until the budget ends; only
// a plane that the budget cuts in two is decoded bit by bit, because the serial rules give a truncated code its
// own meaning. Results are bit-identical to encodeBlock / decodeBlock.
constexpr int kPlaneEncEntries = 5 * 16;    // [n][x]
constexpr int kPlaneDecEntries = 5 * 128;   // [n][next 7 bits]

// bits 0-7: code, LSB first; bits 8-11: length; bits 12-14: n after the plane
COCCL_HD uint16_t planeCode(int n, uint32_t x) {
  uint32_t code = x & ((1u << n) - 1u);
  int len = n;
  uint32_t r = x >> n;
  while (n < kBlock) {
    const uint32_t any = r != 0;
    code |= any << len;
    ++len;
    if (!any) break;
    while (n < kBlock - 1) {
      const uint32_t bit = r & 1u;
      code |= bit << len;
      ++len;
      if (bit) break;
      r >>= 1;
      ++n;
    }
    r >>= 1;
    ++n;
  }
  return (uint16_t)(code | ((uint32_t)len << 8) | ((uint32_t)n << 12));
}
// bits 0-3: plane; bits 4-7: code length; bits 8-10: n after the plane
COCCL_HD uint16_t planeDecode(int n, uint32_t peek) {
  for (uint32_t x = 0; x < 16; ++x) {
    const uint16_t e = planeCode(n, x);
    const uint32_t len = (e >> 8) & 15u;
    if ((peek & ((1u << len) - 1u)) == (uint32_t)(e & 0xffu)) return (uint16_t)(x | (len << 4) | ((uint32_t)(e >> 12) << 8));
  }
  return (uint16_t)(1u << 4);  // not reached: the codes of one n cover every bit pattern
}

COCCL_HD uint64_t encodeBlock64T(const float* x, int maxbits, const uint16_t* encTab) {
  const int emax = blockExponent(x);
  if (emax == -kEbias) return 0;
  uint64_t acc = (uint64_t)(2 * (emax + kEbias) + 1);
  int pos = 9;
  int32_t q[kBlock];
  const float scale = ldexpf(1.f, 30 - emax);
  for (int i = 0; i < kBlock; ++i) q[i] = (int32_t)(x[i] * scale);
  forwardLift(q);
  const uint32_t u0 = toNegabinary(q[0]), u1 = toNegabinary(q[1]), u2 = toNegabinary(q[2]), u3 = toNegabinary(q[3]);
  uint32_t n = 0;
  for (int k = 31; k >= 0 && pos < maxbits; --k) {
    const uint32_t plane = ((u0 >> k) & 1u) | (((u1 >> k) & 1u) << 1) | (((u2 >> k) & 1u) << 2) | (((u3 >> k) & 1u) << 3);
    const uint32_t e = encTab[n * 16u + plane];
    acc |= (uint64_t)(e & 0xffu) << pos;
    pos += (int)((e >> 8) & 15u);
    n = e >> 12;
  }
  return maxbits >= 64 ? acc : (acc & ((1ull << maxbits) - 1ull));
}

// `s` must be zero above bit maxbits - 1.
COCCL_HD void decodeBlock64T(uint64_t s, int maxbits, const uint16_t* decTab, float* x) {
  if ((s & 1u) == 0) {
    for (int i = 0; i < kBlock; ++i) x[i] = 0.f;
    return;
  }
  const int emax = (int)((s >> 1) & 0xffu) - kEbias;
  int pos = 9;
  uint32_t u0 = 0, u1 = 0, u2 = 0, u3 = 0;
  uint32_t n = 0;
  for (int k = 31; k >= 0 && pos < maxbits; --k) {
    const uint32_t e = decTab[n * 128u + ((uint32_t)(s >> pos) & 0x7fu)];
    const int len = (int)((e >> 4) & 15u);
    uint32_t plane;
    if (pos + len <= maxbits) {
      plane = e & 15u;
      n = (e >> 8) & 7u;
      pos += len;
    } else {
      int bits = maxbits - pos;
      const int m = (int)n < bits ? (int)n : bits;
      bits -= m;
      plane = (uint32_t)(s >> pos) & ((1u << m) - 1u);
      pos += m;
      while (n < (uint32_t)kBlock && bits) {
        --bits;
        const uint32_t any = (uint32_t)(s >> pos) & 1u;
        ++pos;
        if (!any) break;
        while (n < (uint32_t)kBlock - 1 && bits) {
          --bits;
          const uint32_t bit = (uint32_t)(s >> pos) & 1u;
          ++pos;
          if (bit) break;
          ++n;
        }
        plane |= 1u << n;
        ++n;
      }
      pos = maxbits;
    }
    u0 |= (plane & 1u) << k;
    u1 |= ((plane >> 1) & 1u) << k;
    u2 |= ((plane >> 2) & 1u) << k;
    u3 |= ((plane >> 3) & 1u) << k;
  }
  int32_t q[kBlock] = {fromNegabinary(u0), fromNegabinary(u1), fromNegabinary(u2), fromNegabinary(u3)};
  inverseLift(q);
  const float scale = ldexpf(1.f, emax - 30);
  for (int i = 0; i < kBlock; ++i) x[i] = (float)q[i] * scale;
}

}  // namespace zfp1d
}  // namespace coccl
