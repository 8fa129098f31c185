// CPU oracles of the codecs (plain C++, no CUDA): the reference's own CPU code is the oracle where it has some
// (zfp/src/template/{encode,decode}.c run with the serial policy, zfp/src/zfp.c:1116-1135); for SDP4Bit the
// reference has GPU kernels only, so the oracle restates their arithmetic
// (sdp4bit/includes/quantization_utils.h:126-272, fast_hadamard_transform_common.h:248-264).
// Exported from libcoccl.so for the tests and for `coccl-config-check --oracle`.
#include "oracle/oracle.h"
#include "oracle/zfp1d.h"
#include "oracle/rans.h"

#include <math.h>
#include <string.h>
#include <algorithm>
#include <vector>

namespace {
void hadamard32(float* v) {
  for (int s = 1; s < 32; s <<= 1)
    for (int i = 0; i < 32; ++i)
      if ((i & s) == 0) { const float a = v[i], b = v[i | s]; v[i] = a + b; v[i | s] = a - b; }
}
}  // namespace

extern "C" int cocclOracleSdp4bitRoundTrip(const float* x, long count, long chunks, int bits, int group, int asym,
                                           int hadamard, float* out, double* maxErr, double* rmsErr) {
  if (!x || !out || count <= 0 || chunks <= 0 || (bits != 4 && bits != 8) || group < 8 || (group & (group - 1)) ||
      (hadamard && group < 32))
    return -1;
  const float qlo = -(float)(1 << (bits - 1)), qhi = (float)((1 << (bits - 1)) - 1);
  double worst = 0, sq = 0;
  std::vector<float> v;
  for (long ch = 0; ch < chunks; ++ch) {
    const float* src = x + ch * count;
    float* dst = out + ch * count;
    const long padded = (count + group - 1) / group * group;
    v.assign((size_t)padded, 0.f);
    memcpy(v.data(), src, sizeof(float) * (size_t)count);
    if (hadamard) for (long r = 0; r < padded; r += 32) hadamard32(&v[(size_t)r]);
    for (long g = 0; g < padded; g += group) {
      float scale, offset = 0.f;
      if (!asym) {
        float m = 0.f;
        for (int i = 0; i < group; ++i) m = fmaxf(m, fabsf(v[(size_t)(g + i)]));
        scale = m == 0.f ? 1.f : qhi / m;
      } else {
        float mx = v[(size_t)g], mn = v[(size_t)g];
        for (int i = 1; i < group; ++i) { mx = fmaxf(mx, v[(size_t)(g + i)]); mn = fminf(mn, v[(size_t)(g + i)]); }
        const float range = mx - mn;
        scale = range == 0.f ? 1.f : (float)(1 << bits) / range;
        offset = 0.5f * (mx + mn);
      }
      const float inv = 1.f / scale;
      for (int i = 0; i < group; ++i) {
        volatile float y = (v[(size_t)(g + i)] - offset) * scale;  // rounded to fp32 before the integer rounding
        float q = nearbyintf(y);                                   // round half to even (default rounding mode)
        q = fminf(fmaxf(q, qlo), qhi);
        v[(size_t)(g + i)] = q * inv + offset;
      }
    }
    if (hadamard)
      for (long r = 0; r < padded; r += 32) {
        hadamard32(&v[(size_t)r]);
        for (int i = 0; i < 32; ++i) v[(size_t)(r + i)] *= 1.f / 32.f;
      }
    for (long i = 0; i < count; ++i) {
      dst[i] = v[(size_t)i];
      const double e = fabs((double)dst[i] - (double)src[i]);
      if (e > worst) worst = e;
      sq += e * e;
    }
  }
  if (maxErr) *maxErr = worst;
  if (rmsErr) *rmsErr = sqrt(sq / (double)(count * chunks));
  return 0;
}

extern "C" long cocclOracleZfpChunkBytes(long count, int rate) {
  const long blocks = (count + 3) / 4;
  return (blocks * coccl::zfp1d::maxBits(rate) + 63) / 64 * 8;
}

extern "C" int cocclOracleZfpEncode(const float* x, long count, int rate, unsigned char* out) {
  using namespace coccl::zfp1d;
  if (!x || !out || count <= 0 || rate < 1 || rate > 32) return -1;
  const int mb = maxBits(rate);
  const long bytes = cocclOracleZfpChunkBytes(count, rate);
  memset(out, 0, (size_t)bytes);
  uint32_t* words = reinterpret_cast<uint32_t*>(out);
  const long blocks = (count + 3) / 4;
  for (long b = 0; b < blocks; ++b) {
    float v[4];
    for (int i = 0; i < 4; ++i) v[i] = 4 * b + i < count ? x[4 * b + i] : 0.f;
    BitWindow s;
    memset(&s, 0, sizeof(s));
    const long bit0 = b * mb;
    s.pos = (int)(bit0 & 31);
    const int p0 = s.pos;
    encodeBlock(v, mb, s);
    const int n = (p0 + mb + 31) >> 5;
    for (int i = 0; i < n; ++i) words[(bit0 >> 5) + i] |= s.w[i];
  }
  return 0;
}

extern "C" int cocclOracleZfpDecode(const unsigned char* in, long count, int rate, float* out) {
  using namespace coccl::zfp1d;
  if (!in || !out || count <= 0 || rate < 1 || rate > 32) return -1;
  const int mb = maxBits(rate);
  const long totalWords = cocclOracleZfpChunkBytes(count, rate) / 4;
  const uint32_t* words = reinterpret_cast<const uint32_t*>(in);
  const long blocks = (count + 3) / 4;
  for (long b = 0; b < blocks; ++b) {
    BitWindow s;
    memset(&s, 0, sizeof(s));
    const long bit0 = b * mb;
    s.pos = (int)(bit0 & 31);
    const int n = (s.pos + mb + 31) >> 5;
    for (int i = 0; i < n; ++i) s.w[i] = (bit0 >> 5) + i < totalWords ? words[(bit0 >> 5) + i] : 0u;
    float v[4];
    decodeBlock(s, mb, v);
    for (int i = 0; i < 4; ++i)
      if (4 * b + i < count) out[4 * b + i] = v[i];
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// rANS frame coder, sequential restatement of the 32-lane schedule of the ans plugin (oracle/rans.h).
// ---------------------------------------------------------------------------------------------
extern "C" long cocclOracleRansFrameBound(long rawBytes) { return (long)coccl::rans::frameBound((uint64_t)rawBytes); }

// Returns the coded frame size in bytes, or 0 when the frame would not be smaller than the input (the plugin
// then stores the bytes raw), or -1 on bad arguments.
extern "C" long cocclOracleRansEncode(const unsigned char* in, long rawBytes, int probBits, unsigned char* frame) {
  using namespace coccl::rans;
  if (!in || !frame || rawBytes <= 0 || rawBytes > (1l << 30) || probBits < 9 || probBits > 11) return -1;
  const uint32_t nb = numBlocks((uint32_t)rawBytes);
  uint32_t hist[256] = {0};
  for (long i = 0; i < rawBytes; ++i) ++hist[in[i]];
  uint16_t* pdf = reinterpret_cast<uint16_t*>(frame + 32);
  normalise(hist, (uint32_t)rawBytes, probBits, pdf);
  uint32_t cdf[256], run = 0;
  for (int i = 0; i < 256; ++i) { cdf[i] = run; run += pdf[i]; }
  uint32_t* states = reinterpret_cast<uint32_t*>(frame + 32 + 512);
  uint32_t* words = states + (size_t)nb * kLanes;
  uint32_t* starts = words + nb;
  const uint32_t hdr = headerBytes(nb);
  uint16_t* streams = reinterpret_cast<uint16_t*>(frame + hdr);
  uint32_t total = 0;
  std::vector<uint16_t> tmp((size_t)kMaxBlockWords);
  for (uint32_t b = 0; b < nb; ++b) {
    const long off = (long)b * kBlockBytes;
    const int n = (int)std::min<long>(kBlockBytes, rawBytes - off);
    uint32_t st[kLanes];
    for (int l = 0; l < kLanes; ++l) st[l] = kLower;
    uint32_t written = 0;
    for (int j = 0; j * kLanes < n; ++j)
      for (int l = 0; l < kLanes && j * kLanes + l < n; ++l) {
        const uint32_t s = in[off + j * kLanes + l];
        uint16_t w;
        if (encodeStep(st[l], pdf[s], cdf[s], probBits, w)) tmp[written++] = w;
      }
    for (int l = 0; l < kLanes; ++l) states[(size_t)b * kLanes + l] = st[l];
    words[b] = written;
    starts[b] = total;
    if ((uint64_t)hdr + ((uint64_t)total + written) * 2 <= frameBound((uint64_t)rawBytes))
      memcpy(streams + total, tmp.data(), (size_t)written * 2);
    total += (written + 7) & ~7u;
  }
  const uint64_t coded = (uint64_t)hdr + (uint64_t)total * 2;
  FrameHeader h{kMagic, nb, (uint32_t)rawBytes, total, (uint32_t)probBits, {0, 0, 0}};
  memcpy(frame, &h, sizeof(h));
  return coded < (uint64_t)rawBytes ? (long)coded : 0;
}

extern "C" int cocclOracleRansDecode(const unsigned char* frame, long rawBytes, unsigned char* out) {
  using namespace coccl::rans;
  if (!frame || !out || rawBytes <= 0) return -1;
  FrameHeader h;
  memcpy(&h, frame, sizeof(h));
  if (h.magic != kMagic || h.rawBytes != (uint32_t)rawBytes || h.probBits < 9 || h.probBits > 11) return -1;
  const int pb = (int)h.probBits;
  const uint32_t nb = h.numBlocks, mask = (1u << pb) - 1;
  const uint16_t* pdf = reinterpret_cast<const uint16_t*>(frame + 32);
  uint32_t cdf[256], run = 0;
  std::vector<uint8_t> lookup((size_t)1 << pb);
  for (int i = 0; i < 256; ++i) {
    cdf[i] = run;
    for (uint32_t s = run; s < run + pdf[i] && s <= mask; ++s) lookup[s] = (uint8_t)i;
    run += pdf[i];
  }
  const uint32_t* states = reinterpret_cast<const uint32_t*>(frame + 32 + 512);
  const uint32_t* words = states + (size_t)nb * kLanes;
  const uint32_t* starts = words + nb;
  const uint16_t* streams = reinterpret_cast<const uint16_t*>(frame + headerBytes(nb));
  for (uint32_t b = 0; b < nb; ++b) {
    const long off = (long)b * kBlockBytes;
    const int n = (int)std::min<long>(kBlockBytes, rawBytes - off);
    uint32_t st[kLanes];
    for (int l = 0; l < kLanes; ++l) st[l] = states[(size_t)b * kLanes + l];
    const uint16_t* in = streams + starts[b];
    uint32_t avail = words[b];
    for (int j = (n + kLanes - 1) / kLanes - 1; j >= 0; --j) {
      // the lanes of a step pushed their words in lane order: pop them in reverse
      for (int l = kLanes - 1; l >= 0; --l) {
        if (j * kLanes + l >= n) continue;
        const uint32_t s = lookup[st[l] & mask];
        out[off + j * kLanes + l] = (uint8_t)s;
        if (decodeStep(st[l], pdf[s], cdf[s], pb)) {
          if (avail == 0) return -2;
          st[l] = (st[l] << 16) | in[--avail];
        }
      }
    }
  }
  return 0;
}
