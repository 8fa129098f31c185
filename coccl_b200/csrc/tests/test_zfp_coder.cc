// The two forms of the ZFP block coder (oracle/zfp1d.h): the windowed one used by the CPU oracle and the plugin,
// and the one that keeps a block of up to 64 bits in a register for the fused tile codec. They must agree bit
// for bit, and decode to the same values, for every rate the tile codec offers.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "host_test.h"
#include "oracle/zfp1d.h"

using namespace coccl::zfp1d;

namespace {
float sample(unsigned& st, int kind) {
  st = st * 1664525u + 1013904223u;
  const float u = (float)((st >> 8) & 0xffff) / 65536.f - 0.5f;
  switch (kind) {
    case 0: return u;
    case 1: return u * 1e-2f;
    case 2: return u * 3e4f;
    case 3: return ((st >> 3) & 7) == 0 ? 0.f : u * 1e-6f;
    default: return ldexpf(u, (int)((st >> 20) & 63) - 40);
  }
}
}  // namespace

TEST(zfp_register_coder_matches_window_coder) {
  unsigned st = 12345u;
  static uint16_t encTab[kPlaneEncEntries], decTab[kPlaneDecEntries];
  for (int n = 0; n < 5; ++n) {
    for (uint32_t x = 0; x < 16; ++x) {
      encTab[n * 16 + x] = planeCode(n, x);
      EXPECT(((encTab[n * 16 + x] >> 8) & 15) <= 7);   // a plane code fits the decoder's 7-bit look-ahead
    }
    for (uint32_t pk = 0; pk < 128; ++pk) decTab[n * 128 + pk] = planeDecode(n, pk);
  }
  const int rates[] = {4, 8, 16};
  long checked = 0;
  for (int rate : rates) {
    const int mb = maxBits(rate);
    for (int kind = 0; kind < 5; ++kind) {
      for (int rep = 0; rep < 4000; ++rep) {
        float x[4];
        for (int i = 0; i < 4; ++i) x[i] = sample(st, kind);
        if (rep % 97 == 0) x[0] = x[1] = x[2] = x[3] = 0.f;
        BitWindow w;
        memset(&w, 0, sizeof(w));
        w.pos = 0;
        encodeBlock(x, mb, w);
        const uint64_t ref = (uint64_t)w.w[0] | ((uint64_t)w.w[1] << 32);
        const uint64_t got = encodeBlock64(x, mb);
        const uint64_t mask = mb == 64 ? ~0ull : ((1ull << mb) - 1ull);
        EXPECT((ref & mask) == (got & mask));
        EXPECT((got & ~mask) == 0);
        EXPECT(encodeBlock64T(x, mb, encTab) == got);   // table-driven planes: the same stream
        float a[4], b[4];
        BitWindow r;
        memset(&r, 0, sizeof(r));
        r.w[0] = (uint32_t)got;
        r.w[1] = (uint32_t)(got >> 32);
        r.pos = 0;
        decodeBlock(r, mb, a);
        decodeBlock64(got, mb, b);
        for (int i = 0; i < 4; ++i) EXPECT(a[i] == b[i]);
        float c[4];
        decodeBlock64T(got, mb, decTab, c);
        for (int i = 0; i < 4; ++i) EXPECT(a[i] == c[i]);
        ++checked;
      }
    }
  }
  EXPECT(checked == 3 * 5 * 4000);
}
