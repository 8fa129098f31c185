// CPU oracles exported from libcoccl.so (see oracle.cc).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// SDP4Bit encode -> decode of `chunks` chunks of `count` fp32 values, round to nearest even; writes the decoded
// values and, if asked, the maximum and RMS error against the input. Returns 0 or -1 on bad arguments.
int cocclOracleSdp4bitRoundTrip(const float* x, long count, long chunks, int bits, int group, int asym, int hadamard,
                                float* out, double* maxErr, double* rmsErr);
// ZFP fixed-rate, 1-D blocks of four fp32 values, rate in bits per value (1..32).
long cocclOracleZfpChunkBytes(long count, int rate);
int cocclOracleZfpEncode(const float* x, long count, int rate, unsigned char* out);
int cocclOracleZfpDecode(const unsigned char* in, long count, int rate, float* out);
// Byte-wise rANS frames (same frame layout and lane schedule as the ans plugin).
long cocclOracleRansFrameBound(long rawBytes);
long cocclOracleRansEncode(const unsigned char* in, long rawBytes, int probBits, unsigned char* frame);
int cocclOracleRansDecode(const unsigned char* frame, long rawBytes, unsigned char* out);
#ifdef __cplusplus
}
#endif
