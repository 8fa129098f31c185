// Shared device-side helpers for every sm_100a kernel in this library:
// vector loads/stores, a counter-based RNG for stochastic rounding, the
// bounded-wait signal primitives (release/acquire flags in peer memory with a
// globaltimer deadline) and the per-communicator error word.
//
// Reference behaviour covered here: NCCL's device spin loops poll an abort
// flag (src/device/prims_simple.h:97-132); this library instead gives every
// wait a deadline and reports {phase, peer} through a status word.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace coccl {

constexpr int kMaxRanks = 8;          // one NVSwitch domain
constexpr int kTileThreads = 256;     // threads per CTA in codec / collective kernels
constexpr int kElemsPerThread = 32;    // one aligned run of 32 elements (one Hadamard block) per thread
constexpr int kTileElems = kTileThreads * kElemsPerThread;  // 8192

enum DType : int { kF32 = 0, kF16 = 1, kBF16 = 2 };

__host__ __device__ inline int dtypeSize(int dt) { return dt == kF32 ? 4 : 2; }

// ---------------------------------------------------------------------------
// Error/status word: one per communicator, in device memory mapped to the host.
// bit 31 set = a bounded wait ran out; low bits = phase (8) | peer (8) | slice (15).
// ---------------------------------------------------------------------------
struct StatusWord {
  unsigned int code;      // 0 = ok
  unsigned int detail;
  unsigned long long when;
};

__device__ __forceinline__ unsigned long long globalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void reportTimeout(StatusWord* st, int phase, int peer, int slice) {
  if (st == nullptr) return;
  unsigned int code = 0x80000000u | ((phase & 0xff) << 23) | ((peer & 0xff) << 15) | (slice & 0x7fff);
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->detail = (unsigned)phase;
    st->when = globalTimerNs();
  }
}

// Release store / acquire load at system scope: flags live in (peer) global memory.
__device__ __forceinline__ void stReleaseSys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ldAcquireSys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ldRelaxedSys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Wait until *flag has reached `epoch` (wrap-safe), or until `deadlineNs`
// nanoseconds have passed. Returns false on timeout; never traps, never spins
// without a limit.
__device__ __forceinline__ bool waitFlag(const unsigned int* flag, unsigned int epoch,
                                         unsigned long long deadlineNs) {
  unsigned int v = ldAcquireSys(flag);
  if ((int)(v - epoch) >= 0) return true;
  unsigned long long start = globalTimerNs();
  unsigned int spins = 0;
  while (true) {
    v = ldAcquireSys(flag);
    if ((int)(v - epoch) >= 0) return true;
    if ((++spins & 63u) == 0u) {
      if (globalTimerNs() - start > deadlineNs) return false;
      __nanosleep(64);
    }
  }
}

// ---------------------------------------------------------------------------
// Counter-based RNG: one 32-bit hash per 4 elements, 8 random bits each.
// Keyed by (seed, element index) so results do not depend on the launch shape.
// ---------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint32_t hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du;
  x ^= x >> 15; x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
__host__ __device__ __forceinline__ uint32_t rngWord(uint32_t seed, uint64_t quadIndex) {
  uint32_t lo = (uint32_t)quadIndex, hi = (uint32_t)(quadIndex >> 32);
  return hash32(lo ^ hash32(seed + 0x9e3779b9u * (hi + 1u)));
}
// uniform in (0,1) with 8-bit resolution, centred so that E[floor(y+u)] = y up to 2^-9.
__host__ __device__ __forceinline__ float rngUnit(uint32_t word, int k) {
  return ((float)((word >> (8 * k)) & 0xffu) + 0.5f) * (1.0f / 256.0f);
}

// ---------------------------------------------------------------------------
// 8-element loads/stores with tail guards. `n` = elements still valid from p.
// Vector path needs 16-byte alignment of p (checked by the caller once per chunk).
// ---------------------------------------------------------------------------
template <typename T> struct Vec8;

template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, long n, bool vec, float (&v)[8]) {
    if (vec && n >= 8) {
      float4 a = __ldg(reinterpret_cast<const float4*>(p));
      float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (i < n) ? p[i] : 0.f;
    }
  }
  static __device__ __forceinline__ void store(float* p, long n, bool vec, const float (&v)[8]) {
    if (vec && n >= 8) {
      reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
      reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) if (i < n) p[i] = v[i];
    }
  }
};

template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, long n, bool vec, float (&v)[8]) {
    if (vec && n >= 8) {
      uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (i < n) ? __bfloat162float(p[i]) : 0.f;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, long n, bool vec, const float (&v)[8]) {
    if (vec && n >= 8) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) if (i < n) p[i] = __float2bfloat16_rn(v[i]);
    }
  }
};

template <> struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, long n, bool vec, float (&v)[8]) {
    if (vec && n >= 8) {
      uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        float2 f = __half22float2(h);
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (i < n) ? __half2float(p[i]) : 0.f;
    }
  }
  static __device__ __forceinline__ void store(__half* p, long n, bool vec, const float (&v)[8]) {
    if (vec && n >= 8) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) if (i < n) p[i] = __float2half_rn(v[i]);
    }
  }
};

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace coccl
