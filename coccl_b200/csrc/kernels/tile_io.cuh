// Raw-value tile I/O for the codec and collective kernels.
//
// A CTA of 256 threads owns a tile of 8192 consecutive elements; thread t owns the aligned run of 32
// elements [32 t, 32 t + 32) and keeps it in registers as fp32. A run is one Hadamard block and a whole
// number of quantisation groups (or a fraction 1/lpg of one), so the transform and most of the group
// statistics need no cross-lane traffic.
//
// Global memory is still accessed with fully coalesced 16-byte vectors: a warp reads its 1024 elements as
// consecutive uint4, parks them in a per-warp shared-memory window with the 16-byte chunks XOR-swizzled by
// the run index, and every thread then picks up its own run with conflict-free 16-byte shared loads (and the
// reverse for stores). Tiles that are ragged (the tail of a chunk) or not 16-byte aligned take a plain
// guarded path.
#pragma once
#include "common.cuh"

namespace coccl {

// Shared staging of one CTA: 8192 elements of T.
template <typename T>
struct TileStage {
  uint4 buf[kTileElems * sizeof(T) / 16];
};

template <typename T> struct Scalar;
template <> struct Scalar<float> {
  static __device__ __forceinline__ float toF(float x) { return x; }
  static __device__ __forceinline__ float fromF(float x) { return x; }
};
template <> struct Scalar<__nv_bfloat16> {
  static __device__ __forceinline__ float toF(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 fromF(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Scalar<__half> {
  static __device__ __forceinline__ float toF(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half fromF(float x) { return __float2half_rn(x); }
};

// 8 packed 16-bit values <-> 8 floats
template <typename T> struct Pack16;
template <> struct Pack16<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack(const uint4& a, float* v) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Pack16<__half> {
  static __device__ __forceinline__ void unpack(const uint4& a, float* v) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <typename T>
struct TileIO {
  static constexpr bool k32 = sizeof(T) == 4;
  static constexpr int kChunksPerRun = 32 * sizeof(T) / 16;       // 16-byte chunks in one run: 8 | 4
  static constexpr int kWarpChunks = 32 * kChunksPerRun;          // chunks in a warp's window: 256 | 128
  static constexpr int kRunsPerInstr = 32 / kChunksPerRun;        // runs covered by one warp-wide vector: 4 | 8

  // swizzled position of chunk c of run r inside the warp window
  static __device__ __forceinline__ int slot(int r, int c) {
    return k32 ? r * 8 + (c ^ (r & 7)) : r * 4 + (c ^ ((r >> 1) & 3));
  }

  // v <- elements [e0 + 32 t, +32) of `chunk` (zero beyond `count`). `fast` must be uniform over the CTA.
  static __device__ __forceinline__ void load(const T* chunk, long count, long e0, bool fast, TileStage<T>& st,
                                              float (&v)[32]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (fast) {
      const uint4* g = reinterpret_cast<const uint4*>(chunk + e0) + warp * kWarpChunks;
      uint4* w = st.buf + warp * kWarpChunks;
      uint4 x[kChunksPerRun];
#pragma unroll
      for (int j = 0; j < kChunksPerRun; ++j) x[j] = __ldg(g + j * 32 + lane);
      __syncwarp();  // the previous user of the window is done
#pragma unroll
      for (int j = 0; j < kChunksPerRun; ++j)
        w[slot(j * kRunsPerInstr + lane / kChunksPerRun, lane % kChunksPerRun)] = x[j];
      __syncwarp();
#pragma unroll
      for (int c = 0; c < kChunksPerRun; ++c) {
        const uint4 y = w[slot(lane, c)];
        if constexpr (k32) {
          v[4 * c] = __uint_as_float(y.x); v[4 * c + 1] = __uint_as_float(y.y);
          v[4 * c + 2] = __uint_as_float(y.z); v[4 * c + 3] = __uint_as_float(y.w);
        } else {
          Pack16<T>::unpack(y, &v[8 * c]);
        }
      }
    } else {
      const long e = e0 + (long)threadIdx.x * 32;
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = (e + i < count) ? Scalar<T>::toF(chunk[e + i]) : 0.f;
    }
  }

  // elements [e0 + 32 t, +32) of `chunk` <- v (nothing beyond `count`).
  static __device__ __forceinline__ void store(T* chunk, long count, long e0, bool fast, TileStage<T>& st,
                                               const float (&v)[32]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (fast) {
      uint4* w = st.buf + warp * kWarpChunks;
      __syncwarp();
#pragma unroll
      for (int c = 0; c < kChunksPerRun; ++c) {
        uint4 y;
        if constexpr (k32) {
          y = make_uint4(__float_as_uint(v[4 * c]), __float_as_uint(v[4 * c + 1]), __float_as_uint(v[4 * c + 2]),
                         __float_as_uint(v[4 * c + 3]));
        } else {
          y = Pack16<T>::pack(&v[8 * c]);
        }
        w[slot(lane, c)] = y;
      }
      __syncwarp();
      uint4* g = reinterpret_cast<uint4*>(chunk + e0) + warp * kWarpChunks;
#pragma unroll
      for (int j = 0; j < kChunksPerRun; ++j)
        g[j * 32 + lane] = w[slot(j * kRunsPerInstr + lane / kChunksPerRun, lane % kChunksPerRun)];
    } else {
      const long e = e0 + (long)threadIdx.x * 32;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (e + i < count) chunk[e + i] = Scalar<T>::fromF(v[i]);
    }
  }

  // whether the tile starting at element e0 can take the vector path
  static __device__ __forceinline__ bool fastTile(const T* chunk, long count, long e0) {
    return aligned16(chunk) && e0 + kTileElems <= count;
  }
};

}  // namespace coccl
