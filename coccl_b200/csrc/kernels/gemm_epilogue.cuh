// Epilogue of one 128-row x 256-column fp32 accumulator held in TMEM: each of the four epilogue
// warps drains its 32 lanes (rows), 32 columns at a time, applies the fused epilogue and stores.
#pragma once
#include "gemm_tcgen05.cuh"
#include "gemm_api.h"

namespace coccl {

struct GemmArgs {
  void* C;
  void* Z;
  const void* bias;
  int M, N, K;
  long ldc;
  int epi;
  int aMN, bMN;
  unsigned int* err;
  int stages;  // pair kernel: ring depth of this launch (fp32 epilogues give one stage to the TMA boxes)
};

// tbase: TMEM address of (lane quadrant of this warp, first accumulator column); row: the global row
// this thread owns; colBase: global column of accumulator column 0.
__device__ __forceinline__ void epilogueStoreTile(const GemmArgs& g, uint32_t tbase, int row, int colBase) {
  using namespace sm100;
#pragma unroll 1
  for (int c = 0; c < 256 / 32; ++c) {
    uint32_t r[32];
    tmemLd32x32(tbase + c * 32, r);
    tmemLdWait();
    const int col0 = colBase + c * 32;
    if (row < g.M && col0 < g.N) {
      const int ncols = min(32, g.N - col0);
      if (g.epi == GEMM_EPI_F32 || g.epi == GEMM_EPI_F32_ACC) {
        float* cp = reinterpret_cast<float*>(g.C) + (long)row * g.ldc + col0;
        for (int j = 0; j < ncols; j += 4) {
          float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                 __uint_as_float(r[j + 3]));
          if (g.epi == GEMM_EPI_F32_ACC) {
            float4 o = *reinterpret_cast<float4*>(cp + j);
            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
          }
          *reinterpret_cast<float4*>(cp + j) = v;
        }
      } else {
        __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(g.C) + (long)row * g.ldc + col0;
        __nv_bfloat16* zp = g.Z ? reinterpret_cast<__nv_bfloat16*>(g.Z) + (long)row * g.ldc + col0 : nullptr;
        const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(g.bias) + col0;
        for (int j = 0; j < ncols; j += 8) {
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[j + i]);
          if (g.epi == GEMM_EPI_BIAS || g.epi == GEMM_EPI_BIAS_GELU) {
            uint4 bw = __ldg(reinterpret_cast<const uint4*>(bp + j));
            const uint32_t w[4] = {bw.x, bw.y, bw.z, bw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              v[2 * i] += __uint_as_float(w[i] << 16);
              v[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
            }
          }
          uint32_t o[4];
          if (g.epi == GEMM_EPI_BIAS_GELU) {
            if (zp) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                o[i] = *reinterpret_cast<uint32_t*>(&h);
              }
              *reinterpret_cast<uint4*>(zp + j) = make_uint4(o[0], o[1], o[2], o[3]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = geluTanh(v[i]);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            o[i] = *reinterpret_cast<uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(cp + j) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }
}

// fp32 outputs (weight gradients, fp32 products): each epilogue warp drains its 32 rows, 32 columns at a time, into a
// 4 KiB shared-memory box laid out for SWIZZLE_128B (16-byte chunk j of row i sits at chunk j ^ (i & 7): the 32 lanes,
// one row each, write without bank conflicts) and one lane hands the box to the TMA unit: a plain store, or with
// `accumulate` a reduce-add that the L2 performs, so the previous gradient never travels to the SM. Two boxes per warp
// alternate; the TMA unit clips rows and columns past the matrix.
constexpr int kEpiBoxBytes = 32 * 128;
constexpr int kEpiStageBytesPerWarp = 2 * kEpiBoxBytes;
constexpr int kEpiStageBytes = 4 * kEpiStageBytesPerWarp;

// stage: this warp's two boxes (1024-byte aligned); boxCounter: running count of boxes this warp has issued.
__device__ __forceinline__ void epilogueTmaTileF32(const CUtensorMap* tmC, bool accumulate, uint32_t tbase, int row0,
                                                  int colBase, int nCols, uint8_t* stage, uint32_t& boxCounter) {
  using namespace sm100;
  const int lane = threadIdx.x & 31;
#pragma unroll 1
  for (int c = 0; c < 256 / 32; ++c) {
    uint32_t r[32];
    tmemLd32x32(tbase + c * 32, r);
    tmemLdWait();
    const int col0 = colBase + c * 32;
    if (col0 >= nCols) continue;  // uniform over the warp
    uint8_t* box = stage + (boxCounter & 1u) * kEpiBoxBytes;
    // the box was handed to the TMA unit two boxes ago: wait until that transfer has read it
    if (lane == 0) bulkWaitGroupRead<1>();
    __syncwarp();
    uint4* rowp = reinterpret_cast<uint4*>(box + lane * 128);
#pragma unroll
    for (int j = 0; j < 8; ++j) rowp[j ^ (lane & 7)] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    fenceProxyAsyncShared();
    __syncwarp();
    if (lane == 0) {
      if (accumulate) tmaReduceAdd2d(tmC, box, col0, row0);
      else tmaStore2d(tmC, box, col0, row0);
      bulkCommitGroup();
    }
    ++boxCounter;
  }
}

// bf16 outputs through the TMA unit: the same 32-row x 128-byte swizzled boxes, here 64 columns wide (two accumulator
// chunks per box). Bias and GELU are applied in registers; the optional pre-activation Z keeps its direct stores.
__device__ __forceinline__ void epilogueTmaTileBf16(const GemmArgs& g, const CUtensorMap* tmC, uint32_t tbase, int row0,
                                                   int colBase, uint8_t* stage, uint32_t& boxCounter) {
  using namespace sm100;
  const int lane = threadIdx.x & 31;
  const int row = row0 + lane;
  const bool hasBias = g.epi == GEMM_EPI_BIAS || g.epi == GEMM_EPI_BIAS_GELU;
#pragma unroll 1
  for (int cp = 0; cp < 256 / 64; ++cp) {
    const int col0 = colBase + cp * 64;
    if (col0 >= g.N) continue;  // uniform over the warp
    uint8_t* box = stage + (boxCounter & 1u) * kEpiBoxBytes;
    if (lane == 0) bulkWaitGroupRead<1>();
    __syncwarp();
    uint4* rowp = reinterpret_cast<uint4*>(box + lane * 128);
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      uint32_t r[32];
      tmemLd32x32(tbase + (cp * 2 + half) * 32, r);
      tmemLdWait();
      const int colh = col0 + half * 32;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = colh + 8 * j;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[8 * j + i]);
        uint32_t o[4] = {0, 0, 0, 0};
        if (col < g.N) {  // N is a multiple of 8: a group of 8 columns is inside or outside as a whole
          if (hasBias) {
            const uint4 bw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g.bias) + col));
            const uint32_t w[4] = {bw.x, bw.y, bw.z, bw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              v[2 * i] += __uint_as_float(w[i] << 16);
              v[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
            }
          }
          if (g.epi == GEMM_EPI_BIAS_GELU) {
            if (g.Z != nullptr && row < g.M) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                o[i] = *reinterpret_cast<uint32_t*>(&h);
              }
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(g.Z) + (long)row * g.ldc + col) = make_uint4(o[0], o[1], o[2], o[3]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = geluTanh(v[i]);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            o[i] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        rowp[(half * 4 + j) ^ (lane & 7)] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    fenceProxyAsyncShared();
    __syncwarp();
    if (lane == 0) {
      tmaStore2d(tmC, box, col0, row0);
      bulkCommitGroup();
    }
    ++boxCounter;
  }
}

}  // namespace coccl
