// Memory-bound training kernels of the GPT trainer (bf16 activations, fp32
// statistics): residual-add + LayerNorm forward/backward, GELU backward,
// column sums (bias gradients), fused cross-entropy forward+backward, fused
// Adam with fp32 master weights, squared-norm reduction and clip coefficient.
//
// The reference ships no trainer (its training layer is an empty submodule,
// .gitmodules:1-3); these kernels belong to the framework layer that drives the
// compressed collectives. Each kernel touches every byte once.
#include "launch_count.h"
#include "common.cuh"
#include "train_api.h"
#include "no_alloc_api.h"
#include <mutex>
#include <stdio.h>
#include <math.h>

namespace coccl {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float warpSum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warpMax(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
// Block-wide sum; `sm` holds 32 floats. All threads get the result.
__device__ __forceinline__ float blockSum(float x, float* sm) {
  x = warpSum(x);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sm[w] = x;
  __syncthreads();
  float t = (threadIdx.x & 31) < nw ? sm[threadIdx.x & 31] : 0.f;
  return warpSum(t);
}
__device__ __forceinline__ float blockMax(float x, float* sm) {
  x = warpMax(x);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sm[w] = x;
  __syncthreads();
  float t = (threadIdx.x & 31) < nw ? sm[threadIdx.x & 31] : -INFINITY;
  return warpMax(t);
}

// ---------------------------------------------------------------- LayerNorm
constexpr int kLnThreads = 256;
constexpr int kLnMaxVec = 8;  // H <= 256*8*8 = 16384

// xs = x (+ res); xOut = xs (optional); y = (xs - mean) * rstd * gamma + beta
template <int NV>
__global__ void __launch_bounds__(kLnThreads) lnFwdKernel(const bf16* x, const bf16* res, const bf16* gamma,
                                                          const bf16* beta, bf16* y, bf16* xOut, float* mean,
                                                          float* rstd, int M, int H, float eps) {
  __shared__ float sm[32];
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const bf16* xr = x + (long)row * H;
    float v[NV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * kLnThreads;
      if (vi < nvec) {
        Vec8<bf16>::load(xr + vi * 8, 8, true, v[i]);
        if (res) {
          float r[8];
          Vec8<bf16>::load(res + (long)row * H + vi * 8, 8, true, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        }
        if (xOut) {
          Vec8<bf16>::store(xOut + (long)row * H + vi * 8, 8, true, v[i]);
          // keep the statistics consistent with the rounded value that is saved
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j]));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[i][j];
      }
    }
    const float mu = blockSum(s, sm) / H;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * kLnThreads;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mu; q += d * d; }
      }
    }
    const float rs = rsqrtf(blockSum(q, sm) / H + eps);
    if (threadIdx.x == 0) { mean[row] = mu; rstd[row] = rs; }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * kLnThreads;
      if (vi < nvec) {
        float g[8], b[8], o[8];
        Vec8<bf16>::load(gamma + vi * 8, 8, true, g);
        Vec8<bf16>::load(beta + vi * 8, 8, true, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mu) * rs * g[j] + b[j];
        Vec8<bf16>::store(y + (long)row * H + vi * 8, 8, true, o);
      }
    }
  }
}

// dx = rstd * (dy*gamma - mean(dy*gamma) - xhat * mean(dy*gamma*xhat)) (+ dres)
// partial[blockIdx.x][0][h] = sum_rows dy*xhat, partial[blockIdx.x][1][h] = sum_rows dy
template <int NV>
__global__ void __launch_bounds__(kLnThreads) lnBwdKernel(const bf16* dy, const bf16* x, const float* mean,
                                                          const float* rstd, const bf16* gamma, const bf16* dres,
                                                          bf16* dx, float* partial, int M, int H) {
  __shared__ float sm[32];
  const int nvec = H / 8;
  float dg[NV][8], db[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { dg[i][j] = 0.f; db[i][j] = 0.f; }

  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const float mu = mean[row], rs = rstd[row];
    float xh[NV][8], dyg[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * kLnThreads;
      if (vi < nvec) {
        float d[8], xv[8], g[8];
        Vec8<bf16>::load(dy + (long)row * H + vi * 8, 8, true, d);
        Vec8<bf16>::load(x + (long)row * H + vi * 8, 8, true, xv);
        Vec8<bf16>::load(gamma + vi * 8, 8, true, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mu) * rs;
          dyg[i][j] = d[j] * g[j];
          s1 += dyg[i][j];
          s2 += dyg[i][j] * xh[i][j];
          dg[i][j] += d[j] * xh[i][j];
          db[i][j] += d[j];
        }
      }
    }
    const float c1 = blockSum(s1, sm) / H;
    const float c2 = blockSum(s2, sm) / H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * kLnThreads;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (dyg[i][j] - c1 - xh[i][j] * c2);
        if (dres) {
          float r[8];
          Vec8<bf16>::load(dres + (long)row * H + vi * 8, 8, true, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        Vec8<bf16>::store(dx + (long)row * H + vi * 8, 8, true, o);
      }
    }
  }
  float* pg = partial + (long)blockIdx.x * 2 * H;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * kLnThreads;
    if (vi < nvec) {
      Vec8<float>::store(pg + vi * 8, 8, true, dg[i]);
      Vec8<float>::store(pg + H + vi * 8, 8, true, db[i]);
    }
  }
}

// out[c] (+)= sum_r partial[r][c]; `cols` columns, `rows` partial rows. A CTA owns 32 columns; its 8 warps take every
// 8th row (a warp reads 128 contiguous bytes of a row) and fold their sums through shared memory in a fixed order.
constexpr int kColReduceCols = 32;
__global__ void __launch_bounds__(256) colReduceKernel(const float* partial, float* out, int rows, long cols, long stride, int accumulate) {
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
  const long c = (long)blockIdx.x * kColReduceCols + lane;
  float s = 0.f;
  if (c < cols) {
    int r = wy;
    for (; r + 24 < rows; r += 32) {
      const float a0 = partial[(long)r * stride + c], a1 = partial[(long)(r + 8) * stride + c];
      const float a2 = partial[(long)(r + 16) * stride + c], a3 = partial[(long)(r + 24) * stride + c];
      s += (a0 + a1) + (a2 + a3);
    }
    for (; r < rows; r += 8) s += partial[(long)r * stride + c];
  }
  red[wy][lane] = s;
  __syncthreads();
  if (wy == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][lane];
    out[c] = accumulate ? out[c] + t : t;
  }
}

// ---------------------------------------------------------------- column sum of a bf16 matrix
// partial[blockIdx.y][n] = sum over this block's rows of x[m][n]
// A CTA owns 256 columns (32 lanes x 8) and `rowsPerBlock` rows; its 8 warps take every 8th row, four rows in
// flight per thread, and fold their sums through shared memory. A warp reads 512 contiguous bytes of one row.
__global__ void __launch_bounds__(256) colSumPartialKernel(const bf16* x, float* partial, int M, int N, int rowsPerBlock) {
  __shared__ float red[8][32][9];
  const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + lane) * 8;
  const int r0 = blockIdx.y * rowsPerBlock;
  const int r1 = min(M, r0 + rowsPerBlock);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (col < N) {
    const bf16* base = x + col;
    int r = r0 + wy;
    for (; r + 24 < r1; r += 32) {
      float v[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) Vec8<bf16>::load(base + (long)(r + 8 * u) * N, 8, true, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[u][j];
    }
    for (; r < r1; r += 8) {
      float v[8];
      Vec8<bf16>::load(base + (long)r * N, 8, true, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[wy][lane][j] = acc[j];
  __syncthreads();
  if (wy == 0 && col < N) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += red[w][lane][j];   // fixed order: the result does not depend on scheduling
      acc[j] = s;
    }
    Vec8<float>::store(partial + (long)blockIdx.y * N + col, 8, true, acc);
  }
}

// ---------------------------------------------------------------- GELU (tanh form)
__device__ __forceinline__ float geluF(float x) {
  const float u = 0.7978845608028654f * x * (1.f + 0.044715f * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float geluGrad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * x * (1.f + k1 * x * x);
  const float t = tanhf(u);
  const float du = k0 * (1.f + 3.f * k1 * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}
// y = gelu(z (+ bias)); zOut = z + bias (optional)
__global__ void __launch_bounds__(256) geluFwdKernel(const bf16* z, const bf16* bias, bf16* y, bf16* zOut, long n, int N) {
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (long)gridDim.x * blockDim.x * 8) {
    float v[8];
    Vec8<bf16>::load(z + i, 8, true, v);
    if (bias) {
      float b[8];
      Vec8<bf16>::load(bias + (i % N), 8, true, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b[j];
      if (zOut) {
        Vec8<bf16>::store(zOut + i, 8, true, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = geluF(v[j]);
    Vec8<bf16>::store(y + i, 8, true, v);
  }
}
// dz = dy * gelu'(z)
__global__ void __launch_bounds__(256) geluBwdKernel(const bf16* dy, const bf16* z, bf16* dz, long n) {
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (long)gridDim.x * blockDim.x * 8) {
    float d[8], v[8];
    Vec8<bf16>::load(dy + i, 8, true, d);
    Vec8<bf16>::load(z + i, 8, true, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) d[j] *= geluGrad(v[j]);
    Vec8<bf16>::store(dz + i, 8, true, d);
  }
}

// ---------------------------------------------------------------- cross-entropy
constexpr int kCeThreads = 1024;
constexpr int kCeMaxVec = 7;  // V <= 1024*7*8 = 57344 held in registers

// loss[row] = logsumexp(logits[row]) - logits[row][target]; logits <- (softmax - onehot) * gscale
// rows with target < 0 get loss 0 and a zero gradient.
__global__ void __launch_bounds__(kCeThreads) crossEntropyKernel(bf16* logits, const long* targets, float* loss,
                                                                 int M, int V, long ld, float gscale) {
  __shared__ float sm[32];
  const int nvec = V / 8;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    bf16* lr = logits + (long)row * ld;
    const long tgt = targets[row];
    float v[kCeMaxVec][8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kCeMaxVec; ++i) {
      const int vi = threadIdx.x + i * kCeThreads;
      if (vi < nvec) {
        Vec8<bf16>::load(lr + vi * 8, 8, true, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) mx = fmaxf(mx, v[i][j]);
      }
    }
    mx = blockMax(mx, sm);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kCeMaxVec; ++i) {
      const int vi = threadIdx.x + i * kCeThreads;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[i][j] = __expf(v[i][j] - mx); s += v[i][j]; }
      }
    }
    s = blockSum(s, sm);
    const float inv = 1.f / s;
    const bool ignore = tgt < 0;
    if (threadIdx.x == 0 && ignore) loss[row] = 0.f;
#pragma unroll
    for (int i = 0; i < kCeMaxVec; ++i) {
      const int vi = threadIdx.x + i * kCeThreads;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float p = v[i][j] * inv;
          const bool hit = (long)(vi * 8 + j) == tgt;
          if (hit) loss[row] = -__logf(fmaxf(p, 1e-37f));
          o[j] = ignore ? 0.f : (p - (hit ? 1.f : 0.f)) * gscale;
        }
        Vec8<bf16>::store(lr + vi * 8, 8, true, o);
      }
    }
  }
}

// ---------------------------------------------------------------- vocabulary-parallel cross-entropy
// The vocabulary is sharded over the tensor-parallel ranks: a rank holds columns [vocabOffset, vocabOffset + V) of
// every logit row. Pass 1 leaves per row {local max, sum of exp(logit - local max), target logit if the target lies
// in this shard, else 0}; the ranks exchange these 16 bytes per row (an all-gather of a few hundred KB, issued by the
// caller), and pass 2 combines them (global max, rescaled sums), writes the loss and overwrites the logits with
// (softmax - onehot) * gscale. Rows with target < 0 get loss 0 and a zero gradient.
__global__ void __launch_bounds__(kCeThreads) ceStatsKernel(const bf16* logits, const long* targets, float4* stats,
                                                            int M, int V, long ld, long vocabOffset) {
  __shared__ float sm[32];
  const int nvec = V / 8;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const bf16* lr = logits + (long)row * ld;
    const long tgt = targets[row] - vocabOffset;
    float v[kCeMaxVec][8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kCeMaxVec; ++i) {
      const int vi = threadIdx.x + i * kCeThreads;
      if (vi < nvec) {
        Vec8<bf16>::load(lr + vi * 8, 8, true, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) mx = fmaxf(mx, v[i][j]);
      }
    }
    mx = blockMax(mx, sm);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kCeMaxVec; ++i) {
      const int vi = threadIdx.x + i * kCeThreads;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) s += __expf(v[i][j] - mx);
      }
    }
    s = blockSum(s, sm);
    if (threadIdx.x == 0) {
      const bool inside = tgt >= 0 && tgt < V;
      stats[row] = make_float4(mx, s, inside ? __bfloat162float(lr[tgt]) : 0.f, inside ? 1.f : 0.f);
    }
  }
}

// statsAll: [tp][M] entries of pass 1 from every rank (this rank's included).
__global__ void __launch_bounds__(kCeThreads) ceFinishKernel(bf16* logits, const long* targets, const float4* statsAll, int tp,
                                                             float* loss, int M, int V, long ld, long vocabOffset, float gscale) {
  const int nvec = V / 8;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    bf16* lr = logits + (long)row * ld;
    const long tgtGlobal = targets[row];
    const long tgt = tgtGlobal - vocabOffset;
    float gm = -INFINITY;
    for (int r = 0; r < tp; ++r) gm = fmaxf(gm, statsAll[(long)r * M + row].x);
    float S = 0.f, tl = 0.f;
    for (int r = 0; r < tp; ++r) {
      const float4 st = statsAll[(long)r * M + row];
      S += st.y * __expf(st.x - gm);
      tl += st.z;
    }
    const bool ignore = tgtGlobal < 0;
    if (threadIdx.x == 0) loss[row] = ignore ? 0.f : (__logf(S) + gm - tl);
    const float inv = 1.f / S;
#pragma unroll
    for (int i = 0; i < kCeMaxVec; ++i) {
      const int vi = threadIdx.x + i * kCeThreads;
      if (vi < nvec) {
        float v[8], o[8];
        Vec8<bf16>::load(lr + vi * 8, 8, true, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float p = __expf(v[j] - gm) * inv;
          const bool hit = (long)(vi * 8 + j) == tgt;
          o[j] = ignore ? 0.f : (p - (hit ? 1.f : 0.f)) * gscale;
        }
        Vec8<bf16>::store(lr + vi * 8, 8, true, o);
      }
    }
  }
}

// ---------------------------------------------------------------- optimizer
// AdamW on a flat shard: fp32 master/m/v, fp32 or bf16 gradients, bf16 model copy.
// gradScale (device scalar, optional) multiplies every gradient (loss scaling x clip).
template <typename G>
__global__ void __launch_bounds__(256) adamKernel(float* master, float* m, float* v, const G* grad, bf16* param,
                                                  long n, float lr, float b1, float b2, float eps, float wd,
                                                  float bc1, float bc2, const float* gradScale) {
  const float gs = gradScale ? *gradScale : 1.f;
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (long)gridDim.x * blockDim.x * 8) {
    const long left = n - i;
    const bool vec = left >= 8;
    float w[8], mm[8], vv[8], g[8];
    Vec8<float>::load(master + i, left, vec, w);
    Vec8<float>::load(m + i, left, vec, mm);
    Vec8<float>::load(v + i, left, vec, vv);
    Vec8<G>::load(grad + i, left, vec && aligned16(grad + i), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gs;
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      const float mh = mm[j] / bc1, vh = vv[j] / bc2;
      w[j] = w[j] - lr * (mh / (sqrtf(vh) + eps) + wd * w[j]);
    }
    Vec8<float>::store(master + i, left, vec, w);
    Vec8<float>::store(m + i, left, vec, mm);
    Vec8<float>::store(v + i, left, vec, vv);
    if (param) Vec8<bf16>::store(param + i, left, vec && aligned16(param + i), w);
  }
}

template <typename G>
__global__ void __launch_bounds__(256) sumSqPartialKernel(const G* x, long n, float* partial) {
  __shared__ float sm[32];
  float s = 0.f;
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (long)gridDim.x * blockDim.x * 8) {
    float v[8];
    const long left = n - i;
    Vec8<G>::load(x + i, left, left >= 8 && aligned16(x + i), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[j] * v[j];
  }
  s = blockSum(s, sm);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// out[0] (+)= sum(partial)
__global__ void __launch_bounds__(256) sumFinalKernel(const float* partial, int n, float* out, int accumulate) {
  __shared__ float sm[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = blockSum(s, sm);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}
// coef = gradScaleIn * min(1, maxNorm / (sqrt(sumsq) * gradScaleIn + 1e-6))
__global__ void clipCoefKernel(const float* sumsq, float maxNorm, float gradScaleIn, float* coef, float* normOut) {
  const float norm = sqrtf(sumsq[0]) * gradScaleIn;
  if (normOut) normOut[0] = norm;
  float c = 1.f;
  if (maxNorm > 0.f && norm > maxNorm) c = maxNorm / (norm + 1e-6f);
  coef[0] = c * gradScaleIn;
}

// dst(fp32) += src(bf16)  /  dst = src
__global__ void __launch_bounds__(256) accumBf16Kernel(float* dst, const bf16* src, long n, int accumulate) {
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (long)gridDim.x * blockDim.x * 8) {
    const long left = n - i;
    const bool vec = left >= 8;
    float a[8], b[8];
    Vec8<bf16>::load(src + i, left, vec && aligned16(src + i), b);
    if (accumulate) {
      Vec8<float>::load(dst + i, left, vec, a);
#pragma unroll
      for (int j = 0; j < 8; ++j) b[j] += a[j];
    }
    Vec8<float>::store(dst + i, left, vec, b);
  }
}

static int gridForElems(long n, int per) {
  long b = (n + per - 1) / per;
  const long cap = 148L * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace coccl

using namespace coccl;

extern "C" int cocclkLayerNormFwd(const void* x, const void* res, const void* gamma, const void* beta, void* y,
                                  void* xOut, float* mean, float* rstd, int M, int H, float eps, cudaStream_t s) {
  if (H % 8 || H > kLnThreads * kLnMaxVec * 8 || M <= 0) return -1;
  const int grid = M < 148 * 8 ? M : 148 * 8;
  const int nv = (H / 8 + kLnThreads - 1) / kLnThreads;
#define LN_FWD(NV) lnFwdKernel<NV><<<grid, kLnThreads, 0, s>>>((const bf16*)x, (const bf16*)res, (const bf16*)gamma, \
      (const bf16*)beta, (bf16*)y, (bf16*)xOut, mean, rstd, M, H, eps)
  if (nv <= 1) LN_FWD(1); else if (nv <= 2) LN_FWD(2); else if (nv <= 4) LN_FWD(4); else LN_FWD(8);
#undef LN_FWD
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

extern "C" int cocclkLayerNormBwdGrid(int M) { return M < 148 * 2 ? M : 148 * 2; }

extern "C" int cocclkLayerNormBwd(const void* dy, const void* x, const float* mean, const float* rstd,
                                  const void* gamma, const void* dres, void* dx, float* dgamma, float* dbeta,
                                  int accumulate, float* scratch, int M, int H, cudaStream_t s) {
  if (H % 8 || H > kLnThreads * kLnMaxVec * 8 || M <= 0) return -1;
  const int grid = cocclkLayerNormBwdGrid(M);
  const int nv = (H / 8 + kLnThreads - 1) / kLnThreads;
#define LN_BWD(NV) lnBwdKernel<NV><<<grid, kLnThreads, 0, s>>>((const bf16*)dy, (const bf16*)x, mean, rstd, \
      (const bf16*)gamma, (const bf16*)dres, (bf16*)dx, scratch, M, H)
  if (nv <= 1) LN_BWD(1); else if (nv <= 2) LN_BWD(2); else if (nv <= 4) LN_BWD(4); else LN_BWD(8);
#undef LN_BWD
  // scratch rows are [dgamma | dbeta], 2H floats each
  colReduceKernel<<<(H + kColReduceCols - 1) / kColReduceCols, 256, 0, s>>>(scratch, dgamma, grid, H, 2L * H, accumulate);
  colReduceKernel<<<(H + kColReduceCols - 1) / kColReduceCols, 256, 0, s>>>(scratch + H, dbeta, grid, H, 2L * H, accumulate);
  cocclkCountLaunches(3);
  return (int)cudaGetLastError();
}

extern "C" int cocclkColSumBlocks(int M) { int b = (M + 127) / 128; return b > 64 ? 64 : (b < 1 ? 1 : b); }

extern "C" int cocclkColSum(const void* x, float* out, int accumulate, float* scratch, int M, int N, cudaStream_t s) {
  if (N % 8 || M <= 0) return -1;
  const int by = cocclkColSumBlocks(M);
  const int rowsPer = (M + by - 1) / by;
  dim3 grid((N / 8 + 31) / 32, by);
  colSumPartialKernel<<<grid, 256, 0, s>>>((const bf16*)x, scratch, M, N, rowsPer);
  colReduceKernel<<<(N + kColReduceCols - 1) / kColReduceCols, 256, 0, s>>>(scratch, out, by, N, N, accumulate);
  cocclkCountLaunches(2);
  return (int)cudaGetLastError();
}

extern "C" int cocclkGeluFwd(const void* z, const void* bias, void* y, void* zOut, long n, int N, cudaStream_t s) {
  if (n % 8 || N % 8) return -1;
  geluFwdKernel<<<gridForElems(n, 2048), 256, 0, s>>>((const bf16*)z, (const bf16*)bias, (bf16*)y, (bf16*)zOut, n, N);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}
extern "C" int cocclkGeluBwd(const void* dy, const void* z, void* dz, long n, cudaStream_t s) {
  if (n % 8) return -1;
  geluBwdKernel<<<gridForElems(n, 2048), 256, 0, s>>>((const bf16*)dy, (const bf16*)z, (bf16*)dz, n);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

extern "C" int cocclkCrossEntropy(void* logits, const long* targets, float* loss, int M, int V, long ld,
                                  float gscale, cudaStream_t s) {
  if (V % 8 || V > kCeThreads * kCeMaxVec * 8 || ld % 8 || M <= 0) return -1;
  const int grid = M < 148 * 2 ? M : 148 * 2;
  crossEntropyKernel<<<grid, kCeThreads, 0, s>>>((bf16*)logits, targets, loss, M, V, ld, gscale);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

extern "C" int cocclkCrossEntropyStats(const void* logits, const long* targets, float* stats, int M, int V, long ld,
                                       long vocabOffset, cudaStream_t s) {
  if (V % 8 || V > kCeThreads * kCeMaxVec * 8 || ld % 8 || M <= 0) return -1;
  const int grid = M < 148 * 2 ? M : 148 * 2;
  ceStatsKernel<<<grid, kCeThreads, 0, s>>>((const bf16*)logits, targets, reinterpret_cast<float4*>(stats), M, V, ld, vocabOffset);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}
extern "C" int cocclkCrossEntropyFinish(void* logits, const long* targets, const float* statsAll, int tp, float* loss, int M,
                                        int V, long ld, long vocabOffset, float gscale, cudaStream_t s) {
  if (V % 8 || V > kCeThreads * kCeMaxVec * 8 || ld % 8 || M <= 0 || tp < 1) return -1;
  const int grid = M < 148 * 2 ? M : 148 * 2;
  ceFinishKernel<<<grid, kCeThreads, 0, s>>>((bf16*)logits, targets, reinterpret_cast<const float4*>(statsAll), tp, loss, M, V, ld,
                                             vocabOffset, gscale);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

extern "C" int cocclkAdam(float* master, float* m, float* v, const void* grad, int gradIsBf16, void* param, long n,
                          float lr, float b1, float b2, float eps, float wd, int step, const float* gradScale,
                          cudaStream_t s) {
  if (n <= 0) return -1;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  const int grid = gridForElems(n, 2048);
  if (gradIsBf16)
    adamKernel<bf16><<<grid, 256, 0, s>>>(master, m, v, (const bf16*)grad, (bf16*)param, n, lr, b1, b2, eps, wd, bc1, bc2, gradScale);
  else
    adamKernel<float><<<grid, 256, 0, s>>>(master, m, v, (const float*)grad, (bf16*)param, n, lr, b1, b2, eps, wd, bc1, bc2, gradScale);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

extern "C" int cocclkSumSqBlocks(long n) { return gridForElems(n, 8192); }

extern "C" int cocclkSumSq(const void* x, int isBf16, long n, float* out, int accumulate, float* scratch,
                           cudaStream_t s) {
  if (n <= 0) return -1;
  const int grid = cocclkSumSqBlocks(n);
  if (isBf16) sumSqPartialKernel<bf16><<<grid, 256, 0, s>>>((const bf16*)x, n, scratch);
  else sumSqPartialKernel<float><<<grid, 256, 0, s>>>((const float*)x, n, scratch);
  sumFinalKernel<<<1, 256, 0, s>>>(scratch, grid, out, accumulate);
  cocclkCountLaunches(2);
  return (int)cudaGetLastError();
}

extern "C" int cocclkClipCoef(const float* sumsq, float maxNorm, float gradScaleIn, float* coef, float* normOut,
                              cudaStream_t s) {
  clipCoefKernel<<<1, 1, 0, s>>>(sumsq, maxNorm, gradScaleIn, coef, normOut);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

extern "C" int cocclkAccumBf16(float* dst, const void* src, long n, int accumulate, cudaStream_t s) {
  if (n <= 0) return -1;
  accumBf16Kernel<<<gridForElems(n, 2048), 256, 0, s>>>(dst, (const bf16*)src, n, accumulate);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Allocation-free column sum (see no_alloc_api.h). The scratch lives in the library
// image; host code must not pass the symbol itself to a kernel (on the host the name
// is only a stand-in), so the device address is looked up once per device.
// ---------------------------------------------------------------------------
namespace coccl {
constexpr int kNoAllocRows = 64;  // == upper bound of cocclkColSumBlocks
static __device__ __align__(256) float gColSumScratch[kNoAllocRows * COCCLK_NOALLOC_MAX_COLS];
static float* gColSumScratchAddr[COCCLK_NOALLOC_MAX_DEVICES];
static std::mutex gNoAllocMutex;
static thread_local char gNoAllocError[256] = "";
}  // namespace coccl

extern "C" const char* cocclkNoAllocLastError(void) { return coccl::gNoAllocError; }

extern "C" int cocclkColSumNoAlloc(const void* x, float* out, int accumulate, int M, int N, cudaStream_t s) {
  using namespace coccl;
  gNoAllocError[0] = 0;
  if (M <= 0 || N <= 0 || (N % 8) != 0) {
    snprintf(gNoAllocError, sizeof(gNoAllocError), "cocclkColSumNoAlloc: need M > 0 and N a positive multiple of 8 (M=%d N=%d)", M, N);
    return COCCLK_NOALLOC_BAD_SHAPE;
  }
  if (N > COCCLK_NOALLOC_MAX_COLS) {
    snprintf(gNoAllocError, sizeof(gNoAllocError),
             "cocclkColSumNoAlloc: N=%d exceeds the built-in scratch (max %d columns); use cocclkColSum with caller scratch",
             N, COCCLK_NOALLOC_MAX_COLS);
    return COCCLK_NOALLOC_TOO_LARGE;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= COCCLK_NOALLOC_MAX_DEVICES) {
    snprintf(gNoAllocError, sizeof(gNoAllocError), "cocclkColSumNoAlloc: device index %d is outside the address cache (0..%d)", dev,
             COCCLK_NOALLOC_MAX_DEVICES - 1);
    return COCCLK_NOALLOC_BAD_SHAPE;
  }
  float* scratch;
  {
    std::lock_guard<std::mutex> lock(gNoAllocMutex);
    if (gColSumScratchAddr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, gColSumScratch);  // device `dev` is current
      if (e != cudaSuccess) {
        snprintf(gNoAllocError, sizeof(gNoAllocError), "cocclkColSumNoAlloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        return (int)e;
      }
      gColSumScratchAddr[dev] = static_cast<float*>(p);
    }
    scratch = gColSumScratchAddr[dev];
  }
  const int by = cocclkColSumBlocks(M);  // <= kNoAllocRows
  const int rowsPer = (M + by - 1) / by;
  dim3 grid((N / 8 + 31) / 32, by);
  colSumPartialKernel<<<grid, 256, 0, s>>>((const bf16*)x, scratch, M, N, rowsPer);
  colReduceKernel<<<(N + kColReduceCols - 1) / kColReduceCols, 256, 0, s>>>(scratch, out, by, N, N, accumulate);
  cocclkCountLaunches(2);
  return (int)cudaGetLastError();
}
