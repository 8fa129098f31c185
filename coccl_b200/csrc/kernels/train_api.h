// C entry points of the trainer's memory-bound kernels (libcoccl.so).
// All tensors are bf16 unless stated; statistics and gradients of parameters
// are fp32. `scratch` arguments are caller-provided device buffers whose
// required size is given next to each function. Return 0 or a cudaError_t;
// -1 = unsupported shape.
#pragma once
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif

// y = LayerNorm(x (+ res)); xOut (optional) = x + res. H % 8 == 0, H <= 16384.
int cocclkLayerNormFwd(const void* x, const void* res, const void* gamma, const void* beta, void* y, void* xOut,
                       float* mean, float* rstd, int M, int H, float eps, cudaStream_t s);
// Number of partial rows the backward uses; scratch = grid * 2 * H floats.
int cocclkLayerNormBwdGrid(int M);
// dx = dLN/dx (+ dres); dgamma/dbeta (fp32) are overwritten or accumulated into.
int cocclkLayerNormBwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma,
                       const void* dres, void* dx, float* dgamma, float* dbeta, int accumulate, float* scratch,
                       int M, int H, cudaStream_t s);
// out[n] (+)= sum_m x[m][n]; scratch = cocclkColSumBlocks(M) * N floats.
int cocclkColSumBlocks(int M);
int cocclkColSum(const void* x, float* out, int accumulate, float* scratch, int M, int N, cudaStream_t s);
// y = gelu_tanh(z (+ bias[n % N])); zOut (optional) = z + bias.
int cocclkGeluFwd(const void* z, const void* bias, void* y, void* zOut, long n, int N, cudaStream_t s);
int cocclkGeluBwd(const void* dy, const void* z, void* dz, long n, cudaStream_t s);
// loss[m] = CE(logits[m], targets[m]); logits are overwritten by their gradient times gscale.
int cocclkCrossEntropy(void* logits, const long* targets, float* loss, int M, int V, long ld, float gscale,
                       cudaStream_t s);
// Vocabulary-parallel cross-entropy (the vocabulary is sharded over tensor-parallel ranks; this rank holds columns
// [vocabOffset, vocabOffset + V)). Stats writes 4 floats per row {local max, sum exp(logit - max), target logit or 0,
// target-in-shard flag}; the caller all-gathers them over the group into statsAll [tp][M][4]; Finish writes
// loss[m] (the same value on every rank) and overwrites the logits with (softmax - onehot) * gscale.
int cocclkCrossEntropyStats(const void* logits, const long* targets, float* stats, int M, int V, long ld, long vocabOffset,
                            cudaStream_t s);
int cocclkCrossEntropyFinish(void* logits, const long* targets, const float* statsAll, int tp, float* loss, int M, int V,
                             long ld, long vocabOffset, float gscale, cudaStream_t s);
// AdamW over a flat shard. grad is fp32 or bf16; param (optional) receives the bf16 copy.
int cocclkAdam(float* master, float* m, float* v, const void* grad, int gradIsBf16, void* param, long n, float lr,
               float b1, float b2, float eps, float wd, int step, const float* gradScale, cudaStream_t s);
// out[0] (+)= sum x^2; scratch = cocclkSumSqBlocks(n) floats.
int cocclkSumSqBlocks(long n);
int cocclkSumSq(const void* x, int isBf16, long n, float* out, int accumulate, float* scratch, cudaStream_t s);
int cocclkClipCoef(const float* sumsq, float maxNorm, float gradScaleIn, float* coef, float* normOut, cudaStream_t s);
// dst(fp32) (+)= src(bf16)
int cocclkAccumBf16(float* dst, const void* src, long n, int accumulate, cudaStream_t s);

#ifdef __cplusplus
}
#endif
