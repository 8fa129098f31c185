// C entry points of the tcgen05 GEMM family (libcoccl.so).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  GEMM_EPI_NONE = 0,       // C(bf16) = A*B^T
  GEMM_EPI_BIAS = 1,       // C = A*B^T + bias[n]
  GEMM_EPI_BIAS_GELU = 2,  // Z = A*B^T + bias (optional), C = gelu_tanh(Z)
  GEMM_EPI_F32_ACC = 3,    // C(fp32) += A*B^T
  GEMM_EPI_F32 = 4,        // C(fp32) = A*B^T
};

// bf16 inputs, fp32 accumulation in TMEM.
//   aMN == 0: A is [M,K] with K contiguous, rows lda elements apart
//   aMN == 1: A is stored [K,M] with M contiguous (lda = distance between k rows)
//   bMN likewise for B ([N,K] or [K,N]).
// N and K must be multiples of 8; base pointers 16-byte aligned.
// `err` (optional, device memory) receives a non-zero code if a bounded wait ran out.
// Returns 0 or a cudaError_t / negative argument error.
int cocclkGemmBf16(const void* A, long lda, int aMN, const void* B, long ldb, int bMN, void* C, long ldc, int M,
                   int N, int K, int epi, const void* bias, void* Z, unsigned int* err, int maxCtas,
                   cudaStream_t stream);

// Tensor maps of repeated (address, shape, pitch) requests come from a per-thread table instead of the driver:
// (hits, misses) since the library was loaded.
void cocclkTensorMapCacheStats(unsigned long long* hits, unsigned long long* misses);

#ifdef __cplusplus
}
#endif
