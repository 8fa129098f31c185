// C entry points of the tensor-parallel fusions (libcoccl.so): all-gather -> GEMM and
// GEMM -> FP8-compressed reduce-scatter, each ONE persistent tcgen05 kernel that moves its operand or
// result tiles over peer memory while the tensor cores work on other tiles.
//
// The reference has no GEMM; these kernels serve the traffic its policy slots
// training.tp.{all_gather,reduce_scatter} (core/config/coccl_config.cc:669-695) compress.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { COCCLK_TP_MAX_RANKS = 8, COCCLK_TP_MAX_EMULATED = 4 };

// Arrays are indexed by rank. A production launch (emulatedRanks == 1) reads a/b/c/bias/z/err only at
// [rankBase]; ws/flags/status must hold every rank's buffer as mapped into this process. An emulated launch
// (all ranks on one GPU, for tests) fills every entry with local pointers.
typedef struct {
  int nRanks, rankBase;
  int M, N, K;        // ag_gemm: C[M,N] = gather(A)[M,K] * B[N,K]^T; gemm_rs: out[M/nRanks,N] = reduce_scatter(A[M,K] * B[N,K]^T)
  int epi;            // ag_gemm: GEMM_EPI_NONE | GEMM_EPI_BIAS | GEMM_EPI_BIAS_GELU
  int bMN;            // 0: B is [N, K] with K contiguous; 1: B is stored [K, N] with N contiguous (backward passes)
  unsigned int epoch; // strictly increasing per workspace; flags carry it
  unsigned long long timeoutNs;
  const void* a[COCCLK_TP_MAX_RANKS];     // ag_gemm: own shard [M/nRanks, K] bf16; gemm_rs: A [M, K] bf16
  const void* b[COCCLK_TP_MAX_RANKS];     // bf16 weights, layout per bMN
  void* c[COCCLK_TP_MAX_RANKS];           // ag_gemm: [M, N] bf16; gemm_rs: [M/nRanks, N] bf16
  const void* bias[COCCLK_TP_MAX_RANKS];  // optional bf16 [N]: ag_gemm adds it in the epilogue; gemm_rs (CTA-pair kernel only)
                                          // adds it once, to the reduced rows
  void* z[COCCLK_TP_MAX_RANKS];           // ag_gemm with GELU: optional pre-activation output
  void* ws[COCCLK_TP_MAX_RANKS];          // ag_gemm: gather buffer [M, K] bf16; gemm_rs: nRanks receive slots
  unsigned int* flags[COCCLK_TP_MAX_RANKS];  // cocclkFlagBytes() bytes each
  void* status[COCCLK_TP_MAX_RANKS];         // StatusWord
  unsigned int* err[COCCLK_TP_MAX_RANKS];    // optional: GEMM pipeline error word
  void* gathered[COCCLK_TP_MAX_RANKS];       // ag_gemm (CTA-pair kernel only), optional: [M, K] bf16 that receives the whole
                                             // gathered operand (the backward pass needs it for the weight gradient);
                                             // the kernel's push warps copy it out of the gather buffer as shards arrive
  int agPayload;      // ag_gemm (CTA-pair kernel only): what travels between the ranks. 0: the bf16 rows as they are.
                      // 1: E4M3 with one UE8M0 scale per 32 columns (half the bytes on the wire); the push warps of the
                      // sender quantise, the push warps of the receiver dequantise each piece on arrival into the bf16
                      // gather buffer the tensor cores read. Needs K % 32 == 0 and the larger workspace of
                      // cocclkAgGemmWorkspaceBytesFor; the single-CTA kernel ignores it.
} cocclkTpArgs;

// Which kernel family served the last fusion call of this process: 1 = single-CTA tiles, 2 = CTA pairs. The single-CTA
// kernels ignore `gathered` and gemm_rs's `bias`; a caller that passed them applies them itself in that case.
int cocclkTpLastVariant(void);

// Bytes of ws[] per rank.
long cocclkAgGemmWorkspaceBytes(int M, int K);
long cocclkAgGemmWorkspaceBytesFor(int M, int K, int agPayload);   // bf16 gather buffer [+ FP8 rows + scales]
long cocclkGemmRsWorkspaceBytes(int M, int N, int nRanks);

// Constraints: M % (nRanks * 128) == 0, K % 8 == 0; gemm_rs also N % 256 == 0; ag_gemm N % 8 == 0.
// maxCtas limits the CTAs per rank (0 = one per SM). Returns 0, a cudaError_t or a negative argument error.
int cocclkAgGemm(const cocclkTpArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream);
int cocclkGemmRs(const cocclkTpArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
