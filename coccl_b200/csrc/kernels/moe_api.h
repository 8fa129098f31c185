// C entry points of the expert-parallel token exchange (libcoccl.so).
//
// The reference offers only a compressed AllToAll of equal chunks for this traffic
// (extensions/primitives/coccl_alltoall.cc:12-21); here the top-k routing is part of the kernels:
//   cocclkMoeLayout    ranks every (token, choice) inside its expert's queue (stable, deterministic)
//   cocclkMoeDispatch  gathers the routed rows, quantises them to E4M3 with UE8M0 scales per 32 values and
//                      stores them straight into the destination ranks' receive slots; the receiving side
//                      dequantises them into an expert-major bf16 matrix
//   cocclkMoeCombine   sends the expert outputs back as bf16 and forms the gate-weighted sum per token
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { COCCLK_MOE_MAX_RANKS = 8, COCCLK_MOE_MAX_LOCAL_EXPERTS = 64, COCCLK_MOE_MAX_EXPERTS = 256 };

// Arrays are indexed by rank; a production launch (emulatedRanks == 1) reads the per-rank inputs and outputs
// only at [rankBase], while ws/flags/status hold every rank's buffer as mapped into this process.
typedef struct {
  int nRanks, rankBase;
  int tokens;            // tokens per rank
  int hidden;            // multiple of 256
  int topk;              // choices per token (<= 8)
  int experts;           // total experts, multiple of nRanks
  int capacity;          // rows a rank can receive from ONE source; rows past it are dropped (tokens * topk never overflows)
  unsigned int epoch;
  unsigned long long timeoutNs;
  const void* x[COCCLK_MOE_MAX_RANKS];           // dispatch: [tokens, hidden] bf16
  const int* expertIds[COCCLK_MOE_MAX_RANKS];    // [tokens, topk]
  const float* gates[COCCLK_MOE_MAX_RANKS];      // combine: [tokens, topk]
  const int* pos[COCCLK_MOE_MAX_RANKS];          // from cocclkMoeLayout: position inside the destination rank's block
  const int* sendCounts[COCCLK_MOE_MAX_RANKS];   // from cocclkMoeLayout: [experts] rows routed to each expert
  void* recv[COCCLK_MOE_MAX_RANKS];              // dispatch out: [nRanks * capacity, hidden] bf16, expert-major, packed
  int* recvOffsets[COCCLK_MOE_MAX_RANKS];        // dispatch out: [localExperts + 1] row offsets into recv
  int* recvCounts[COCCLK_MOE_MAX_RANKS];         // dispatch out / combine in: [nRanks, localExperts] rows per (source, expert)
  const void* y[COCCLK_MOE_MAX_RANKS];           // combine: expert outputs, same layout as recv
  void* out[COCCLK_MOE_MAX_RANKS];               // combine out: [tokens, hidden] bf16
  const float* rowScale[COCCLK_MOE_MAX_RANKS];   // dispatch, optional: [tokens, topk] factor applied to the row of every entry
  const void* dotWith[COCCLK_MOE_MAX_RANKS];     // combine, optional: [tokens, hidden] bf16 ...
  float* dotOut[COCCLK_MOE_MAX_RANKS];           // ... dotOut[t, j] = <returned row of entry (t, j), dotWith[t]> (gate gradients)
  void* ws[COCCLK_MOE_MAX_RANKS];                // cocclkMoeWorkspaceBytes() bytes
  unsigned int* flags[COCCLK_MOE_MAX_RANKS];     // cocclkFlagBytes() bytes
  void* status[COCCLK_MOE_MAX_RANKS];
} cocclkMoeArgs;

long cocclkMoeWorkspaceBytes(int nRanks, int capacity, int hidden, int localExperts);

// expertIds [entries] -> pos [entries], counts [experts]; one CTA, deterministic. entries = tokens * topk.
int cocclkMoeLayout(const int* expertIds, int entries, int experts, int expertsPerRank, int* pos, int* counts,
                    cudaStream_t stream);
int cocclkMoeDispatch(const cocclkMoeArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream);
int cocclkMoeCombine(const cocclkMoeArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
