// C entry points of the device layer (libcoccl.so). Everything here takes raw
// device pointers and a CUDA stream; nothing allocates unless stated.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Mirrors coccl::CodecCfg (kernels/codecs.cuh).
typedef struct cocclkCodec {
  int kind;        // 0 sdp4bit, 1 mxfp8, 3 taco, 4 zfp
  int bits;        // zfp: the rate (4, 8 or 16 bits per value on the tile path)
  int group;       // zfp: 4
  int asym;
  int hadamard;
  int stochastic;
  int paramBytes;  // taco: 8; zfp: 0
  uint32_t seed;
  int aux;         // taco: bit 0 = E5M2, bit 1 = saturate
  float f0, f1, f2;  // taco: targetRange, lambda, fp8 maximum
} cocclkCodec;

// dtype: 0 fp32, 1 fp16, 2 bf16. All return a cudaError_t value (0 = ok) or
// -1 for an unsupported configuration.
long cocclkEncodedChunkBytes(const cocclkCodec* codec, long count);
int cocclkTileCodecSupported(const cocclkCodec* codec);

// `chunks` raw chunks of `count` elements (rawPitch elements apart) ->
// `chunks` encoded chunks `encStride` bytes apart.
int cocclkEncode(const void* in, void* out, long count, long chunks, long rawPitch, long encStride, int dtype,
                 const cocclkCodec* codec, cudaStream_t stream);
// out chunk j (j < chunks) = sum over i < reduce of decode(in chunk i*chunks + j).
int cocclkDecodeReduce(const void* in, void* out, long count, long chunks, long reduce, long rawPitch,
                       long encStride, int dtype, const cocclkCodec* codec, cudaStream_t stream);
// encoded out chunk j = encode(sum over i < reduce of decode(in chunk i*chunks + j)).
int cocclkDecodeReduceEncode(const void* in, void* out, long count, long chunks, long reduce, long encStrideIn,
                             long encStrideOut, const cocclkCodec* codec, cudaStream_t stream);

// Fused collectives. Mirrors coccl::CollArgs.
enum { COCCLK_MAX_RANKS = 8, COCCLK_MAX_SLICES = 4096, COCCLK_TRACE_MAX_CTAS = 2048 };
typedef struct cocclkCollArgs {
  int op;        // 0 RS, 1 AG, 2 A2A, 3 AR one-shot, 4 AR two-shot
  int nRanks;
  int rankBase;
  int dtype;
  long count;
  int sliceTiles;
  unsigned int epoch;
  unsigned long long timeoutNs;
  cocclkCodec codec;
  long slotBytes;
  long regionBOffset;
  const void* in[COCCLK_MAX_RANKS];
  void* out[COCCLK_MAX_RANKS];
  uint8_t* ws[COCCLK_MAX_RANKS];
  unsigned int* flags[COCCLK_MAX_RANKS];
  void* status[COCCLK_MAX_RANKS];
  /* Optional per-rank phase trace (NULL = off): CTA c writes four globaltimer values (ns) at
     trace[rank][4 c + {0: kernel start, 1: encode+push done, 2: decode(-reduce) done, 3: gather done}].
     Needs 32 bytes per CTA of the launch (COCCLK_TRACE_MAX_CTAS CTAs at most are recorded). */
  unsigned long long* trace[COCCLK_MAX_RANKS];
} cocclkCollArgs;

// Bytes of flag storage one rank needs (zero-initialised once).
long cocclkFlagBytes(void);
/* Elements per CTA tile of the codec and collective kernels (slice sizes are given in tiles). */
int cocclkTileElems(void);
// Smallest slot size (16-byte aligned) for one encoded chunk of `count` elements.
long cocclkSlotBytes(const cocclkCodec* codec, long count);
// emulatedRanks == 1: production launch for rank `rankBase` (peer pointers in
// ws/flags). emulatedRanks == nRanks: one cooperative launch plays every rank
// on the current device. maxCtas <= 0 lets the library size the grid.
int cocclkFusedCollective(const cocclkCollArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
// Staged-pipeline helpers (kernels/reduce_kernels.cu). ncclType uses NCCL's datatype codes.
int cocclkReduceChunks(const void* in, void* out, long count, int numChunks, long pitchElems, int ncclType,
                       cudaStream_t stream);
int cocclkPackSlice(const void* src, void* dst, long sliceBytes, long srcPitchBytes, long srcOffsetBytes, int chunks,
                    int ranksPerNode, int nNodes, int unpack, cudaStream_t stream);
/* Byte exchange over peer memory for the staged pipeline (kernels/exchange_kernels.cu): all-to-all (gather = 0: block p
   of send goes to rank p) or all-gather (gather = 1: the one block of send goes to every rank) of blocks made of
   `frames` frames of `frameStride` bytes capacity. With sendMeta (one 16-byte record per frame: payload bytes as a
   64-bit integer, then encoding) only the bytes that exist travel, and recvMeta receives the records in source order.
   staging[r]: cocclkExchangeStagingBytes() bytes on rank r as mapped here; flags[r]: cocclkFlagBytes() bytes.
   Arrays are indexed by rank; a production launch (emulatedRanks == 1) reads send/recv/meta at [rankBase] only. */
typedef struct {
  int nRanks, rankBase;
  int gather;
  int frames;
  int pieces;                    /* from cocclkExchangePieces */
  long frameStride, pieceBytes;  /* multiples of 16 */
  const uint8_t* send[COCCLK_MAX_RANKS];
  uint8_t* recv[COCCLK_MAX_RANKS];
  const void* sendMeta[COCCLK_MAX_RANKS];
  void* recvMeta[COCCLK_MAX_RANKS];
  uint8_t* staging[COCCLK_MAX_RANKS];
  unsigned int* flags[COCCLK_MAX_RANKS];
  void* status[COCCLK_MAX_RANKS];
  unsigned int epoch;
  unsigned long long timeoutNs;
} cocclkExchangeArgs;
long cocclkExchangeStagingBytes(int nRanks, int frames, long frameStride);
int cocclkExchangePieces(int frames, long frameStride, long* pieceBytes);
int cocclkPeerExchange(const cocclkExchangeArgs* args, int emulatedRanks, int maxCtas, cudaStream_t stream);
/* Uncompressed all-reduce of a symmetric buffer through the NVSwitch (multimem.ld_reduce / multimem.st).
   multicastPtr: multicast address of element 0 of a buffer every rank has bound to the same multicast object;
   flags[r]: cocclkNvlsFlagBytes() zero-initialised bytes on rank r as mapped here. count * size must be a multiple of
   16 * nRanks. The result replaces the buffer's contents on every rank. */
long cocclkNvlsFlagBytes(void);
int cocclkNvlsAllReduce(void* multicastPtr, long count, int dtype, int nRanks, int rank, unsigned int* const* flags,
                        void* status, unsigned int epoch, unsigned long long timeoutNs, int maxCtas, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
