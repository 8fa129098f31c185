// Generic helpers of the staged (plugin) pipeline:
//  * reduceChunks: out = sum of `numChunks` equal chunks, fp32 accumulation for floating types and
//    native wrap-around arithmetic for integer types (lossless codecs route integers). Replaces the
//    reference's reduceChunk / reduceChunkInteger (core/device/reduce_helper/reduce_extend_kernel.cu:285-393).
//  * packSlice / unpackSlice: gather the same element range of every rank chunk into a contiguous
//    buffer and back, with the optional hierarchical rank swizzle
//    dest = (src % ranksPerNode) * nNodes + src / ranksPerNode
//    (core/device/pipeline/coccl_pipeline_layout.cu:13-121).
#include "common.cuh"
#include "kernels_api.h"
#include "launch_count.h"

namespace coccl {

template <typename T, typename Acc>
__global__ void __launch_bounds__(256) reduceChunksKernel(const T* in, T* out, long count, int numChunks, long pitch) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long)gridDim.x * blockDim.x) {
    Acc acc = (Acc)in[i];
    for (int c = 1; c < numChunks; ++c) acc += (Acc)in[(long)c * pitch + i];
    out[i] = (T)acc;
  }
}

template <typename V>
__global__ void __launch_bounds__(256) packKernel(const char* src, char* dst, long sliceBytes, long srcPitch,
                                                  long srcOffset, int chunks, int ranksPerNode, int nNodes,
                                                  int unpack) {
  const long vecs = sliceBytes / (long)sizeof(V);
  for (int ch = blockIdx.y; ch < chunks; ch += gridDim.y) {
    int dch = ch;
    if (ranksPerNode > 0) dch = (ch % ranksPerNode) * nNodes + ch / ranksPerNode;
    const char* s = unpack ? src + (long)ch * sliceBytes : src + (long)ch * srcPitch + srcOffset;
    char* d = unpack ? dst + (long)ch * srcPitch + srcOffset : dst + (long)dch * sliceBytes;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (long)gridDim.x * blockDim.x)
      reinterpret_cast<V*>(d)[i] = reinterpret_cast<const V*>(s)[i];
  }
}

}  // namespace coccl

using namespace coccl;

// dtype codes here are NCCL's: 0 i8, 1 u8, 2 i32, 3 u32, 4 i64, 5 u64, 6 f16, 7 f32, 8 f64, 9 bf16
extern "C" int cocclkReduceChunks(const void* in, void* out, long count, int numChunks, long pitchElems, int ncclType,
                                  cudaStream_t stream) {
  if (count <= 0 || numChunks <= 0) return -1;
  long blocks = (count + 255) / 256;
  const int grid = (int)(blocks > 148 * 16 ? 148 * 16 : blocks);
#define RUN(T, A) reduceChunksKernel<T, A><<<grid, 256, 0, stream>>>((const T*)in, (T*)out, count, numChunks, pitchElems)
  switch (ncclType) {
    case 0: RUN(signed char, int); break;
    case 1: RUN(unsigned char, unsigned int); break;
    case 2: RUN(int, int); break;
    case 3: RUN(unsigned int, unsigned int); break;
    case 4: RUN(long long, long long); break;
    case 5: RUN(unsigned long long, unsigned long long); break;
    case 6: RUN(__half, float); break;
    case 7: RUN(float, float); break;
    case 8: RUN(double, double); break;
    case 9: RUN(__nv_bfloat16, float); break;
    default: return -1;
  }
#undef RUN
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}

// pack (unpack=0): dst[dchunk][0..sliceBytes) = src[chunk*srcPitch + srcOffset ...]; unpack (1): the inverse
// (no swizzle on unpack). ranksPerNode <= 0 disables the swizzle.
extern "C" int cocclkPackSlice(const void* src, void* dst, long sliceBytes, long srcPitchBytes, long srcOffsetBytes,
                               int chunks, int ranksPerNode, int nNodes, int unpack, cudaStream_t stream) {
  if (sliceBytes <= 0 || chunks <= 0) return -1;
  const uintptr_t bits = (uintptr_t)src | (uintptr_t)dst | (uintptr_t)sliceBytes | (uintptr_t)srcPitchBytes |
                         (uintptr_t)srcOffsetBytes;
  int width = 16;
  while (width > 1 && (bits & (uintptr_t)(width - 1))) width >>= 1;
  const long vecs = sliceBytes / width;
  long bx = (vecs + 255) / 256;
  if (bx > 1024) bx = 1024;
  dim3 grid((unsigned)bx, (unsigned)(chunks > 65535 ? 65535 : chunks));
  const char* s = (const char*)src;
  char* d = (char*)dst;
#define RUN(V) packKernel<V><<<grid, 256, 0, stream>>>(s, d, sliceBytes, srcPitchBytes, srcOffsetBytes, chunks, unpack ? 0 : ranksPerNode, nNodes, unpack)
  switch (width) {
    case 16: RUN(uint4); break;
    case 8: RUN(uint2); break;
    case 4: RUN(unsigned int); break;
    case 2: RUN(unsigned short); break;
    default: RUN(unsigned char); break;
  }
#undef RUN
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}
