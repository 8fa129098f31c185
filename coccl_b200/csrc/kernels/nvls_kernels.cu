// Uncompressed all-reduce through the NVSwitch: every rank reduces its 1/N slice of a symmetric buffer with
// multimem.ld_reduce (the switch adds the N copies) and broadcasts the result with multimem.st. This is the
// candidate the algorithm selector uses below the compression threshold, where quantisation cannot pay for
// itself (reference counterpart: NCCL's NVLS all-reduce kernels, src/device/all_reduce.h, selected inside
// ncclAllReduce when the call stays native).
//
// The multicast address comes from a symmetric allocation that every rank has bound to one multicast object
// (torch.distributed._symmetric_memory on the Python side). Flags are ordinary peer-mapped words with the
// call's epoch; CTA c of every rank forms its own barrier with the CTAs c of the other ranks, before the
// reduction (all inputs are in place) and after it (all slices are written). Waits are bounded.
#include "common.cuh"
#include "kernels_api.h"
#include "launch_count.h"

namespace coccl {

constexpr int kNvlsMaxCtas = 256;

struct NvlsArgs {
  int nRanks, rank, dtype;
  long count;                       // elements of the whole vector; count * size % (16 * nRanks) == 0
  void* mc;                         // multicast address of element 0
  unsigned int* flags[kMaxRanks];   // [2][kMaxRanks][kNvlsMaxCtas] words on every rank
  StatusWord* status;
  unsigned int epoch;
  unsigned long long timeoutNs;
};

__device__ __forceinline__ bool ctaBarrier(const NvlsArgs& a, int which) {
  __syncthreads();
  if (threadIdx.x < a.nRanks) {
    __threadfence_system();
    stReleaseSys(a.flags[threadIdx.x] + ((long)which * kMaxRanks + a.rank) * kNvlsMaxCtas + blockIdx.x, a.epoch);
  }
  bool ok = true;
  if (threadIdx.x < a.nRanks) {
    ok = waitFlag(a.flags[a.rank] + ((long)which * kMaxRanks + threadIdx.x) * kNvlsMaxCtas + blockIdx.x, a.epoch, a.timeoutNs);
    if (!ok) reportTimeout(a.status, 8 + which, threadIdx.x, blockIdx.x);
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

__global__ void __launch_bounds__(256) nvlsAllReduceKernel(const NvlsArgs a) {
  if (!ctaBarrier(a, 0)) return;
  const long bytes = a.count * (a.dtype == kF32 ? 4 : 2);
  const long sliceVecs = bytes / a.nRanks / 16;
  char* base = reinterpret_cast<char*>(a.mc) + (long)a.rank * sliceVecs * 16;
  // four independent 16-byte reductions in flight per thread: one load per thread leaves the switch round trip exposed
  constexpr int kUnroll = 4;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long i0 = (long)blockIdx.x * blockDim.x + threadIdx.x; i0 < sliceVecs; i0 += stride * kUnroll) {
    uint32_t v[kUnroll][4];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long i = i0 + u * stride;
      if (i >= sliceVecs) break;
      char* p = base + i * 16;
      if (a.dtype == kF32)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v[u][0]), "=r"(v[u][1]), "=r"(v[u][2]), "=r"(v[u][3]) : "l"(p) : "memory");
      else if (a.dtype == kBF16)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v[u][0]), "=r"(v[u][1]), "=r"(v[u][2]), "=r"(v[u][3]) : "l"(p) : "memory");
      else
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v[u][0]), "=r"(v[u][1]), "=r"(v[u][2]), "=r"(v[u][3]) : "l"(p) : "memory");
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long i = i0 + u * stride;
      if (i >= sliceVecs) break;
      char* p = base + i * 16;
      if (a.dtype == kF32)
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                     ::"l"(p), "r"(v[u][0]), "r"(v[u][1]), "r"(v[u][2]), "r"(v[u][3]) : "memory");
      else if (a.dtype == kBF16)
        asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                     ::"l"(p), "r"(v[u][0]), "r"(v[u][1]), "r"(v[u][2]), "r"(v[u][3]) : "memory");
      else
        asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1, %2, %3, %4};"
                     ::"l"(p), "r"(v[u][0]), "r"(v[u][1]), "r"(v[u][2]), "r"(v[u][3]) : "memory");
    }
  }
  ctaBarrier(a, 1);
}

}  // namespace coccl

using namespace coccl;

extern "C" long cocclkNvlsFlagBytes(void) { return 2L * kMaxRanks * kNvlsMaxCtas * (long)sizeof(unsigned int); }

extern "C" int cocclkNvlsAllReduce(void* multicastPtr, long count, int dtype, int nRanks, int rank, unsigned int* const* flags,
                                   void* status, unsigned int epoch, unsigned long long timeoutNs, int maxCtas,
                                   cudaStream_t stream) {
  if (!multicastPtr || nRanks < 2 || nRanks > kMaxRanks || rank < 0 || rank >= nRanks || count <= 0) return -1;
  const long bytes = count * (dtype == kF32 ? 4 : 2);
  if (bytes % (16L * nRanks) != 0) return -1;
  NvlsArgs a{};
  a.nRanks = nRanks; a.rank = rank; a.dtype = dtype; a.count = count; a.mc = multicastPtr;
  for (int r = 0; r < nRanks; ++r) a.flags[r] = flags[r];
  a.status = static_cast<StatusWord*>(status);
  a.epoch = epoch; a.timeoutNs = timeoutNs;
  // the grid must be the same on every rank: it depends on the size and on maxCtas only
  // one CTA per 4 x 256 vectors of the slice, up to the number of per-CTA barrier slots
  long ctas = (bytes / nRanks / 16 + 1023) / 1024;
  if (ctas > kNvlsMaxCtas) ctas = kNvlsMaxCtas;
  if (maxCtas > 0 && ctas > maxCtas) ctas = maxCtas;
  if (ctas < 1) ctas = 1;
  nvlsAllReduceKernel<<<(unsigned)ctas, 256, 0, stream>>>(a);
  cocclkCountLaunches(1);
  return (int)cudaGetLastError();
}
