// sm_100a GEMM building blocks: raw PTX wrappers for TMA (cp.async.bulk.tensor),
// mbarrier, tcgen05.mma with TMEM accumulators and tcgen05.ld, plus the shared
// memory / instruction descriptor encoders. Used by the plain GEMM, the
// GEMM -> compressed reduce-scatter and the all-gather -> GEMM kernels.
//
// The reference has no GEMM at all (it is a collective library); these kernels
// implement the tensor-parallel fusions that the policy slots
// training.tp.{all_gather,reduce_scatter,all_reduce}
// (core/config/coccl_config.cc:669-695) are meant to accelerate.
//
// No TMA load in this file uses cluster multicast.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace coccl {
namespace sm100 {

__device__ __forceinline__ uint32_t smemAddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool electOne() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbarInit(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void mbarFenceInit() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbarArriveExpectTx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\tmbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\tselp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smemAddr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up after `limitNs`, or as soon as another role has set *abortFlag.
__device__ __forceinline__ bool mbarWait(uint64_t* bar, uint32_t parity, volatile int* abortFlag,
                                         unsigned long long limitNs) {
  if (mbarTryWait(bar, parity)) return true;
  const unsigned long long start = gtimer();
  uint32_t spins = 0;
  while (!mbarTryWait(bar, parity)) {
    if ((++spins & 255u) == 0u) {
      if (*abortFlag) return false;
      if (gtimer() - start > limitNs) { *abortFlag = 1; return false; }
    }
  }
  return true;
}

// ------------------------------------------------------------------ TMA
__device__ __forceinline__ void tmaLoad2d(void* smemDst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smemAddr(smemDst)), "l"(map), "r"(smemAddr(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void prefetchTensorMap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ------------------------------------------------------------------ TMEM / tcgen05
__device__ __forceinline__ void tmemAlloc(uint32_t* smemSlot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(smemSlot)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmemRelinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemDealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; accumulate = 0 overwrites D.
__device__ __forceinline__ void umma(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every previously issued tcgen05.mma has completed.
__device__ __forceinline__ void ummaCommit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemAddr(bar))
               : "memory");
}
// 32 lanes x 32 columns of fp32: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmemLd32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmemLdWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor, 128-byte swizzle (tile rows are 128 bytes).
//  K-major operand : rows of 64 bf16 along K; 8-row atoms 1024 B apart (SBO).
//  MN-major operand: rows of 64 bf16 along M/N, one row per k; 8-k atoms 1024 B
//                    apart (SBO); 64-wide M/N blocks `lboBytes` apart (LBO).
__device__ __forceinline__ uint64_t makeSmemDesc(uint32_t saddr, uint32_t lboBytes, uint32_t sboBytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fffu);
  d |= (uint64_t)((lboBytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sboBytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}
// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
__host__ __device__ inline uint32_t makeInstrDescBf16(int M, int N, bool aMN, bool bMN) {
  uint32_t d = 0;
  d |= 1u << 4;                         // D format: f32
  d |= 1u << 7;                         // A format: bf16
  d |= 1u << 10;                        // B format: bf16
  d |= (aMN ? 1u : 0u) << 15;           // A major: 0 = K, 1 = MN
  d |= (bMN ? 1u : 0u) << 16;           // B major
  d |= ((uint32_t)(N >> 3) & 0x3f) << 17;
  d |= ((uint32_t)(M >> 4) & 0x1f) << 24;
  return d;
}

// ------------------------------------------------------------------ CTA pairs (cta_group::2)
__device__ __forceinline__ uint32_t clusterCtaRank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Cluster-window address of the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t mapToCta(uint32_t localAddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(localAddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void clusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbarArriveRemote(uint32_t clusterAddr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
__device__ __forceinline__ void stSharedRemote(uint32_t clusterAddr, int v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(clusterAddr), "r"(v) : "memory");
}
// TMA load issued by either CTA of a pair; the completion bytes are credited to the mbarrier at
// cluster address `barClusterAddr` (the leader CTA's barrier). No multicast.
__device__ __forceinline__ void tmaLoad2dPair(void* smemDst, const CUtensorMap* map, uint32_t barClusterAddr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smemAddr(smemDst)), "l"(map), "r"(barClusterAddr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmemAlloc2(uint32_t* smemSlot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(smemSlot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmemRelinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemDealloc2(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// One MMA over the CTA pair: M = 256 (128 rows from each CTA), B halves from each CTA.
__device__ __forceinline__ void umma2(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the mbarrier at the same offset in every CTA of `ctaMask` once all earlier MMAs are done.
__device__ __forceinline__ void ummaCommit2(uint64_t* bar, uint16_t ctaMask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smemAddr(bar)), "h"(ctaMask) : "memory");
}

// ------------------------------------------------------------------ TMA stores / reductions (shared -> global)
// Make generic-proxy writes to shared memory visible to the async proxy (TMA) before it reads them.
__device__ __forceinline__ void fenceProxyAsyncShared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Write a box from shared memory to the tensor at (x, y); parts outside the tensor are clipped.
__device__ __forceinline__ void tmaStore2d(const CUtensorMap* map, const void* smemSrc, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smemAddr(smemSrc)), "r"(x), "r"(y) : "memory");
}
// Add a box from shared memory into the tensor at (x, y) (element type from the tensor map); the addition runs in L2.
__device__ __forceinline__ void tmaReduceAdd2d(const CUtensorMap* map, const void* smemSrc, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smemAddr(smemSrc)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulkCommitGroup() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N> __device__ __forceinline__ void bulkWaitGroupRead() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Wait until at most N of this thread's bulk groups are still in flight at all.
template <int N> __device__ __forceinline__ void bulkWaitGroup() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ float geluTanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * x * (1.f + k1 * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.f + t);
}

}  // namespace sm100
}  // namespace coccl
