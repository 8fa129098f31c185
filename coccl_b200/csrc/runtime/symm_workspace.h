// Collective life cycle of a peer-mapped region (workspace, flags) shared by the ranks of one communicator.
//
// Opening, growing and closing such a region is a collective act: every rank maps every peer's allocation, so
// no rank may free its allocation while a peer still has it mapped (CUDA leaves that undefined), and a rank
// whose mapping failed must not be the only one that leaves the fused path (its peers' kernels would wait for
// flags that never come). `SymmRegion::reopen` therefore runs a fixed protocol of small host-level all-gathers:
//
//   1. agree on the size (maximum over ranks); this exchange is also the point where every rank has drained
//      the stream that used the old mapping
//   2. every rank closes its imports of the old region; exchange; every rank frees its own old allocation
//   3. allocate, export; all-gather {ok, handle}; import every peer
//   4. all-gather the outcome; unless EVERY rank succeeded, every rank unwinds (close imports, meet, free)
//      and returns false, so that all of them take the same fallback
// With a backend that can grow a buffer in place (cuMem VMM) steps 2-3 become "grow, export, all-gather, import the
// new chunks": nothing is unmapped or freed and no pointer changes; if that fails on any rank, all ranks close the
// region and open a fresh one by the steps above.
//
// The reference grows its workspace in place with cuMem VMM and never unmaps
// (src/coccl-extend/core/memory/coccl_buffer_vmm.cc:200-240); a failure there is local because NCCL moves the
// bytes. Here the kernels themselves store into peer memory, which is why the outcome must be agreed.
//
// The CUDA calls and the exchange sit behind two small interfaces so that the protocol runs in host tests
// with several threads as ranks and injected failures.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "symm/symm.h"

namespace coccl {

struct SymmApi {
  int (*alloc)(size_t bytes, cocclSymmBuffer** out);
  int (*exportHandle)(const cocclSymmBuffer* buf, void* handle);
  int (*importPeer)(cocclSymmBuffer* owner, int peer, const void* handle, void** mapped);
  void* (*localPtr)(const cocclSymmBuffer* buf);
  int (*closeImports)(cocclSymmBuffer* buf);
  int (*free)(cocclSymmBuffer* buf);
  // Optional (null where the backend cannot): make the buffer longer where it is. Peers then import the buffer's new
  // export handle, which maps only what they do not have yet and leaves every pointer as it was.
  int (*grow)(cocclSymmBuffer* buf, size_t bytes);
};
const SymmApi& cudaSymmApi();

// Blocking host-level all-gather of small blobs over the ranks of one communicator.
class HostExchange {
 public:
  virtual ~HostExchange() {}
  virtual int rank() const = 0;
  virtual int nRanks() const = 0;
  // `all` receives nRanks * bytes in rank order. False when the exchange itself failed.
  virtual bool allGather(const void* mine, void* all, size_t bytes) = 0;
};

constexpr int kSymmMaxRanks = 8;

class SymmRegion {
 public:
  // Collective. Replaces the region by one of at least `bytes` bytes on every rank (the maximum over ranks is
  // used). The caller has drained every stream that used the old mapping. True only if every rank succeeded;
  // on false the region is closed on every rank.
  bool reopen(const SymmApi& api, HostExchange& x, size_t bytes);
  // Collective close (imports first, then the allocations).
  void close(const SymmApi& api, HostExchange& x);
  // Local close for teardown paths where the peers cannot be reached any more.
  void closeLocal(const SymmApi& api);

  bool open() const { return buf_ != nullptr; }
  size_t bytes() const { return bytes_; }
  void* ptr(int rank) const { return ptrs_[rank]; }

 private:
  cocclSymmBuffer* buf_ = nullptr;
  void* ptrs_[kSymmMaxRanks] = {};
  size_t bytes_ = 0;
};

}  // namespace coccl
