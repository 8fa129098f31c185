#include "runtime/symm_workspace.h"

#include <string.h>
#include <vector>

namespace coccl {

const SymmApi& cudaSymmApi() {
  static const SymmApi api = {&cocclSymmAlloc, &cocclSymmExport, &cocclSymmImport, &cocclSymmLocalPtr,
                              &cocclSymmCloseImports, &cocclSymmFree, &cocclSymmGrow};
  return api;
}

namespace {
struct Offer {
  int64_t ok;
  char handle[COCCL_SYMM_HANDLE_BYTES];
};

// all-gather one integer; returns false if the exchange failed. min/max over ranks come back.
bool agree(HostExchange& x, int64_t mine, int64_t* mn, int64_t* mx) {
  std::vector<int64_t> all((size_t)x.nRanks());
  if (!x.allGather(&mine, all.data(), sizeof(mine))) return false;
  int64_t lo = all[0], hi = all[0];
  for (int64_t v : all) { if (v < lo) lo = v; if (v > hi) hi = v; }
  if (mn) *mn = lo;
  if (mx) *mx = hi;
  return true;
}
}  // namespace

void SymmRegion::closeLocal(const SymmApi& api) {
  if (buf_) api.free(buf_);
  buf_ = nullptr;
  bytes_ = 0;
  memset(ptrs_, 0, sizeof(ptrs_));
}

void SymmRegion::close(const SymmApi& api, HostExchange& x) {
  if (buf_) api.closeImports(buf_);
  int64_t lo = 0;
  agree(x, 1, &lo, nullptr);  // every rank has unmapped its peers
  closeLocal(api);
}

bool SymmRegion::reopen(const SymmApi& api, HostExchange& x, size_t bytes) {
  const int n = x.nRanks(), me = x.rank();
  if (n > kSymmMaxRanks) return false;
  // 1. size agreement; also the rendezvous after which nobody uses the old mapping
  int64_t need = 0;
  if (!agree(x, (int64_t)bytes, nullptr, &need)) { closeLocal(api); return false; }
  // in place, where the backend can: grow, export, exchange, map the new chunks; every rank learns whether all managed
  if (buf_ && api.grow != nullptr) {
    Offer mine;
    memset(&mine, 0, sizeof(mine));
    mine.ok = api.grow(buf_, (size_t)need) == 0 && api.exportHandle(buf_, mine.handle) == 0 ? 1 : 0;
    std::vector<Offer> all((size_t)n);
    bool ok = x.allGather(&mine, all.data(), sizeof(Offer));
    for (int p = 0; ok && p < n; ++p) ok = all[p].ok == 1;
    for (int p = 0; ok && p < n; ++p) {
      if (p == me) continue;
      void* again = nullptr;
      ok = api.importPeer(buf_, p, all[p].handle, &again) == 0 && again == ptrs_[p];
    }
    int64_t everyone = 0;
    if (agree(x, ok ? 1 : 0, &everyone, nullptr) && everyone == 1) {
      bytes_ = (size_t)need;
      return true;
    }
    // some rank could not (IPC-backed buffer, address range exhausted, ...): all ranks start over below
  }
  // 2. old region: imports first, allocations after everybody has unmapped
  if (buf_) api.closeImports(buf_);
  if (!agree(x, 1, nullptr, nullptr)) { closeLocal(api); return false; }
  closeLocal(api);
  // 3. allocate, export, exchange, import
  Offer mine;
  memset(&mine, 0, sizeof(mine));
  mine.ok = api.alloc((size_t)need, &buf_) == 0 && api.exportHandle(buf_, mine.handle) == 0 ? 1 : 0;
  std::vector<Offer> all((size_t)n);
  bool ok = x.allGather(&mine, all.data(), sizeof(Offer));
  for (int p = 0; ok && p < n; ++p) ok = all[p].ok == 1;
  if (ok) {
    for (int p = 0; p < n && ok; ++p) {
      if (p == me) { ptrs_[p] = api.localPtr(buf_); continue; }
      ok = api.importPeer(buf_, p, all[p].handle, &ptrs_[p]) == 0;
    }
  }
  // 4. one outcome for all ranks
  int64_t everyone = 0;
  const bool exchanged = agree(x, ok ? 1 : 0, &everyone, nullptr);
  if (exchanged && everyone == 1) {
    bytes_ = (size_t)need;
    return true;
  }
  if (buf_) api.closeImports(buf_);
  if (exchanged) agree(x, 1, nullptr, nullptr);
  closeLocal(api);
  return false;
}

}  // namespace coccl
