// Collective open / regrow / close of a peer-mapped region (runtime/symm_workspace.h), run with one thread per
// rank, an in-memory exchange and a fake of the CUDA symmetric-memory calls that logs what happens in which
// order and fails on demand.
#include <condition_variable>
#include <mutex>
#include <string.h>
#include <atomic>
#include <thread>

#include "host_test.h"
#include "runtime/symm_workspace.h"

using namespace coccl;

// the production struct is opaque to the protocol; the fakes use their own definition
struct cocclSymmBuffer {
  int rank = 0;
  size_t bytes = 0;
  bool mapped[8] = {};
};

namespace {

constexpr int kRanks = 4;

struct World {
  std::mutex m;
  std::condition_variable cv;
  int arrived = 0;
  long generation = 0;
  int copyOut_ = 0;
  std::vector<char> slots;
  // fake CUDA state
  int liveImportsOf[kRanks] = {};   // how many peers currently map rank r's allocation
  int freedWhileMapped = 0;        // the undefined behaviour the protocol must never produce
  int failImportOnRank = -1, failAllocOnRank = -1;
  int allocs = 0, frees = 0;
};
World* gWorld = nullptr;
thread_local int tRank = 0;

class ThreadExchange : public HostExchange {
 public:
  explicit ThreadExchange(int r) : r_(r) {}
  int rank() const override { return r_; }
  int nRanks() const override { return kRanks; }
  bool allGather(const void* mine, void* all, size_t bytes) override {
    World& w = *gWorld;
    std::unique_lock<std::mutex> lk(w.m);
    if (w.slots.size() < bytes * kRanks) w.slots.resize(bytes * kRanks);
    memcpy(w.slots.data() + (size_t)r_ * bytes, mine, bytes);
    const long gen = w.generation;
    if (++w.arrived == kRanks) {
      // last arrival: everyone copies out before the next round may overwrite
      w.copyOut_ = 0;
      ++w.generation;
      w.arrived = 0;
      w.cv.notify_all();
    } else {
      w.cv.wait(lk, [&] { return w.generation != gen; });
    }
    memcpy(all, w.slots.data(), bytes * kRanks);
    // second phase so that a fast rank cannot start the next round while a slow one still reads
    const long gen2 = w.generation;
    if (++w.copyOut_ == kRanks) { ++w.generation; w.cv.notify_all(); }
    else w.cv.wait(lk, [&] { return w.generation != gen2; });
    return true;
  }
 private:
  int r_;
};

int fAlloc(size_t bytes, cocclSymmBuffer** out) {
  World& w = *gWorld;
  std::lock_guard<std::mutex> lk(w.m);
  if (w.failAllocOnRank == tRank) return 2;
  cocclSymmBuffer* b = new cocclSymmBuffer();
  b->rank = tRank;
  b->bytes = bytes;
  ++w.allocs;
  *out = b;
  return 0;
}
int fExport(const cocclSymmBuffer* b, void* h) { memset(h, 0, COCCL_SYMM_HANDLE_BYTES); memcpy(h, &b->rank, sizeof(int)); return 0; }
int fImport(cocclSymmBuffer* owner, int peer, const void* h, void** mapped) {
  World& w = *gWorld;
  std::lock_guard<std::mutex> lk(w.m);
  int src = -1;
  memcpy(&src, h, sizeof(int));
  if (src != peer) return 1;
  if (w.failImportOnRank == tRank && peer == (tRank + 1) % kRanks) return 1;
  ++w.liveImportsOf[peer];
  owner->mapped[peer] = true;
  *mapped = reinterpret_cast<void*>((uintptr_t)(0x1000 * (peer + 1)));
  return 0;
}
void* fLocal(const cocclSymmBuffer* b) { return reinterpret_cast<void*>((uintptr_t)(0x1000 * (b->rank + 1))); }
int fCloseImports(cocclSymmBuffer* b) {
  World& w = *gWorld;
  std::lock_guard<std::mutex> lk(w.m);
  for (int p = 0; p < kRanks; ++p) {
    if (b->mapped[p]) { --w.liveImportsOf[p]; b->mapped[p] = false; }
  }
  return 0;
}
int fFree(cocclSymmBuffer* b) {
  fCloseImports(b);
  World& w = *gWorld;
  std::lock_guard<std::mutex> lk(w.m);
  if (w.liveImportsOf[b->rank] != 0) ++w.freedWhileMapped;
  ++w.frees;
  delete b;
  return 0;
}
const SymmApi kFakeApi = {&fAlloc, &fExport, &fImport, &fLocal, &fCloseImports, &fFree};

// a backend that grows where it is (the cuMem VMM one): same fake, plus grow
int gFailGrowOnRank = -1;
std::atomic<int> gGrows{0};
int fGrow(cocclSymmBuffer* b, size_t bytes) {
  if (gFailGrowOnRank == tRank) return 3;
  if (bytes > b->bytes) b->bytes = bytes;
  ++gGrows;
  return 0;
}
// importing a peer a second time maps "the new chunks" and must not count as a second live mapping
int fImportAgain(cocclSymmBuffer* owner, int peer, const void* h, void** mapped) {
  if (owner->mapped[peer]) { *mapped = reinterpret_cast<void*>((uintptr_t)(0x1000 * (peer + 1))); return 0; }
  return fImport(owner, peer, h, mapped);
}
const SymmApi kGrowingApi = {&fAlloc, &fExport, &fImportAgain, &fLocal, &fCloseImports, &fFree, &fGrow};

template <class F>
void runRanks(F&& body) {
  std::vector<std::thread> th;
  for (int r = 0; r < kRanks; ++r) th.emplace_back([&, r] { tRank = r; body(r); });
  for (auto& t : th) t.join();
}

}  // namespace

TEST(symm_region_opens_grows_and_closes_in_order) {
  World w;
  gWorld = &w;
  SymmRegion regions[kRanks];
  bool ok1[kRanks], ok2[kRanks];
  runRanks([&](int r) {
    ThreadExchange x(r);
    // ranks ask for different sizes: the maximum is allocated everywhere
    ok1[r] = regions[r].reopen(kFakeApi, x, 1000 + 100 * r);
    ok2[r] = regions[r].reopen(kFakeApi, x, 5000);
  });
  for (int r = 0; r < kRanks; ++r) {
    EXPECT(ok1[r] && ok2[r]);
    EXPECT_EQ(regions[r].bytes(), (size_t)5000);
    for (int p = 0; p < kRanks; ++p) EXPECT(regions[r].ptr(p) == reinterpret_cast<void*>((uintptr_t)(0x1000 * (p + 1))));
  }
  EXPECT_EQ(w.allocs, 2 * kRanks);
  EXPECT_EQ(w.frees, kRanks);          // the first generation was freed by the regrowth
  EXPECT_EQ(w.freedWhileMapped, 0);    // and never while a peer still had it mapped
  runRanks([&](int r) { ThreadExchange x(r); regions[r].close(kFakeApi, x); });
  EXPECT_EQ(w.frees, 2 * kRanks);
  EXPECT_EQ(w.freedWhileMapped, 0);
  for (int r = 0; r < kRanks; ++r) EXPECT_EQ(w.liveImportsOf[r], 0);
}

TEST(symm_region_grows_in_place_where_the_backend_can) {
  World w;
  gWorld = &w;
  gFailGrowOnRank = -1;
  gGrows = 0;
  SymmRegion regions[kRanks];
  bool ok1[kRanks], ok2[kRanks], ok3[kRanks];
  runRanks([&](int r) {
    ThreadExchange x(r);
    ok1[r] = regions[r].reopen(kGrowingApi, x, 1000);
    ok2[r] = regions[r].reopen(kGrowingApi, x, 5000 + r);   // in place: nothing freed, nothing unmapped
  });
  for (int r = 0; r < kRanks; ++r) {
    EXPECT(ok1[r] && ok2[r]);
    EXPECT_EQ(regions[r].bytes(), (size_t)(5000 + kRanks - 1));
  }
  EXPECT_EQ(w.allocs, kRanks);
  EXPECT_EQ(w.frees, 0);
  EXPECT_EQ((int)gGrows, kRanks);
  for (int r = 0; r < kRanks; ++r) EXPECT_EQ(w.liveImportsOf[r], kRanks - 1);
  // one rank cannot grow (its address range is used up): every rank closes and opens a fresh region together
  gFailGrowOnRank = 1;
  runRanks([&](int r) { ThreadExchange x(r); ok3[r] = regions[r].reopen(kGrowingApi, x, 20000); });
  for (int r = 0; r < kRanks; ++r) { EXPECT(ok3[r]); EXPECT_EQ(regions[r].bytes(), (size_t)20000); }
  EXPECT_EQ(w.allocs, 2 * kRanks);
  EXPECT_EQ(w.frees, kRanks);
  EXPECT_EQ(w.freedWhileMapped, 0);
  gFailGrowOnRank = -1;
  runRanks([&](int r) { ThreadExchange x(r); regions[r].close(kGrowingApi, x); });
  for (int r = 0; r < kRanks; ++r) EXPECT_EQ(w.liveImportsOf[r], 0);
}

TEST(symm_region_failure_on_one_rank_is_seen_by_all) {
  for (int mode = 0; mode < 2; ++mode) {
    World w;
    gWorld = &w;
    if (mode == 0) w.failImportOnRank = 2; else w.failAllocOnRank = 1;
    SymmRegion regions[kRanks];
    bool ok[kRanks];
    runRanks([&](int r) { ThreadExchange x(r); ok[r] = regions[r].reopen(kFakeApi, x, 4096); });
    for (int r = 0; r < kRanks; ++r) {
      EXPECT(!ok[r]);               // one rank failed: every rank leaves the fused path together
      EXPECT(!regions[r].open());
    }
    EXPECT_EQ(w.freedWhileMapped, 0);
    EXPECT_EQ(w.allocs, w.frees);
    for (int r = 0; r < kRanks; ++r) EXPECT_EQ(w.liveImportsOf[r], 0);
  }
}
