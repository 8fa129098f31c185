// Group batching (ncclGroupStart/End semantics for compressed calls).
// Behavioural model: src/coccl-extend/core/runtime/coccl_group.cc:12-71 and the hooks in
// src/group.cc:103-116: calls issued inside a group are deferred; at group end the whole batch
// is replayed natively if the transport has native work pending in the same group, if any
// deferred entry is native, or if send/recv is mixed with collectives; otherwise the transport
// group is flushed first and the compressed calls run afterwards, send/recv as ONE batch and
// collectives one by one.
#include "runtime/log.h"
#include "runtime/runtime.h"

namespace coccl {

namespace {
struct PendingEntry {
  bool native = false;
  CallInfo info;
  PreparedCall prepared;
};
struct GroupState {
  int depth = 0;
  std::vector<PendingEntry> pending;
};
thread_local GroupState tlsGroup;
}  // namespace

void Runtime::groupStart() { ++tlsGroup.depth; }
int Runtime::groupDepth() const { return tlsGroup.depth; }
bool Runtime::groupHasPending() const { return !tlsGroup.pending.empty(); }

void Runtime::groupEnqueuePrepared(const PreparedCall& call) {
  PendingEntry e;
  e.native = false;
  e.info = call.info;
  e.prepared = call;
  tlsGroup.pending.push_back(e);
  ++stats_.deferredCalls;
}

void Runtime::groupEnqueueNative(const CallInfo& info) {
  PendingEntry e;
  e.native = true;
  e.info = info;
  tlsGroup.pending.push_back(e);
  ++stats_.deferredCalls;
}

// A call that stays native: outside a group (or for collectives) the caller simply proceeds on the
// native path; a grouped send/recv is queued so that its order relative to compressed send/recv of
// the same group is kept.
ncclResult_t Runtime::routeNativeGrouped(const CallInfo& info, bool* enqueued) {
  if (tlsGroup.depth == 0 || info.op != Operation::SendRecv) return ncclSuccess;
  groupEnqueueNative(info);
  *enqueued = true;
  return ncclSuccess;
}

ncclResult_t Runtime::groupPrepareEnd(Transport*, bool nativePending) {
  std::vector<PendingEntry>& q = tlsGroup.pending;
  if (q.empty()) return ncclSuccess;
  bool anyNative = nativePending, anyP2p = false, anyColl = false;
  for (const PendingEntry& e : q) {
    anyNative = anyNative || e.native;
    if (e.info.op == Operation::SendRecv) anyP2p = true; else anyColl = true;
  }
  if (!(anyNative || (anyP2p && anyColl))) return ncclSuccess;
  // replay everything natively, in issue order, inside the transport's still open group
  std::vector<PendingEntry> batch;
  batch.swap(q);
  ncclResult_t first = ncclSuccess;
  for (const PendingEntry& e : batch) {
    ncclResult_t r = replayNative(e.info);
    if (first == ncclSuccess) first = r;
  }
  return first;
}

ncclResult_t Runtime::groupDrain() {
  std::vector<PendingEntry> batch;
  batch.swap(tlsGroup.pending);
  if (batch.empty()) return ncclSuccess;
  if (executor_ == nullptr) return ncclInvalidArgument;
  std::vector<PreparedCall> p2p;
  ncclResult_t first = ncclSuccess;
  for (const PendingEntry& e : batch) {
    if (e.info.op == Operation::SendRecv) { p2p.push_back(e.prepared); continue; }
    ncclResult_t r = executePrepared(e.prepared);
    if (first == ncclSuccess) first = r;
  }
  if (!p2p.empty()) {
    struct Guard { bool prev; Guard() : prev(Runtime::internalCall()) {} } g;
    (void)g;
    stats_.compressedCalls += p2p.size();
    ncclResult_t r = executor_->executeSendRecvBatch(this, p2p);
    if (first == ncclSuccess) first = r;
  }
  return first;
}

void Runtime::groupAbort() { tlsGroup.pending.clear(); }

ncclResult_t Runtime::groupEnd(Transport* t, bool nativePending) {
  if (tlsGroup.depth <= 0) return ncclInvalidUsage;
  if (--tlsGroup.depth > 0) return t ? t->groupEnd() : ncclSuccess;
  ncclResult_t r = groupPrepareEnd(t, nativePending);
  ncclResult_t g = t ? t->groupEnd() : ncclSuccess;
  if (r != ncclSuccess || g != ncclSuccess) {
    groupAbort();
    return r != ncclSuccess ? r : g;
  }
  return groupDrain();
}

}  // namespace coccl
