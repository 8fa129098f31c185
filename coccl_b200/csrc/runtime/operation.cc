#include "coccl/operation.h"

namespace coccl {

static const OperationDescriptor kTable[] = {
    {Operation::AllGather, "all_gather", kTraitScaleBytesByRanks | kTraitGrouped},
    {Operation::ReduceScatter, "reduce_scatter", kTraitScaleBytesByRanks | kTraitReduction | kTraitGrouped | kTraitHierarchicalPolicy},
    {Operation::AllReduce, "all_reduce", kTraitReduction | kTraitGrouped | kTraitCountDivisibleByRanks | kTraitHierarchicalPolicy},
    {Operation::AllToAll, "all_to_all", kTraitScaleBytesByRanks | kTraitGrouped},
    {Operation::SendRecv, "sendrecv", kTraitGrouped | kTraitDirectionalPolicy},
};

const OperationDescriptor* describe(Operation op) {
  const unsigned i = static_cast<unsigned>(op);
  return i < static_cast<unsigned>(Operation::Count) ? &kTable[i] : nullptr;
}

bool supportsVariant(const OperationDescriptor* d, Variant v) {
  if (d == nullptr) return false;
  if (v == Variant::Default) return true;
  return d->has(kTraitDirectionalPolicy);
}

const char* scopeName(Scope s) {
  switch (s) {
    case Scope::Default: return "default";
    case Scope::Intra: return "intra";
    case Scope::Inter: return "inter";
    default: return "?";
  }
}

}  // namespace coccl
