// Operation descriptors: the five operations the router knows, their trait bits, and
// the (operation, variant, scope) key that addresses a policy slot.
// Behavioural model: src/coccl-extend/include/runtime/coccl_operation.h:6-104 and the
// trait table in core/runtime/coccl_operation.cc:7-24.
#pragma once
#include <stdint.h>

namespace coccl {

enum class Operation : uint8_t { AllGather = 0, ReduceScatter, AllReduce, AllToAll, SendRecv, Count };
enum class Variant : uint8_t { Default = 0, Forward, Backward };
enum class Scope : uint8_t { Default = 0, Intra, Inter, Count };

enum Trait : uint32_t {
  kTraitScaleBytesByRanks = 1u << 0,      // logical bytes = count * size * nRanks
  kTraitReduction = 1u << 1,              // carries a reduction operator (only sum compresses)
  kTraitGrouped = 1u << 2,                // may be deferred inside group start/end
  kTraitCountDivisibleByRanks = 1u << 3,  // count % nRanks == 0 required to compress
  kTraitHierarchicalPolicy = 1u << 4,     // may use separate intra / inter node codecs
  kTraitDirectionalPolicy = 1u << 5,      // forward / backward variants exist (pipeline p2p)
};

struct PolicyKey {
  Operation op = Operation::Count;
  Variant variant = Variant::Default;
  Scope scope = Scope::Default;
  bool operator==(const PolicyKey& o) const { return op == o.op && variant == o.variant && scope == o.scope; }
  bool operator<(const PolicyKey& o) const {
    if (op != o.op) return op < o.op;
    if (variant != o.variant) return variant < o.variant;
    return scope < o.scope;
  }
  PolicyKey withScope(Scope s) const { PolicyKey k = *this; k.scope = s; return k; }
};

struct OperationDescriptor {
  Operation op;
  const char* name;
  uint32_t traits;
  bool has(Trait t) const { return (traits & t) != 0; }
};

const OperationDescriptor* describe(Operation op);
// Directional variants are only meaningful for operations with kTraitDirectionalPolicy.
bool supportsVariant(const OperationDescriptor* d, Variant v);
const char* scopeName(Scope s);

}  // namespace coccl
