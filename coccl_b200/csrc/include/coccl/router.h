// Routing sessions: the policy file, the plugin catalogue and the router of the host runtime, usable without an
// NCCL communicator. The framework layer (one process per GPU under torch.distributed, which owns its own
// communicators and launches the fused kernels itself) asks a session, for every collective, what the C API would
// do with the same call: native or compressed, which algorithm, which codec. Both front ends therefore follow ONE
// implementation of the rules of src/coccl-extend/core/runtime/coccl_runtime.cc:181-229 (Runtime::enqueueCheck),
// of the policy model (TOML, scopes, thresholds) and of the algorithm selector.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "kernels/kernels_api.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cocclRouter cocclRouter;

enum { COCCL_ROLE_NORMAL = 0, COCCL_ROLE_DP = 1, COCCL_ROLE_TP = 2, COCCL_ROLE_PP = 3 };
enum { COCCL_OP_ALL_GATHER = 0, COCCL_OP_REDUCE_SCATTER = 1, COCCL_OP_ALL_REDUCE = 2, COCCL_OP_ALL_TO_ALL = 3, COCCL_OP_SEND_RECV = 4 };
// algorithm of a decision (coccl::Algorithm)
enum { COCCL_ALGO_NONE = 0, COCCL_ALGO_RS_ONESHOT = 1, COCCL_ALGO_RS_TWOSHOT = 2, COCCL_ALGO_AR_ONESHOT = 3,
       COCCL_ALGO_AR_TWOSHOT = 4, COCCL_ALGO_AR_TRIPLESHOT = 5 };
// variant of an uncompressed small all-reduce chosen from measurements
enum { COCCL_NATIVE_NCCL = 0, COCCL_NATIVE_NVLS = 1 };

typedef struct {
  int compressed;          // 0: run natively (see nativeVariant); 1: run compressed
  int algorithm;           // COCCL_ALGO_*
  int fusable;             // the codec is one of the library's tile codecs for this datatype: `codec` is valid
  int delta;               // the codec sends changes against the previous result (sdp4bit subAdd)
  int nativeVariant;       // COCCL_NATIVE_* (all-reduce below the threshold only)
  int role;                // coccl::Role the call was routed under
  size_t thresholdBytes;   // threshold that applied
  size_t totalBytes;       // logical bytes the router compared with it
  cocclkCodec codec;
  char compressor[32];     // plugin name, "" when native
} cocclRouteDecision;

// configPath == NULL: a disabled session (everything native). The file is parsed with the rules of the C API's
// COCCL_CONFIG_FILE; `nodes` x `devicesPerNode` is the topology handed to the plugins' parseConfig. Returns 0 or an
// ncclResult_t; on failure `error` (may be NULL) receives the reason.
int cocclRouterOpen(const char* configPath, int nodes, int devicesPerNode, cocclRouter** out, char* error, size_t errorCap);
void cocclRouterClose(cocclRouter* r);
// Flat "key = value" text of the effective configuration (owned by the session) and a 64-bit FNV-1a hash of it.
const char* cocclRouterEffectiveConfig(cocclRouter* r);
uint64_t cocclRouterConfigHash(cocclRouter* r);
int cocclRouterEnabled(cocclRouter* r);
// [runtime] fused_kernel_max_ctas of the policy (0 = no limit).
int cocclRouterFusedMaxCtas(cocclRouter* r);
int cocclRouterTrainingMode(cocclRouter* r);

// What happens to a collective of `count` elements (the count of the matching nccl* call) on a communicator of
// nRanks ranks over nNodes nodes. redOp: ncclRedOp_t. explicitAlgorithm: -1 for an implicit call, else COCCL_ALGO_*
// of an explicit coccl*Comp* call (which ignores the threshold). Returns 0 or an ncclResult_t.
int cocclRouterDecide(cocclRouter* r, int role, int op, int ncclDatatype, size_t count, int nRanks, int nNodes, int rank,
                      int redOp, int explicitAlgorithm, cocclRouteDecision* out);

// Measured preferences, filled by whoever timed the kernels that actually serve the calls (the framework layer
// times one-shot, two-shot and the multimem kernel per size at communicator start-up; max over ranks). The selector
// consults them before its cost model when autotune is enabled and no algorithm is forced. `log2Bytes` is the
// bucket floor(log2(count * size)); buckets without an entry use the nearest measured one below, else above.
int cocclRouterSetMeasured(cocclRouter* r, int op, int ncclDatatype, int nRanks, int log2Bytes, int algorithm, double seconds);
int cocclRouterSetMeasuredNative(cocclRouter* r, int ncclDatatype, int nRanks, int log2Bytes, int nativeVariant, double seconds);
// Router counters of the session: calls decided native / compressed, policy lookups.
void cocclRouterStats(cocclRouter* r, uint64_t* nativeCalls, uint64_t* compressedCalls, uint64_t* policyLookups);

#ifdef __cplusplus
}
#endif
