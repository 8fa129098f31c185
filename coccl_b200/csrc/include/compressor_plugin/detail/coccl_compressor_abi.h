// Binary contract between the runtime and a compressor shared library (ABI v8, host API v3).
// A plugin is one `lib<name>.so` exporting `cocclGetCompressorPlugin`, which returns a
// descriptor of plain-old-data structures; nothing else crosses the boundary. The layouts
// are the wire-level contract of the reference SDK
// (src/coccl-extend/include/compressor_plugin/detail/coccl_compressor_abi.h:13-201) and are
// kept field for field so that a codec built against either header loads in either runtime.
#ifndef COCCL_COMPRESSOR_ABI_H_
#define COCCL_COMPRESSOR_ABI_H_

#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "coccl/nccl_compat.h"

constexpr uint32_t COCCL_COMPRESSOR_ABI_VERSION = 8;
constexpr uint32_t COCCL_COMPRESSOR_HOST_API_VERSION = 3;
constexpr const char* COCCL_COMPRESSOR_ENTRY_SYMBOL = "cocclGetCompressorPlugin";

// What the runtime may ask a codec to do.
enum cocclCompressorOperation : uint32_t {
  cocclCompressorOperationCompress = 0,
  cocclCompressorOperationDecompress,
  cocclCompressorOperationDecompressReduce,          // sum `reduceChunks` encoded copies while decoding
  cocclCompressorOperationDecompressReduceCompress,  // ... and re-encode the sum
};

// Encoded streams travel typed ncclInt8; ncclUint8 marks bytes that were copied through
// unchanged because encoding would have made them larger.
constexpr ncclDataType_t COCCL_COMPRESSOR_RAW_PASSTHROUGH = ncclUint8;

enum cocclCompressorCapability : uint64_t {
  cocclCompressorCapabilityCompress = 1ULL << 0,
  cocclCompressorCapabilityDecompress = 1ULL << 1,
  cocclCompressorCapabilityDecompressReduce = 1ULL << 2,
  cocclCompressorCapabilityDecompressReduceCompress = 1ULL << 3,
  cocclCompressorCapabilityFramed = 1ULL << 4,                    // variable-length frames + metadata
  cocclCompressorCapabilityFusedHierarchicalSwizzle = 1ULL << 5,  // compress applies the rank swizzle itself
  cocclCompressorCapabilityBytewiseLossless = 1ULL << 6,          // any datatype may be routed through it
  // extension of this runtime (bits the reference does not define are ignored by it):
  cocclCompressorCapabilitySeesPassthrough = 1ULL << 7,           // decompress wants raw pass-through inputs too
};
constexpr uint64_t COCCL_COMPRESSOR_REQUIRED_CAPABILITIES =
    cocclCompressorCapabilityCompress | cocclCompressorCapabilityDecompress;

enum cocclCompressorConfigVariant : uint32_t { cocclCompressorConfigDefault = 0, cocclCompressorConfigHierarchical = 1 };

struct cocclConfigPair { const char* key; const char* value; };
struct cocclConfigView { const cocclConfigPair* pairs; size_t count; };
struct cocclCompressorConfigContext { cocclCompressorConfigVariant variant; int nodes; int devicesPerNode; };

enum cocclCompressorFrameEncoding : uint32_t { cocclCompressorFrameEncoded = 0, cocclCompressorFrameRaw = 1 };

// Per-frame header of framed codecs; also the wire header of compressed Send/Recv.
struct cocclCompressorFrameMetadata {
  uint64_t payloadBytes;
  uint32_t encoding;
  uint32_t reserved;
};
static_assert(sizeof(cocclCompressorFrameMetadata) == 16, "frame metadata is a 16-byte wire contract");

// One buffer as seen by a codec; inputs have capacityBytes == bytes.
struct cocclCompressorView {
  void* data;
  size_t capacityBytes;
  size_t bytes;
  size_t elements;
  size_t chunks;
  ncclDataType_t datatype;
  cocclCompressorFrameMetadata* frameMetadata;
  size_t frameStrideBytes;
};

struct cocclCompressorBufferView { void* data; size_t bytes; };

using cocclCompressorCreateStateFn = ncclResult_t (*)(void** state);
using cocclCompressorDestroyStateFn = void (*)(void* state);

// Services the runtime offers a codec while it executes (codecs never allocate on their own).
struct cocclCompressorHostApi {
  uint32_t abiVersion;
  uint32_t structSize;
  ncclResult_t (*allocateScratch)(void* context, size_t bytes, cocclCompressorBufferView* buffer);
  ncclResult_t (*acquirePersistent)(void* context, size_t slot, size_t bytes, cocclCompressorBufferView* buffer);
  ncclResult_t (*getOrCreateState)(void* context, const void* typeKey, cocclCompressorCreateStateFn createState,
                                   cocclCompressorDestroyStateFn destroyState, void** state);
};

struct cocclCompressorExecutionContext {
  uint32_t structSize;
  const cocclCompressorHostApi* hostApi;
  void* hostContext;
  cudaStream_t stream;
  int cudaDev;
  int rank;
  int nRanks;
  int nodes;
  int devicesPerNode;
};

struct cocclCompressorCall {
  uint32_t structSize;
  cocclCompressorOperation operation;
  cocclCompressorView input;
  cocclCompressorView* output;
  int rank;
  size_t reduceChunks;
  ncclDataType_t originalDatatype;
  size_t originalElements;
  const void* config;
  cocclCompressorExecutionContext* execution;
};

// Host-only question asked while planning workspaces: an upper bound of the encoded size of
// a raw shape. Must not launch work or take resources.
struct cocclCompressorSizeQuery {
  uint32_t structSize;
  cocclCompressorOperation operation;
  size_t elements;
  size_t chunks;
  ncclDataType_t datatype;
  const void* config;
};

struct cocclCompressorPlugin {
  uint32_t abiVersion;
  uint32_t structSize;
  const char* name;
  uint64_t capabilities;
  ncclResult_t (*execute)(cocclCompressorCall* call);
  ncclResult_t (*parseConfig)(const cocclConfigView* values, const cocclCompressorConfigContext* context,
                              void** config, char* error, size_t errorCapacity);
  void (*destroyConfig)(void* config);
  ncclResult_t (*getEncodedSizeBound)(const cocclCompressorSizeQuery* query, size_t* encodedBytes);
};

using cocclGetCompressorPluginFn = const cocclCompressorPlugin* (*)();

// Checks a freshly loaded descriptor; on failure writes the reason to `error`.
inline bool cocclValidateCompressorPlugin(const char* expectedName, const cocclCompressorPlugin* plugin, char* error,
                                          size_t errorCapacity) {
  auto say = [&](const char* why) {
    if (error != nullptr && errorCapacity != 0) snprintf(error, errorCapacity, "%s", why);
    return false;
  };
  if (plugin == nullptr) return say("entry returned a null descriptor");
  if (plugin->abiVersion != COCCL_COMPRESSOR_ABI_VERSION) {
    if (error != nullptr && errorCapacity != 0)
      snprintf(error, errorCapacity, "compressor ABI v%u is unsupported; runtime requires v%u", plugin->abiVersion,
               COCCL_COMPRESSOR_ABI_VERSION);
    return false;
  }
  if (plugin->structSize != sizeof(cocclCompressorPlugin)) return say("compressor descriptor size mismatch");
  if (plugin->name == nullptr || expectedName == nullptr || strcmp(plugin->name, expectedName) != 0)
    return say("compressor descriptor name mismatch");
  if ((plugin->capabilities & COCCL_COMPRESSOR_REQUIRED_CAPABILITIES) != COCCL_COMPRESSOR_REQUIRED_CAPABILITIES)
    return say("compressor is missing compress or decompress capability");
  if (plugin->execute == nullptr || plugin->parseConfig == nullptr || plugin->destroyConfig == nullptr)
    return say("compressor descriptor is missing a required callback");
  return true;
}

#endif  // COCCL_COMPRESSOR_ABI_H_
