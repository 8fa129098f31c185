// Logging in the style of the NCCL logger: COCCL_DEBUG=WARN|INFO|TRACE (NCCL_DEBUG is honoured
// too), COCCL_DEBUG_SUBSYS=comma list of INIT,RUNTIME,PIPELINE,COMPRESS,MEMORY,TUNING,ALL.
// Subsystem names follow src/include/nccl_common.h:27-34 / src/debug.cc:88-101; INIT is on by
// default at INFO level (src/debug.cc:19).
#pragma once
#include <stdint.h>

namespace coccl {
enum LogSubsys : uint32_t {
  kLogInit = 1u << 0, kLogRuntime = 1u << 1, kLogPipeline = 1u << 2, kLogCompress = 1u << 3,
  kLogMemory = 1u << 4, kLogTuning = 1u << 5, kLogAll = 0x3f
};
enum LogLevel { kLevelNone = 0, kLevelWarn = 1, kLevelInfo = 2, kLevelTrace = 3 };
void logMessage(LogLevel level, uint32_t subsys, const char* file, int line, const char* fmt, ...)
    __attribute__((format(printf, 5, 6)));
bool logEnabled(LogLevel level, uint32_t subsys);
// Last WARN text of the calling thread (tests and error reporting).
const char* lastWarning();
}  // namespace coccl

#define COCCL_WARN(fmt, ...) ::coccl::logMessage(::coccl::kLevelWarn, ::coccl::kLogAll, __FILE__, __LINE__, fmt, ##__VA_ARGS__)
#define COCCL_INFO(subsys, fmt, ...)                                                              \
  do {                                                                                            \
    if (::coccl::logEnabled(::coccl::kLevelInfo, subsys))                                         \
      ::coccl::logMessage(::coccl::kLevelInfo, subsys, __FILE__, __LINE__, fmt, ##__VA_ARGS__);    \
  } while (0)
#define COCCL_TRACE(subsys, fmt, ...)                                                             \
  do {                                                                                            \
    if (::coccl::logEnabled(::coccl::kLevelTrace, subsys))                                        \
      ::coccl::logMessage(::coccl::kLevelTrace, subsys, __FILE__, __LINE__, fmt, ##__VA_ARGS__);   \
  } while (0)
