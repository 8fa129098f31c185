#include "runtime/log.h"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
#include <mutex>
#include <string>

namespace coccl {
namespace {
struct LogState {
  LogLevel level = kLevelWarn;
  uint32_t mask = kLogInit;
  FILE* out = stderr;
};
LogState* state() {
  static LogState* s = [] {
    LogState* st = new LogState();
    const char* lv = getenv("COCCL_DEBUG");
    if (lv == nullptr) lv = getenv("NCCL_DEBUG");
    if (lv != nullptr) {
      if (!strcasecmp(lv, "INFO")) st->level = kLevelInfo;
      else if (!strcasecmp(lv, "TRACE")) st->level = kLevelTrace;
      else if (!strcasecmp(lv, "WARN")) st->level = kLevelWarn;
      else if (!strcasecmp(lv, "NONE") || !strcasecmp(lv, "VERSION")) st->level = kLevelNone;
    }
    const char* sub = getenv("COCCL_DEBUG_SUBSYS");
    if (sub != nullptr) {
      st->mask = 0;
      std::string s2(sub);
      size_t pos = 0;
      while (pos <= s2.size()) {
        size_t c = s2.find(',', pos);
        std::string tok = s2.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
        if (tok.rfind("COCCL_", 0) == 0) tok = tok.substr(6);
        if (tok == "INIT") st->mask |= kLogInit;
        else if (tok == "RUNTIME") st->mask |= kLogRuntime;
        else if (tok == "PIPELINE") st->mask |= kLogPipeline;
        else if (tok == "COMPRESS") st->mask |= kLogCompress;
        else if (tok == "MEMORY") st->mask |= kLogMemory;
        else if (tok == "TUNING") st->mask |= kLogTuning;
        else if (tok == "ALL" || tok == "COCCL") st->mask |= kLogAll;
        if (c == std::string::npos) break;
        pos = c + 1;
      }
    }
    const char* file = getenv("COCCL_DEBUG_FILE");
    if (file != nullptr && *file) {
      FILE* f = fopen(file, "a");
      if (f) st->out = f;
    }
    return st;
  }();
  return s;
}
thread_local char tlsWarn[512] = "";
std::mutex gLogMutex;
}  // namespace

bool logEnabled(LogLevel level, uint32_t subsys) {
  LogState* s = state();
  return level <= s->level && (level <= kLevelWarn || (s->mask & subsys) != 0);
}

const char* lastWarning() { return tlsWarn; }

void logMessage(LogLevel level, uint32_t subsys, const char* file, int line, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (level == kLevelWarn) snprintf(tlsWarn, sizeof(tlsWarn), "%s", buf);
  if (!logEnabled(level, subsys)) return;
  LogState* s = state();
  const char* base = strrchr(file, '/');
  std::lock_guard<std::mutex> lock(gLogMutex);
  fprintf(s->out, "[%d] COCCL %s %s:%d %s\n", (int)getpid(), level == kLevelWarn ? "WARN" : (level == kLevelInfo ? "INFO" : "TRACE"),
          base ? base + 1 : file, line, buf);
  fflush(s->out);
}
}  // namespace coccl
