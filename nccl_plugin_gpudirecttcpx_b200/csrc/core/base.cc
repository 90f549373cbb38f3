#include "tcpxb/base.h"

#include <atomic>
#include <stdio.h>
#include <stdlib.h>
#include <strings.h>
#include <unistd.h>

namespace tcpxb {

const char* resultString(Result r) {
  switch (r) {
    case kSuccess: return "success";
    case kUnhandledCudaError: return "unhandled cuda error";
    case kSystemError: return "system error";
    case kInternalError: return "internal error";
    case kInvalidArgument: return "invalid argument";
    case kInvalidUsage: return "invalid usage";
    case kRemoteError: return "remote error";
    case kInProgress: return "in progress";
  }
  return "unknown";
}

int standaloneLogLevel() {
  static const int level = [] {
    const char* v = getenv("TCPXB_DEBUG");
    if (v == nullptr) v = getenv("NCCL_DEBUG");
    if (v == nullptr) return (int)kLogWarn;
    if (!strcasecmp(v, "TRACE")) return (int)kLogTrace;
    if (!strcasecmp(v, "INFO")) return (int)kLogInfo;
    if (!strcasecmp(v, "VERSION")) return (int)kLogVersion;
    if (!strcasecmp(v, "NONE")) return (int)kLogNone;
    return (int)kLogWarn;
  }();
  return level;
}

namespace {
void stderrLogger(int level, unsigned long /*flags*/, const char* file, int line, const char* fmt, ...) {
  const int max = standaloneLogLevel();
  if (level == kLogTrace ? max < kLogTrace : (level > max && level != kLogAbort)) return;
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  const char* base = strrchr(file, '/');
  fprintf(stderr, "[tcpxb %d] %s %s:%d %s\n", (int)getpid(),
          level == kLogWarn ? "WARN" : level == kLogTrace ? "TRACE" : "INFO", base ? base + 1 : file,
          line, buf);
}
std::atomic<LoggerFn> g_logger{stderrLogger};
}  // namespace

void setLogger(LoggerFn fn) { g_logger.store(fn ? fn : stderrLogger, std::memory_order_release); }
LoggerFn logger() { return g_logger.load(std::memory_order_acquire); }

}  // namespace tcpxb
