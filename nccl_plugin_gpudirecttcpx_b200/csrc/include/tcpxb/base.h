// Result codes, logging and checking helpers shared by the host core.
//
// Plays the role of the reference's adapter layer (reference: src/adapter/ret.h:22-29,
// src/adapter/debug1.h:39-47, src/misc/checks1.h:25-80): result values are
// numerically NCCL's, so the plugin table can return them unchanged, and log lines
// go to the logger NCCL passes to init() or, outside NCCL, to stderr.  Unlike the
// reference, no helper here ever calls exit(): failures travel as return codes.
#ifndef TCPXB_BASE_H_
#define TCPXB_BASE_H_

#include <errno.h>
#include <stdarg.h>
#include <stdint.h>
#include <string.h>

namespace tcpxb {

enum Result : int {
  kSuccess = 0,
  kUnhandledCudaError = 1,
  kSystemError = 2,
  kInternalError = 3,
  kInvalidArgument = 4,
  kInvalidUsage = 5,
  kRemoteError = 6,
  kInProgress = 7,
};
const char* resultString(Result r);

// NCCL's ncclDebugLogLevel and the subsystem bits the plugin uses.
enum LogLevel : int { kLogNone = 0, kLogVersion = 1, kLogWarn = 2, kLogInfo = 3, kLogAbort = 4, kLogTrace = 5 };
enum LogSubsys : unsigned long { kSubInit = 1, kSubNet = 16, kSubEnv = 128 };

using LoggerFn = void (*)(int level, unsigned long flags, const char* file, int line,
                          const char* fmt, ...);
// Installs NCCL's logger (nullptr restores the stderr logger).
void setLogger(LoggerFn fn);
LoggerFn logger();
// Stand-alone stderr logger level: TCPXB_DEBUG or NCCL_DEBUG = WARN | INFO | TRACE.
int standaloneLogLevel();

}  // namespace tcpxb

#define TCPXB_LOG(level, subsys, ...) \
  (::tcpxb::logger())((level), (subsys), __FILE__, __LINE__, __VA_ARGS__)
#define WARN(...) TCPXB_LOG(::tcpxb::kLogWarn, ~0ul, __VA_ARGS__)
#define INFO(subsys, ...) TCPXB_LOG(::tcpxb::kLogInfo, (subsys), __VA_ARGS__)
#define TRACE(subsys, ...) TCPXB_LOG(::tcpxb::kLogTrace, (subsys), __VA_ARGS__)

#define TCPXB_CHECK(expr)                                          \
  do {                                                             \
    ::tcpxb::Result r_ = (expr);                                   \
    if (r_ != ::tcpxb::kSuccess && r_ != ::tcpxb::kInProgress) {   \
      INFO(::tcpxb::kSubNet, "%s:%d -> %d", __FILE__, __LINE__, (int)r_); \
      return r_;                                                   \
    }                                                              \
  } while (0)

// Retries on EINTR; any other failure is logged and returned as a system error.
#define TCPXB_SYSCHECK(call, name)                                 \
  do {                                                             \
    long rc_;                                                      \
    do { rc_ = (long)(call); } while (rc_ == -1 && errno == EINTR);\
    if (rc_ == -1) {                                               \
      WARN("call to " name " failed: %s", strerror(errno));        \
      return ::tcpxb::kSystemError;                                \
    }                                                              \
  } while (0)

#endif  // TCPXB_BASE_H_
