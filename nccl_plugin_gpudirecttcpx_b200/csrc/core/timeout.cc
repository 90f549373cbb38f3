#include "tcpxb/timeout.h"

#include <time.h>

namespace tcpxb {

uint64_t monotonicNanos() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

bool StallDetector::shouldWarn(uint64_t* stalled_ns) {
  const uint64_t now = clock_();
  if (polls_++ == 0) {
    start_ = now;
    return false;
  }
  const uint64_t stalled = now - start_;
  if (stalled_ns != nullptr) *stalled_ns = stalled;
  if (!warned_) {
    if (stalled < threshold_) return false;
    warned_ = true;
    last_warn_ = now;
    return true;
  }
  if (now - last_warn_ < frequency_) return false;
  last_warn_ = now;
  return true;
}

}  // namespace tcpxb
