// Poll-driven stall detector: the caller invokes shouldWarn() each time it polls
// something that made no progress and reset() when progress happens.  The first
// warning comes after `threshold_ns`, later ones every `frequency_ns`.  The clock
// is injectable for tests.  Warn-only by design: it never aborts anything
// (reference: src/timeout.h:26-49, src/timeout.cc:52-75).
#ifndef TCPXB_TIMEOUT_H_
#define TCPXB_TIMEOUT_H_

#include <stdint.h>

namespace tcpxb {

using ClockFn = uint64_t (*)();
uint64_t monotonicNanos();

class StallDetector {
 public:
  void configure(uint64_t threshold_ns, uint64_t frequency_ns, ClockFn clock = nullptr) {
    threshold_ = threshold_ns;
    frequency_ = frequency_ns;
    clock_ = clock ? clock : monotonicNanos;
    reset();
  }
  void reset() { polls_ = 0; start_ = 0; last_warn_ = 0; warned_ = false; }
  // True when a warning is due; *stalled_ns receives the time since the first
  // fruitless poll.
  bool shouldWarn(uint64_t* stalled_ns);
  uint64_t polls() const { return polls_; }

 private:
  uint64_t threshold_ = 10000000000ull, frequency_ = 30000000000ull;
  ClockFn clock_ = monotonicNanos;
  uint64_t polls_ = 0, start_ = 0, last_warn_ = 0;
  bool warned_ = false;
};

}  // namespace tcpxb
#endif  // TCPXB_TIMEOUT_H_
