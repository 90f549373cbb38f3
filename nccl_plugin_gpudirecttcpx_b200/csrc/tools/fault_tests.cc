// Failure-path tests of the transport, host only: every failure is made on the host
// (a closed peer, a socket shut down in mid-message, a forged control record, a
// full ring, a silent sender) and every wait in the test is bounded.
// Usage: tcpxb_fault_tests [name-substring]
//
// The reference turns most of these situations into exit(1) or an endless poll
// (reference: src/sock/tcpx.h:186-281 exits on cmsg anomalies; a helper thread that
// hits a socket error just returns, src/net_tcpx.cc:329,350, and the proxy then
// polls forever).  Here they must surface as error codes from test().
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <functional>
#include <string>
#include <vector>

#include "tcpxb/transport.h"

using namespace tcpxb;

namespace {

int g_failures = 0;
bool g_ok = true;
#define EXPECT(cond)                                                         \
  do {                                                                       \
    if (!(cond)) {                                                           \
      fprintf(stderr, "  %s:%d expectation failed: %s\n", __FILE__, __LINE__, #cond); \
      g_ok = false;                                                          \
    }                                                                        \
  } while (0)

struct Test { const char* name; std::function<void()> fn; };
std::vector<Test>& tests() { static std::vector<Test> t; return t; }
struct Reg { Reg(const char* n, std::function<void()> f) { tests().push_back({n, f}); } };
#define TEST(name) void test_##name(); Reg reg_##name(#name, test_##name); void test_##name()

std::atomic<int> g_warns_ctrl{0}, g_warns_stall{0};
void countingLogger(int level, unsigned long, const char*, int, const char* fmt, ...) {
  if (level != kLogWarn) return;
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (strstr(buf, "no control record")) ++g_warns_ctrl;
  if (strstr(buf, "stalled")) ++g_warns_stall;
}

struct Pair {
  ListenComm* l = nullptr;
  Comm* s = nullptr;
  Comm* r = nullptr;
};

bool makePair(Pair* p) {
  char handle[kHandleMaxSize];
  if (netListen(0, handle, &p->l) != kSuccess) return false;
  const uint64_t deadline = monotonicNanos() + 10ull * 1000000000ull;
  while ((p->s == nullptr || p->r == nullptr) && monotonicNanos() < deadline) {
    if (p->s == nullptr && netConnect(0, handle, &p->s) != kSuccess) return false;
    if (p->r == nullptr && netAccept(p->l, &p->r) != kSuccess) return false;
  }
  return p->s != nullptr && p->r != nullptr;
}

void closePair(Pair* p) {
  if (p->s) netClose(p->s);
  if (p->r) netClose(p->r);
  if (p->l) netCloseListen(p->l);
  *p = Pair();
}

// A request must not be tested again once test() reported it done, so completions
// seen while polling "the other side" are remembered here.
struct Seen { Request* req; int size; };
std::vector<Seen> g_seen;

// Polls `req` until done, error or 5 s; returns the Result, *done tells which.
Result pollBounded(Request* req, int* done, int* size, Request* other = nullptr) {
  const uint64_t deadline = monotonicNanos() + 5ull * 1000000000ull;
  *done = 0;
  for (size_t i = 0; i < g_seen.size(); ++i) {
    if (g_seen[i].req == req) {
      *done = 1;
      *size = g_seen[i].size;
      g_seen.erase(g_seen.begin() + (long)i);
      return kSuccess;
    }
  }
  bool other_done = false;
  while (monotonicNanos() < deadline) {
    Result r = netTest(req, done, size);
    if (r != kSuccess || *done) return r;
    if (other != nullptr && !other_done) {
      int d2 = 0, s2 = 0;
      if (netTest(other, &d2, &s2) == kSuccess && d2) {
        g_seen.push_back({other, s2});
        other_done = true;
      }
    }
  }
  return kInProgress;  // never finished within the bound: the test treats this as a hang
}

TEST(round_trip_sanity) {
  Pair p;
  EXPECT(makePair(&p));
  std::vector<uint8_t> src(3000000), dst(3000000, 0);
  for (size_t i = 0; i < src.size(); ++i) src[i] = (uint8_t)(i * 7 + 1);
  Request *rs = nullptr, *rr = nullptr;
  void* data = dst.data();
  int sz = (int)dst.size(), tag = 0;
  EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, nullptr, &rr) == kSuccess && rr != nullptr);
  EXPECT(netIsend(p.s, src.data(), (int)src.size(), 0, nullptr, &rs) == kSuccess && rs != nullptr);
  int done = 0, got = -1;
  EXPECT(pollBounded(rr, &done, &got, rs) == kSuccess && done && got == (int)src.size());
  EXPECT(pollBounded(rs, &done, &got) == kSuccess && done && got == (int)src.size());
  EXPECT(src == dst);
  closePair(&p);
}

TEST(request_ring_full_returns_no_request) {
  Pair p;
  EXPECT(makePair(&p));
  std::vector<uint8_t> buf(64);
  std::vector<Request*> reqs;
  for (int i = 0; i < kMaxRequests + 4; ++i) {
    Request* r = nullptr;
    EXPECT(netIsend(p.s, buf.data(), (int)buf.size(), i, nullptr, &r) == kSuccess);
    if (r != nullptr) reqs.push_back(r);
  }
  EXPECT((int)reqs.size() == kMaxRequests);  // the 17th and later get "try again", not an error
  // drain: post matching receives and finish everything
  std::vector<std::vector<uint8_t>> rb(reqs.size(), std::vector<uint8_t>(64));
  for (size_t i = 0; i < reqs.size(); ++i) {
    void* d = rb[i].data();
    int sz = 64, tag = 0, done = 0, got = 0;
    Request* rr = nullptr;
    EXPECT(netIrecv(p.r, 1, &d, &sz, &tag, nullptr, &rr) == kSuccess && rr != nullptr);
    if (rr) EXPECT(pollBounded(rr, &done, &got, reqs[i]) == kSuccess && done && got == 64);
    EXPECT(pollBounded(reqs[i], &done, &got) == kSuccess && done);
  }
  Request* again = nullptr;
  EXPECT(netIsend(p.s, buf.data(), 64, 0, nullptr, &again) == kSuccess && again != nullptr);  // room again
  closePair(&p);
}

TEST(peer_closed_gives_error_not_hang) {
  Pair p;
  EXPECT(makePair(&p));
  std::vector<uint8_t> big(64 << 20, 3);
  netClose(p.r);  // the receiver goes away before the message
  p.r = nullptr;
  Request* rs = nullptr;
  Result r = netIsend(p.s, big.data(), (int)big.size(), 0, nullptr, &rs);
  int done = 0, got = 0;
  if (r == kSuccess && rs != nullptr) r = pollBounded(rs, &done, &got);
  EXPECT(r == kRemoteError || r == kSystemError);  // an error code, neither success nor a time-out
  closePair(&p);
}

TEST(socket_shutdown_mid_message) {
  Pair p;
  EXPECT(makePair(&p));
  std::vector<uint8_t> src(64 << 20, 5), dst(64 << 20);
  Request *rs = nullptr, *rr = nullptr;
  void* data = dst.data();
  int sz = (int)dst.size(), tag = 0;
  EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, nullptr, &rr) == kSuccess && rr != nullptr);
  EXPECT(netIsend(p.s, src.data(), (int)src.size(), 0, nullptr, &rs) == kSuccess && rs != nullptr);
  int done = 0, got = 0;
  shutdown(p.s->sock[0].fd, SHUT_RDWR);  // one data socket dies under the transfer
  Result a = pollBounded(rr, &done, &got, rs);
  EXPECT(a == kRemoteError || a == kSystemError);
  Result b = pollBounded(rs, &done, &got);
  EXPECT(b == kRemoteError || b == kSystemError || (b == kSuccess && done));  // the sender may have queued everything already
  closePair(&p);
}

TEST(forged_control_record_is_rejected) {
  Pair p;
  EXPECT(makePair(&p));
  std::vector<uint8_t> dst(4096);
  Request* rr = nullptr;
  void* data = dst.data();
  int sz = 4096, tag = 0;
  EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, nullptr, &rr) == kSuccess && rr != nullptr);
  CtrlMsg bad = {7 /* no such type */, 0, 100, 0, 100};
  EXPECT(send(p.s->ctrl_fd, &bad, sizeof bad, 0) == (ssize_t)sizeof bad);
  int done = 0, got = 0;
  EXPECT(pollBounded(rr, &done, &got) == kRemoteError);
  closePair(&p);
  // a record that names a socket the comm does not have
  EXPECT(makePair(&p));
  rr = nullptr;
  EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, nullptr, &rr) == kSuccess && rr != nullptr);
  CtrlMsg bad2 = {kCtrlNormal, 99, 100, 0, 100};
  EXPECT(send(p.s->ctrl_fd, &bad2, sizeof bad2, 0) == (ssize_t)sizeof bad2);
  EXPECT(pollBounded(rr, &done, &got) == kRemoteError);
  closePair(&p);
}

TEST(message_larger_than_posted_receive) {
  Pair p;
  EXPECT(makePair(&p));
  std::vector<uint8_t> src(8192, 1), dst(4096);
  Request *rs = nullptr, *rr = nullptr;
  void* data = dst.data();
  int sz = 4096, tag = 0;
  EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, nullptr, &rr) == kSuccess && rr != nullptr);
  EXPECT(netIsend(p.s, src.data(), 8192, 0, nullptr, &rs) == kSuccess && rs != nullptr);
  int done = 0, got = 0;
  EXPECT(pollBounded(rr, &done, &got, rs) == kInvalidUsage);  // refused, and nothing written past the buffer
  closePair(&p);
}

TEST(silent_sender_trips_the_detectors) {
  setenv("NCCL_GPUDIRECTTCPX_SLOWNESS_SWITCH", "ALL", 1);
  setenv("NCCL_GPUDIRECTTCPX_SLOWNESS_REPORT", "ALL", 1);
  setenv("NCCL_GPUDIRECTTCPX_TIMEOUT_THRESHOLD_NS", "20000000", 1);   // 20 ms
  setenv("NCCL_GPUDIRECTTCPX_TIMEOUT_FREQUENCY_NS", "20000000", 1);
  EXPECT(netInit(countingLogger) == kSuccess);
  Pair p;
  EXPECT(makePair(&p));
  std::vector<uint8_t> dst(4096);
  Request* rr = nullptr;
  void* data = dst.data();
  int sz = 4096, tag = 0;
  EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, nullptr, &rr) == kSuccess && rr != nullptr);
  const uint64_t until = monotonicNanos() + 150000000ull;  // nobody sends for 150 ms
  int done = 0, got = 0;
  while (monotonicNanos() < until) EXPECT(netTest(rr, &done, &got) == kSuccess && !done);
  EXPECT(g_warns_ctrl.load() >= 2);   // the control-socket detector warned and repeated
  EXPECT(g_warns_stall.load() >= 1);  // and the per-request stall report fired
  // detection is warn-only: the transfer still completes afterwards
  std::vector<uint8_t> src(4096, 9);
  Request* rs = nullptr;
  EXPECT(netIsend(p.s, src.data(), 4096, 0, nullptr, &rs) == kSuccess && rs != nullptr);
  EXPECT(pollBounded(rr, &done, &got, rs) == kSuccess && done && got == 4096 && dst == src);
  closePair(&p);
  setLogger(nullptr);
  for (const char* e : {"NCCL_GPUDIRECTTCPX_SLOWNESS_SWITCH", "NCCL_GPUDIRECTTCPX_SLOWNESS_REPORT",
                        "NCCL_GPUDIRECTTCPX_TIMEOUT_THRESHOLD_NS", "NCCL_GPUDIRECTTCPX_TIMEOUT_FREQUENCY_NS"})
    unsetenv(e);
  EXPECT(netInit(nullptr) == kSuccess);
}

TEST(connect_to_dead_listener_fails_cleanly) {
  setenv("NCCL_GPUDIRECTTCPX_CONNECT_REFUSED_RETRIES", "300", 1);  // 0.3 s instead of 20 s
  EXPECT(netInit(nullptr) == kSuccess);
  char handle[kHandleMaxSize];
  ListenComm* l = nullptr;
  EXPECT(netListen(0, handle, &l) == kSuccess);
  EXPECT(netCloseListen(l) == kSuccess);  // the port is gone before anyone connects
  Comm* s = nullptr;
  Result r = kSuccess;
  const uint64_t deadline = monotonicNanos() + 40ull * 1000000000ull;
  while (s == nullptr && r == kSuccess && monotonicNanos() < deadline) r = netConnect(0, handle, &s);
  EXPECT(s == nullptr && r != kSuccess);
  unsetenv("NCCL_GPUDIRECTTCPX_CONNECT_REFUSED_RETRIES");
  EXPECT(netInit(nullptr) == kSuccess);
}

}  // namespace

int main(int argc, char** argv) {
  setenv("NCCL_GPUDIRECTTCPX_SOCKET_IFNAME", "lo", 0);
  setenv("NCCL_SOCKET_NTHREADS", "2", 0);
  setenv("NCCL_NSOCKS_PERTHREAD", "2", 0);
  if (netInit(nullptr) != kSuccess) { fprintf(stderr, "transport init failed\n"); return 1; }
  const char* filter = argc > 1 ? argv[1] : "";
  int ran = 0;
  for (const Test& t : tests()) {
    if (*filter && strstr(t.name, filter) == nullptr) continue;
    g_ok = true;
    t.fn();
    printf("%s %s\n", g_ok ? "ok" : "FAIL", t.name);
    fflush(stdout);
    if (!g_ok) ++g_failures;
    ++ran;
  }
  printf("%d test(s), %d failure(s)\n", ran, g_failures);
  return g_failures == 0 && ran > 0 ? 0 : 1;
}
