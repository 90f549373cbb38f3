// Failure-path tests of the transport, host only: every failure is made on the host
// (a closed peer, a socket shut down in mid-message, a forged control record, a
// full ring, a silent sender) and every wait in the test is bounded.
// Usage: tcpxb_fault_tests [name-substring]
//
// The reference turns most of these situations into exit(1) or an endless poll
// (reference: src/sock/tcpx.h:186-281 exits on cmsg anomalies; a helper thread that
// hits a socket error just returns, src/net_tcpx.cc:329,350, and the proxy then
// polls forever).  Here they must surface as error codes from test().
//
// The device-memory cases run on the host-only library's stand-in device
// (TCPXB_FAKE_GPU=1, set by main): a consumer that falls behind, frees slots out of
// order or sits on the pool's pages must see "try again" or an error, never a hang.
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

#include "tcpxb/dev_queue.h"
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

TEST(polling_only_a_younger_request_still_progresses) {
  // test() runs the progress engine from the oldest unreported request; a caller that
  // never polls that one must not starve.
  Pair p;
  EXPECT(makePair(&p));
  std::vector<uint8_t> src0(1 << 20, 1), src1(1 << 20, 2), dst0(1 << 20), dst1(1 << 20);
  Request *rs0 = nullptr, *rs1 = nullptr, *rr0 = nullptr, *rr1 = nullptr;
  void* d0 = dst0.data();
  void* d1 = dst1.data();
  int sz = 1 << 20, tag = 0;
  EXPECT(netIrecv(p.r, 1, &d0, &sz, &tag, nullptr, &rr0) == kSuccess && rr0 != nullptr);
  EXPECT(netIrecv(p.r, 1, &d1, &sz, &tag, nullptr, &rr1) == kSuccess && rr1 != nullptr);
  EXPECT(netIsend(p.s, src0.data(), sz, 0, nullptr, &rs0) == kSuccess && rs0 != nullptr);
  EXPECT(netIsend(p.s, src1.data(), sz, 0, nullptr, &rs1) == kSuccess && rs1 != nullptr);
  int done = 0, got = 0;
  EXPECT(pollBounded(rr1, &done, &got, rs1) == kSuccess && done && got == sz && dst1 == src1);
  EXPECT(pollBounded(rs1, &done, &got) == kSuccess && done);
  EXPECT(pollBounded(rr0, &done, &got, rs0) == kSuccess && done && dst0 == src0);
  EXPECT(pollBounded(rs0, &done, &got) == kSuccess && done);
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

// ---- device-memory receives on the stand-in device
void unpackModeOn(const char* pool_bytes) {
  setenv("NCCL_GPUDIRECTTCPX_RECV_MODE", "unpack", 1);
  setenv("NCCL_GPUDIRECTTCPX_RX_POOL_BYTES", pool_bytes, 1);  // the first device receive sizes the pool for the process
  EXPECT(netInit(nullptr) == kSuccess);
}
void unpackModeOff() {
  unsetenv("NCCL_GPUDIRECTTCPX_RECV_MODE");
  unsetenv("NCCL_GPUDIRECTTCPX_RX_POOL_BYTES");
  EXPECT(netInit(nullptr) == kSuccess);
}

struct DevXfer {
  std::vector<uint8_t> src, dst;
  MemHandle *smh = nullptr, *rmh = nullptr;
  Request *rs = nullptr, *rr = nullptr;
};

// Registers both buffers as device memory and posts the receive, then the send.
bool postDevXfer(Pair* p, DevXfer* x, int size, int tag, uint8_t fill) {
  x->src.assign((size_t)size, fill);
  x->dst.assign((size_t)size, 0);
  if (netRegMr(p->s, x->src.data(), x->src.size(), kPtrCuda, &x->smh) != kSuccess) return false;
  if (netRegMr(p->r, x->dst.data(), x->dst.size(), kPtrCuda, &x->rmh) != kSuccess) return false;
  void* data = x->dst.data();
  int sz = size;
  if (netIrecv(p->r, 1, &data, &sz, &tag, &x->rmh, &x->rr) != kSuccess || x->rr == nullptr) return false;
  return netIsend(p->s, x->src.data(), size, tag, x->smh, &x->rs) == kSuccess && x->rs != nullptr;
}

// The consumer's part: copy the fragments out of the pool.  Records arrive in the order
// the chunks finished, so only bounds and total coverage are checked here; the byte
// comparison by the caller catches overlaps and holes.
bool applyScatterList(Request* rr, std::vector<uint8_t>* dst) {
  ScatterList sl;
  if (netRequestScatterList(rr, &sl) != kSuccess) return false;
  uint64_t covered = 0;
  for (uint64_t i = 0; i < sl.count; ++i) {
    const LoadMeta& m = sl.host[i];
    if (m.dst_off + m.len > dst->size() || (uint64_t)m.src_off + m.len > sl.pool_bytes) return false;
    memcpy(dst->data() + m.dst_off, static_cast<const uint8_t*>(sl.pool_dev) + m.src_off, m.len);
    covered += m.len;
  }
  return covered == dst->size();
}

TEST(device_consumer_behind_gets_try_again) {
  unpackModeOn("8388608");
  Pair p;
  EXPECT(makePair(&p));
  std::vector<DevXfer> x(kUnpackQueueDepth);
  int done = 0, got = 0;
  for (int i = 0; i < kUnpackQueueDepth; ++i) {
    EXPECT(postDevXfer(&p, &x[i], 20000, i, (uint8_t)(i + 1)));
    EXPECT(pollBounded(x[i].rr, &done, &got, x[i].rs) == kSuccess && done && got == 20000);
    EXPECT(pollBounded(x[i].rs, &done, &got) == kSuccess && done);
  }
  // every scatter-list slot now waits for its consumer: a further receive is "try again", not an error
  std::vector<uint8_t> extra(20000);
  MemHandle* emh = nullptr;
  EXPECT(netRegMr(p.r, extra.data(), extra.size(), kPtrCuda, &emh) == kSuccess);
  void* data = extra.data();
  int sz = 20000, tag = 99;
  Request* rr = nullptr;
  EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, &emh, &rr) == kSuccess && rr == nullptr);
  // slots are freed oldest first; freeing a younger one is refused and changes nothing
  EXPECT(netIrecvConsumed(p.r, 1, x[1].rr) == kInvalidUsage);
  EXPECT(applyScatterList(x[0].rr, &x[0].dst) && x[0].dst == x[0].src);
  EXPECT(netIrecvConsumed(p.r, 1, x[0].rr) == kSuccess);
  EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, &emh, &rr) == kSuccess && rr != nullptr);  // room again
  for (int i = 1; i < kUnpackQueueDepth; ++i) {
    EXPECT(applyScatterList(x[i].rr, &x[i].dst) && x[i].dst == x[i].src);
    EXPECT(netIrecvConsumed(p.r, 1, x[i].rr) == kSuccess);
  }
  closePair(&p);
  unpackModeOff();
}

TEST(device_pool_exhaustion_is_backpressure) {
  unpackModeOn("8388608");  // an 8 MiB pool (already created by the previous device test, same size)
  Pair p;
  EXPECT(makePair(&p));
  // four 4 MiB messages want twice the pool; the consumer holds on to what it has received
  std::vector<DevXfer> x(4);
  for (int i = 0; i < 4; ++i) EXPECT(postDevXfer(&p, &x[i], 4 << 20, i, (uint8_t)(0x40 + i)));
  int done = 0, got = 0;
  EXPECT(pollBounded(x[0].rr, &done, &got, x[0].rs) == kSuccess && done);
  EXPECT(pollBounded(x[1].rr, &done, &got, x[1].rs) == kSuccess && done);
  // the third cannot finish while the first two keep the pages: still in progress after a while, no error
  const uint64_t until = monotonicNanos() + 200000000ull;
  while (monotonicNanos() < until) {
    EXPECT(netTest(x[2].rr, &done, &got) == kSuccess && !done);
    if (!g_ok) break;
  }
  for (int i = 0; i < 4; ++i) {
    if (i >= 2) EXPECT(pollBounded(x[i].rr, &done, &got, x[i].rs) == kSuccess && done && got == (4 << 20));
    EXPECT(applyScatterList(x[i].rr, &x[i].dst) && x[i].dst == x[i].src);
    EXPECT(netIrecvConsumed(p.r, 1, x[i].rr) == kSuccess);  // returns the pages; the next message can land
  }
  for (int i = 0; i < 4; ++i) EXPECT(pollBounded(x[i].rs, &done, &got) == kSuccess && done);
  closePair(&p);
  unpackModeOff();
}

}  // namespace

int main(int argc, char** argv) {
  setenv("TCPXB_FAKE_GPU", "1", 0);
  setenv("NCCL_GPUDIRECTTCPX_SOCKET_IFNAME", "lo", 0);
  setenv("NCCL_SOCKET_NTHREADS", "2", 0);
  setenv("NCCL_NSOCKS_PERTHREAD", "2", 0);
  if (netInit(nullptr) != kSuccess) { fprintf(stderr, "transport init failed\n"); return 1; }
  const char* filter = argc > 1 ? argv[1] : "";
  int ran = 0;
  for (const Test& t : tests()) {
    if (*filter && strstr(t.name, filter) == nullptr) continue;
    g_ok = true;
    g_seen.clear();  // request addresses are reused from one test to the next
    t.fn();
    printf("%s %s\n", g_ok ? "ok" : "FAIL", t.name);
    fflush(stdout);
    if (!g_ok) ++g_failures;
    ++ran;
  }
  printf("%d test(s), %d failure(s)\n", ran, g_failures);
  return g_failures == 0 && ran > 0 ? 0 : 1;
}
