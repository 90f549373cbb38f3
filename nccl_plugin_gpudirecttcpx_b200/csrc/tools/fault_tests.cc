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
#include <linux/errqueue.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <deque>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "tcpxb/dev_queue.h"
#include "tcpxb/cu_driver.h"
#include "tcpxb/devmem.h"
#include "tcpxb/engine.h"
#include "tcpxb/kernels.h"
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

TEST(truncated_control_record_then_close) {
  // half a record arrives, then the peer's control socket goes away: an error, not a wait for the rest
  Pair p;
  EXPECT(makePair(&p));
  std::vector<uint8_t> dst(4096);
  Request* rr = nullptr;
  void* data = dst.data();
  int sz = 4096, tag = 0;
  EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, nullptr, &rr) == kSuccess && rr != nullptr);
  CtrlMsg half = {kCtrlNormal, 0, 4096, 0, 4096};
  EXPECT(send(p.s->ctrl_fd, &half, 7, 0) == 7);
  int done = 0, got = 0;
  const uint64_t until = monotonicNanos() + 50000000ull;  // 50 ms: the fragment alone completes nothing
  while (monotonicNanos() < until) EXPECT(netTest(rr, &done, &got) == kSuccess && !done);
  shutdown(p.s->ctrl_fd, SHUT_RDWR);
  Result r = pollBounded(rr, &done, &got);
  EXPECT(r == kRemoteError || r == kSystemError);
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

TEST(close_with_transfers_in_flight) {
  // NCCL's abort path closes comms whatever state they are in: helper threads must
  // stop, nothing may be touched afterwards, and the other side sees an error.
  Pair p;
  EXPECT(makePair(&p));
  std::vector<uint8_t> src(32 << 20, 7), dst(32 << 20);
  std::vector<Request*> rs(4, nullptr);
  Request* rr = nullptr;
  void* data = dst.data();
  int sz = (int)dst.size(), tag = 0;
  EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, nullptr, &rr) == kSuccess && rr != nullptr);
  for (auto& q : rs) EXPECT(netIsend(p.s, src.data(), (int)src.size(), 0, nullptr, &q) == kSuccess && q != nullptr);
  int done = 0, got = 0;
  EXPECT(netTest(rs[0], &done, &got) == kSuccess);  // some bytes are moving, nothing is complete on the wire yet
  const uint64_t t0 = monotonicNanos();
  EXPECT(netClose(p.s) == kSuccess);                // three and a half messages never leave
  p.s = nullptr;
  EXPECT(monotonicNanos() - t0 < 3000000000ull);
  // the first message may or may not have made it; the second receive can only fail
  Result a = pollBounded(rr, &done, &got);
  EXPECT(a == kRemoteError || a == kSystemError || (a == kSuccess && done));
  if (a == kSuccess) {
    Request* rr2 = nullptr;
    Result b = netIrecv(p.r, 1, &data, &sz, &tag, nullptr, &rr2);
    if (b == kSuccess && rr2 != nullptr) b = pollBounded(rr2, &done, &got);
    EXPECT(b == kRemoteError || b == kSystemError);
  }
  closePair(&p);
}

TEST(close_listen_with_nobody_connecting) {
  char handle[kHandleMaxSize];
  ListenComm* l = nullptr;
  EXPECT(netListen(0, handle, &l) == kSuccess);
  Comm* r = nullptr;
  for (int i = 0; i < 3; ++i) EXPECT(netAccept(l, &r) == kSuccess && r == nullptr);  // an accept is pending in the background
  const uint64_t t0 = monotonicNanos();
  EXPECT(netCloseListen(l) == kSuccess);  // must not wait for a peer that never comes
  EXPECT(monotonicNanos() - t0 < 3000000000ull);
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
  setenv("NCCL_PROTO", "Simple", 1);  // the consumer of these tests is the test itself
  setenv("NCCL_ALGO", "Ring", 1);
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
  ~DevXfer() {  // registrations do not refer to the comm, so they may outlive it
    netDeregMr(nullptr, smh);
    netDeregMr(nullptr, rmh);
  }
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
  netDeregMr(nullptr, emh);
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

TEST(device_send_and_the_staging_ring) {
  setenv("NCCL_GPUDIRECTTCPX_TX_STAGING_BYTES", "1048576", 1);
  unpackModeOn("8388608");
  Pair p;
  EXPECT(makePair(&p));
  int done = 0, got = 0;
  // a message larger than the ring can never be staged: refused at once, with a reason
  std::vector<uint8_t> big(2 << 20, 1);
  MemHandle* bmh = nullptr;
  Request* rs = nullptr;
  EXPECT(netRegMr(p.s, big.data(), big.size(), kPtrCuda, &bmh) == kSuccess);
  EXPECT(netIsend(p.s, big.data(), (int)big.size(), 0, bmh, &rs) == kInvalidArgument && rs == nullptr);
  netDeregMr(nullptr, bmh);
  // messages as large as the ring go through one after the other, also after the ring's
  // write position has moved off zero
  const int sizes[] = {300001, 1048576, 4096, 1048576, 1048576};
  for (int i = 0; i < 5; ++i) {
    DevXfer x;
    EXPECT(postDevXfer(&p, &x, sizes[i], i, (uint8_t)(0x10 + i)));
    EXPECT(pollBounded(x.rr, &done, &got, x.rs) == kSuccess && done && got == sizes[i]);
    EXPECT(applyScatterList(x.rr, &x.dst) && x.dst == x.src);
    EXPECT(netIrecvConsumed(p.r, 1, x.rr) == kSuccess);
    EXPECT(pollBounded(x.rs, &done, &got) == kSuccess && done);
  }
  closePair(&p);
  unsetenv("NCCL_GPUDIRECTTCPX_TX_STAGING_BYTES");
  unpackModeOff();
}


// ---- the devmem-TCP datapath against a model of the kernel
// What a devmem NIC + kernel do, with loopback sockets underneath: a receive reads
// the stream's bytes into pages of the bound pool and reports them as fragment records
// with tokens; a transmit reads the payload out of the dma-buf the control message
// names and later posts a completion notice; DONTNEED takes the pages back.
struct KernelModel {
  std::mutex mu;
  uint8_t* pool = nullptr;
  uint64_t pool_bytes = 0;
  std::vector<uint32_t> free_pages;
  std::map<uint32_t, uint32_t> live;            // token -> page
  uint32_t next_token = 1000;
  std::map<uint32_t, const uint8_t*> dmabufs;   // transmit binding id -> base of the exported range
  std::map<int, std::deque<std::pair<uint32_t, uint32_t>>> notices;  // per socket: completed send ids [lo, hi]
  std::map<int, uint32_t> send_seq;
  uint64_t rx_fragments = 0, tx_calls = 0, dontneed_calls = 0, linear_every = 0;
} g_km;

ssize_t kmRecvmsg(int fd, struct msghdr* msg, int flags) {
  std::lock_guard<std::mutex> l(g_km.mu);
  if (flags & MSG_ERRQUEUE) {
    auto& q = g_km.notices[fd];
    if (q.empty()) { errno = EAGAIN; return -1; }
    struct cmsghdr* cm = reinterpret_cast<struct cmsghdr*>(msg->msg_control);
    cm->cmsg_level = SOL_IP;
    cm->cmsg_type = IP_RECVERR;
    cm->cmsg_len = CMSG_LEN(sizeof(struct sock_extended_err));
    struct sock_extended_err ee;
    memset(&ee, 0, sizeof ee);
    ee.ee_origin = 5;  // zero-copy completion
    ee.ee_info = q.front().first;
    ee.ee_data = q.front().second;
    memcpy(CMSG_DATA(cm), &ee, sizeof ee);
    msg->msg_controllen = CMSG_SPACE(sizeof ee);
    q.pop_front();
    return 0;
  }
  if (!(flags & devmem::kMsgSockDevmem)) { errno = EINVAL; return -1; }
  const size_t room = msg->msg_controllen / CMSG_SPACE(sizeof(devmem::DmabufCmsg));
  size_t want = std::min<size_t>(msg->msg_iov[0].iov_len, room * 4096);
  want = std::min<size_t>(want, g_km.free_pages.size() * 4096);
  if (want == 0) { errno = EAGAIN; return -1; }
  static thread_local std::vector<uint8_t> bounce;
  bounce.resize(want);
  const ssize_t n = recv(fd, bounce.data(), want, MSG_DONTWAIT);
  if (n <= 0) return n;
  size_t used = 0;
  char* c = static_cast<char*>(msg->msg_control);
  for (size_t off = 0; off < (size_t)n; off += 4096) {
    const uint32_t len = (uint32_t)std::min<size_t>(4096, (size_t)n - off);
    const uint32_t page = g_km.free_pages.back();
    g_km.free_pages.pop_back();
    memcpy(g_km.pool + (size_t)page * 4096, bounce.data() + off, len);
    const uint32_t tok = g_km.next_token++;
    g_km.live[tok] = page;
    devmem::DmabufCmsg f = {(uint64_t)page * 4096, len, tok, 0, 0};
    struct cmsghdr* cm = reinterpret_cast<struct cmsghdr*>(c + used);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = devmem::kSoDevmemDmabuf;
    cm->cmsg_len = CMSG_LEN(sizeof f);
    memcpy(CMSG_DATA(cm), &f, sizeof f);
    used += CMSG_SPACE(sizeof f);
    ++g_km.rx_fragments;
  }
  msg->msg_controllen = used;
  msg->msg_flags = 0;
  return n;
}

ssize_t kmSendmsg(int fd, const struct msghdr* msg, int flags) {
  std::lock_guard<std::mutex> l(g_km.mu);
  struct cmsghdr* cm = CMSG_FIRSTHDR(const_cast<struct msghdr*>(msg));
  if (cm == nullptr || cm->cmsg_level != SOL_SOCKET || cm->cmsg_type != devmem::kSoDevmemDmabuf) { errno = EINVAL; return -1; }
  uint32_t id = 0;
  memcpy(&id, CMSG_DATA(cm), sizeof id);
  auto it = g_km.dmabufs.find(id);
  if (it == g_km.dmabufs.end()) { errno = ENODEV; return -1; }
  const uint64_t off = (uint64_t)(uintptr_t)msg->msg_iov[0].iov_base;  // an offset, not an address
  const ssize_t n = send(fd, it->second + off, msg->msg_iov[0].iov_len, (flags & ~0x4000000) | MSG_DONTWAIT | MSG_NOSIGNAL);
  if (n > 0) {
    const uint32_t seq = g_km.send_seq[fd]++;
    g_km.notices[fd].push_back({seq, seq});
    ++g_km.tx_calls;
  }
  return n;
}

int kmSetsockopt(int, int level, int optname, const void* val, socklen_t len) {
  std::lock_guard<std::mutex> l(g_km.mu);
  if (level != SOL_SOCKET || optname != devmem::kSoDevmemDontneed) { errno = EINVAL; return -1; }
  const devmem::DmabufToken* t = static_cast<const devmem::DmabufToken*>(val);
  for (size_t i = 0; i < len / sizeof *t; ++i)
    for (uint32_t k = 0; k < t[i].token_count; ++k) {
      auto it = g_km.live.find(t[i].token_start + k);
      if (it == g_km.live.end()) { errno = EINVAL; return -1; }
      g_km.free_pages.push_back(it->second);
      g_km.live.erase(it);
    }
  ++g_km.dontneed_calls;
  return 0;
}

TEST(devmem_datapath_end_to_end_against_a_kernel_model) {
  // RX_BUF_MGR=devmem-local: CUDA buffers travel by devmem sockets; the pool is this process's own
  setenv("NCCL_GPUDIRECTTCPX_RX_BUF_MGR", "devmem-local", 1);
  setenv("NCCL_GPUDIRECTTCPX_RECV_MODE", "unpack", 1);
  setenv("NCCL_PROTO", "Simple", 1);
  setenv("NCCL_ALGO", "Ring", 1);
  setenv("NCCL_GPUDIRECTTCPX_RX_POOL_BYTES", "8388608", 1);
  EXPECT(netInit(nullptr) == kSuccess);
  const devmem::SocketOps model = {kmRecvmsg, kmSendmsg, kmSetsockopt};
  devmem::setOpsForTests(&model);
  Pair p;
  EXPECT(makePair(&p));
  // send buffers live in a shareable device allocation, so that they can be exported as a dma-buf
  cu::SharedAllocation sendmem;
  int pool_fd = -1;
  EXPECT(cu::deviceInit(0) == kSuccess && cu::sharedCreate(0, 4 << 20, &sendmem, &pool_fd) == kSuccess);
  if (pool_fd >= 0) close(pool_fd);
  uint8_t* sbase = static_cast<uint8_t*>(sendmem.dptr);
  for (size_t i = 0; i < (4u << 20); ++i) sbase[i] = (uint8_t)((i * 2654435761u) >> 11);
  const int sizes[3] = {300000, 4096, 1 << 20};
  size_t at = 12345;  // not page-aligned on purpose
  bool pool_known = false;
  for (int k = 0; k < 3; ++k) {
    const int size = sizes[k];
    std::vector<uint8_t> dst((size_t)size, 0);
    MemHandle *smh = nullptr, *rmh = nullptr;
    EXPECT(netRegMr(p.s, sbase + at, (size_t)size, kPtrCuda, &smh) == kSuccess);
    EXPECT(smh != nullptr && smh->dmabuf_fd >= 0 && smh->dmabuf_id != 0 && smh->dmabuf_offset == at);
    EXPECT(netRegMr(p.r, dst.data(), dst.size(), kPtrCuda, &rmh) == kSuccess);
    if (smh == nullptr || rmh == nullptr) break;
    {
      std::lock_guard<std::mutex> l(g_km.mu);
      g_km.dmabufs[smh->dmabuf_id] = sbase + at - smh->dmabuf_offset;  // what the NIC would have bound
    }
    void* data = dst.data();
    int sz = size, tag = k;
    Request *rr = nullptr, *rs = nullptr;
    EXPECT(netIrecv(p.r, 1, &data, &sz, &tag, &rmh, &rr) == kSuccess && rr != nullptr);
    if (!pool_known) {
      // the pool the "NIC" writes into is the receive comm's own: learn it from the first request
      ScatterList sl;
      EXPECT(netRequestScatterList(rr, &sl) == kSuccess);
      std::lock_guard<std::mutex> l(g_km.mu);
      g_km.pool = static_cast<uint8_t*>(sl.pool_dev);
      g_km.pool_bytes = sl.pool_bytes;
      for (uint32_t pg = 0; pg < sl.pool_bytes / 4096; ++pg) g_km.free_pages.push_back((pg * 773u) % (uint32_t)(sl.pool_bytes / 4096));
      pool_known = true;
    }
    EXPECT(netIsend(p.s, sbase + at, size, tag, smh, &rs) == kSuccess && rs != nullptr);
    int done = 0, got = 0;
    EXPECT(pollBounded(rr, &done, &got, rs) == kSuccess && done && got == size);
    EXPECT(pollBounded(rs, &done, &got) == kSuccess && done);  // every transmit's completion notice came back
    EXPECT(applyScatterList(rr, &dst) && memcmp(dst.data(), sbase + at, (size_t)size) == 0);
    const size_t live_before = g_km.live.size();
    EXPECT(live_before == (size_t)(size + 4095) / 4096 || live_before > 0);
    EXPECT(netIrecvConsumed(p.r, 1, rr) == kSuccess);
    EXPECT(g_km.live.empty());  // every page token went back with the consumer's release
    netDeregMr(nullptr, smh);
    netDeregMr(nullptr, rmh);
    at += (size_t)size + 777;
  }
  EXPECT(g_km.rx_fragments >= (300000 + 4096 + (1 << 20)) / 4096 && g_km.tx_calls >= 3 && g_km.dontneed_calls >= 3);
  closePair(&p);
  devmem::setOpsForTests(nullptr);
  cu::sharedRelease(&sendmem);
  unsetenv("NCCL_GPUDIRECTTCPX_RX_BUF_MGR");
  unpackModeOff();
}

// ---- the collective engine on the stand-in device
void* makeEngine(int rank, int world) {
  tcpxbEngineConfig cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.rank = rank;
  cfg.world = world;
  cfg.gpus_per_node = 1;
  cfg.request_bytes = 256 << 10;
  cfg.max_inflight = 4;
  return tcpxb_engine_create(&cfg);
}

float bf16Value(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

TEST(engine_twin_collectives_on_standin_device) {
  void* e = makeEngine(0, 1);
  EXPECT(e != nullptr);
  if (e == nullptr) return;
  std::vector<char> handles((size_t)tcpxb_engine_rails(e) * TCPXB_ENGINE_HANDLE_BYTES);
  EXPECT(tcpxb_engine_listen(e, handles.data()) == 0);
  EXPECT(tcpxb_engine_connect(e, handles.data()) == 0);  // the single rank is its own peer
  const size_t n = 700000 / 4 * 4;  // 2.8 MB of f32: several requests per rail
  std::vector<float> x(n), y(n, -1.f);
  for (size_t i = 0; i < n; ++i) x[i] = (float)(i % 1013) * 0.25f - 100.f;
  EXPECT(tcpxb_engine_all_reduce(e, x.data(), y.data(), n * 4, TCPXB_F32, nullptr) == 0);
  bool same = true;
  for (size_t i = 0; i < n; ++i) same = same && y[i] == 2.f * x[i];
  EXPECT(same);
  // bf16: doubling is exact, so the result is known bit for bit
  std::vector<uint16_t> hx(n), hy(n, 0);
  for (size_t i = 0; i < n; ++i) hx[i] = (uint16_t)(0x3f80 + (i % 64));  // 1.0 .. 1.49
  EXPECT(tcpxb_engine_all_reduce(e, hx.data(), hy.data(), n * 2, TCPXB_BF16, nullptr) == 0);
  same = true;
  for (size_t i = 0; i < n; ++i) same = same && bf16Value(hy[i]) == 2.f * bf16Value(hx[i]);
  EXPECT(same);
  // all_gather: both blocks hold the twin's data; reduce_scatter: twice the block
  std::vector<float> g(2 * n, -1.f), rs(n, -1.f);
  EXPECT(tcpxb_engine_all_gather(e, x.data(), g.data(), n * 4, nullptr) == 0);
  EXPECT(memcmp(g.data(), x.data(), n * 4) == 0 && memcmp(g.data() + n, x.data(), n * 4) == 0);
  EXPECT(tcpxb_engine_reduce_scatter(e, x.data(), rs.data(), n * 4, TCPXB_F32, nullptr) == 0);
  same = true;
  for (size_t i = 0; i < n; ++i) same = same && rs[i] == 2.f * x[i];
  EXPECT(same);
  // argument errors are messages, not crashes
  EXPECT(tcpxb_engine_all_reduce(e, x.data(), y.data(), 24, TCPXB_F32, nullptr) != 0);
  EXPECT(strstr(tcpxb_engine_last_error(), "multiple of") != nullptr);
  EXPECT(tcpxb_engine_all_reduce(e, x.data(), y.data(), n * 4, TCPXB_U8, nullptr) != 0);
  // in place between two nodes: the engine sends and adds from a copy of the input
  std::vector<float> inplace(x);
  EXPECT(tcpxb_engine_all_reduce(e, inplace.data(), inplace.data(), n * 4, TCPXB_F32, nullptr) == 0);
  same = true;
  for (size_t i = 0; i < n; ++i) same = same && inplace[i] == 2.f * x[i];
  EXPECT(same);
  uint32_t st[4] = {9, 9, 9, 9};
  EXPECT(tcpxb_engine_device_status(e, st) == 0 && st[0] == 0);
  tcpxbEngineStats es;
  EXPECT(tcpxb_engine_stats(e, &es) == 0 && es.requests > 0 && es.fragments >= es.requests && es.bytes_received == es.bytes_sent);
  tcpxb_engine_destroy(e);
}

TEST(two_engines_in_one_process_all_reduce) {
  // two ranks as two threads: the transport's shared state (flags, page pool of the one
  // stand-in device, helper threads) is used from both at once
  void* e[2] = {makeEngine(0, 2), makeEngine(1, 2)};
  EXPECT(e[0] != nullptr && e[1] != nullptr);
  if (e[0] == nullptr || e[1] == nullptr) return;
  const size_t hb = (size_t)tcpxb_engine_rails(e[0]) * TCPXB_ENGINE_HANDLE_BYTES;
  std::vector<char> h0(hb), h1(hb);
  EXPECT(tcpxb_engine_listen(e[0], h0.data()) == 0 && tcpxb_engine_listen(e[1], h1.data()) == 0);
  const size_t n = 400000;
  std::vector<float> x[2] = {std::vector<float>(n), std::vector<float>(n)}, y[2] = {std::vector<float>(n), std::vector<float>(n)};
  for (size_t i = 0; i < n; ++i) { x[0][i] = (float)(i % 977); x[1][i] = 0.5f * (float)(i % 31); }
  std::atomic<int> failures{0};
  auto rank = [&](int r) {
    if (tcpxb_engine_connect(e[r], r == 0 ? h1.data() : h0.data()) != 0) { ++failures; return; }
    for (int rep = 0; rep < 3; ++rep)
      if (tcpxb_engine_all_reduce(e[r], x[r].data(), y[r].data(), n * 4, TCPXB_F32, nullptr) != 0) ++failures;
  };
  std::thread t0(rank, 0), t1(rank, 1);
  t0.join();
  t1.join();
  EXPECT(failures.load() == 0);
  bool same = true;
  for (size_t i = 0; i < n; ++i) same = same && y[0][i] == x[0][i] + x[1][i] && y[1][i] == y[0][i];
  EXPECT(same);
  tcpxb_engine_destroy(e[0]);
  tcpxb_engine_destroy(e[1]);
}

TEST(engine_peer_gone_between_steps_is_an_error) {
  void* e[2] = {makeEngine(0, 2), makeEngine(1, 2)};
  EXPECT(e[0] != nullptr && e[1] != nullptr);
  if (e[0] == nullptr || e[1] == nullptr) return;
  const size_t hb = (size_t)tcpxb_engine_rails(e[0]) * TCPXB_ENGINE_HANDLE_BYTES;
  std::vector<char> h0(hb), h1(hb);
  EXPECT(tcpxb_engine_listen(e[0], h0.data()) == 0 && tcpxb_engine_listen(e[1], h1.data()) == 0);
  const size_t n = 200000;
  std::vector<float> x(n, 1.f), y0(n), y1(n);
  std::atomic<int> failures{0};
  std::thread t1([&] {
    if (tcpxb_engine_connect(e[1], h0.data()) != 0 || tcpxb_engine_all_reduce(e[1], x.data(), y1.data(), n * 4, TCPXB_F32, nullptr) != 0) ++failures;
  });
  if (tcpxb_engine_connect(e[0], h1.data()) != 0 || tcpxb_engine_all_reduce(e[0], x.data(), y0.data(), n * 4, TCPXB_F32, nullptr) != 0) ++failures;
  t1.join();
  EXPECT(failures.load() == 0 && y0[0] == 2.f && y1[n - 1] == 2.f);
  // rank 1 leaves at the step boundary; rank 0's next step must come back with an error
  tcpxb_engine_destroy(e[1]);
  const uint64_t t0 = monotonicNanos();
  EXPECT(tcpxb_engine_all_reduce(e[0], x.data(), y0.data(), n * 4, TCPXB_F32, nullptr) != 0);
  EXPECT(monotonicNanos() - t0 < 10000000000ull);
  EXPECT(strlen(tcpxb_engine_last_error()) > 0);
  tcpxb_engine_destroy(e[0]);
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
