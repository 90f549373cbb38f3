// Unit tests of the host core, no GPU and no network peer needed.
// Usage: tcpxb_unit_tests [name-substring]; prints "ok <name>" / "FAIL <name>" lines
// and exits non-zero when any test failed.
//
// Covers what the reference tests (reference: src/stats/tracepoint_test.cc:26-134
// counter arithmetic, src/stats/stats_buffer_test.cc:37-92 concurrent producers and
// consumer wake-up) and the rest of the scheduling primitives, which it leaves
// untested: ring cursor algebra, both flow mappers, control-record coalescing,
// the stall detector on an injected clock, flag parsing and range fallback,
// interface-list syntax, the page allocator and the scatter-list ring.
#include <stdio.h>
#include <sys/time.h>
#include <stdlib.h>
#include <string.h>
#include <linux/errqueue.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <functional>
#include <map>
#include <set>
#include <string>
#include <thread>
#include <vector>

#include "tcpxb/ctrl_sock.h"
#include "tcpxb/cu_driver.h"
#include "tcpxb/dev_queue.h"
#include "tcpxb/devmem.h"
#include "tcpxb/flags.h"
#include "tcpxb/flow_mapper.h"
#include "tcpxb/gpu.h"
#include "tcpxb/rx_buf_mgr.h"
#include "tcpxb/rxdm.h"
#include "tcpxb/rxdm_proto.h"
#include "tcpxb/socket_utils.h"
#include "tcpxb/stage_ring.h"
#include "tcpxb/telemetry.h"
#include "tcpxb/timeout.h"
#include "tcpxb/transport.h"

using namespace tcpxb;

namespace {

int g_failures = 0;
bool g_current_ok = true;
#define EXPECT(cond)                                                         \
  do {                                                                       \
    if (!(cond)) {                                                           \
      fprintf(stderr, "  %s:%d expectation failed: %s\n", __FILE__, __LINE__, #cond); \
      g_current_ok = false;                                                  \
    }                                                                        \
  } while (0)

struct Test { const char* name; std::function<void()> fn; };
std::vector<Test>& tests() { static std::vector<Test> t; return t; }
struct Reg { Reg(const char* n, std::function<void()> f) { tests().push_back({n, f}); } };
#define TEST(name) void test_##name(); Reg reg_##name(#name, test_##name); void test_##name()

uint64_t g_fake_now = 0;
uint64_t fakeClock() { return g_fake_now; }

// ---------------------------------------------------------------- stage ring
TEST(ring_cursor_algebra) {
  StageRing<int, 6, 3, false> r;
  EXPECT(r.empty() && r.numFree() == 6 && !r.has(1) && !r.has(2) && !r.has(3));
  for (int i = 0; i < 6; ++i) { r.nextFree() = 100 + i; r.admit(); }
  EXPECT(!r.hasFree() && r.count(1) == 6 && r.inFlight() == 6);
  EXPECT(r.front(1) == 100);
  r.advance(1);
  r.advance(1);
  EXPECT(r.count(1) == 4 && r.count(2) == 2 && r.front(2) == 100 && r.front(1) == 102);
  r.advance(2);
  EXPECT(r.count(2) == 1 && r.count(3) == 1 && r.front(3) == 100 && r.at(1, 3) == 105);
  EXPECT(!r.hasFree());
  r.advance(3);
  EXPECT(r.numFree() == 1 && r.inFlight() == 5);
  r.nextFree() = 999;
  r.admit();
  EXPECT(r.at(1, 4) == 999);  // wrapped into slot 0
  // wrap many times: invariants hold
  for (int i = 0; i < 100000; ++i) {
    while (r.has(1)) r.advance(1);
    while (r.has(2)) r.advance(2);
    while (r.has(3)) r.advance(3);
    EXPECT(r.empty());
    r.nextFree() = i; r.admit();
    if (!g_current_ok) break;
  }
}

TEST(ring_cursor_crosses_2_32) {
  // capacity 6 does not divide 2^32: with 32-bit cursors the slot of index 2^32 would be
  // slot 0 while index 2^32 - 1 sits in slot 3, and a live item could be overwritten
  StageRing<uint64_t, 6, 3, false> r;
  for (uint64_t start : {(uint64_t)UINT32_MAX - 9, (uint64_t)UINT32_MAX * 3 - 2}) {
    r.reset(start);
    uint64_t next_in = 0, next_out = 0;
    for (int round = 0; round < 40; ++round) {
      while (r.hasFree()) { r.nextFree() = next_in++; r.admit(); }
      EXPECT(r.inFlight() == 6 && r.count(1) == 6);
      // every live item is intact: no admitted item landed on another live one
      for (uint32_t k = 0; k < 6; ++k) EXPECT(r.at(1, k) == next_out + k);
      for (int k = 0; k < 1 + round % 5; ++k) {
        EXPECT(r.front(1) == next_out);
        r.advance(1); r.advance(2); r.advance(3);
        ++next_out;
      }
    }
    EXPECT(r.slot(r.frontIndex(1)) == next_out);
  }
}

TEST(ring_spsc_threads) {
  // producer admits and reaps, consumer moves the two middle boundaries: the
  // ownership split used between the proxy thread and a helper thread
  static StageRing<uint64_t, 6, 3, true> r;
  r.reset();
  const uint64_t total = 200000;
  std::atomic<bool> bad{false};
  std::thread consumer([&] {
    uint64_t next = 0;
    while (next < total) {
      if (r.has(1)) {
        if (r.front(1) != next) bad = true;
        r.advance(1);
        r.advance(2);
        ++next;
      }
    }
  });
  uint64_t sent = 0, reaped = 0;
  while (reaped < total) {
    if (sent < total && r.hasFree()) { r.nextFree() = sent++; r.admit(); }
    while (r.has(3)) { if (r.front(3) != reaped) bad = true; r.advance(3); ++reaped; }
  }
  consumer.join();
  EXPECT(!bad.load() && r.empty());
}

// --------------------------------------------------------------- flow mappers
void mapperNeverPicksFull(FlowMapper* m) {
  srand(7);
  for (int round = 0; round < 2000; ++round) {
    int busy[kMaxSockets];
    m->reset();
    for (int s = 0; s < kMaxSockets; ++s) {
      busy[s] = rand() % (kMaxTasks + 1);
      if (busy[s] < kMaxTasks) m->offer(s, busy[s]);
    }
    int picks = 0;
    for (int s; (s = m->pick()) != -1; ++picks) {
      EXPECT(s >= 0 && s < kMaxSockets);
      EXPECT(busy[s] < kMaxTasks);  // never a socket whose task ring is full
      ++busy[s];
      if (picks > kMaxSockets * kMaxTasks) { EXPECT(false); break; }
    }
    EXPECT(!m->hasFlow() || m->pick() == -1);
  }
}
TEST(flow_mapper_rr) {
  FlowMapperRR m;
  mapperNeverPicksFull(&m);
  // with every socket empty the turn passes round all of them before repeating
  m.reset();
  for (int s = 0; s < 4; ++s) m.offer(s, 0);
  std::set<int> seen;
  for (int i = 0; i < 4; ++i) seen.insert(m.pick());
  EXPECT(seen.size() == 4);
  // all slots are usable: 4 sockets x 6 slots
  int n = 4;
  while (m.pick() != -1) ++n;
  EXPECT(n == 4 * kMaxTasks);
}
TEST(flow_mapper_katy) {
  FlowMapperKaty m;
  mapperNeverPicksFull(&m);
  m.reset();
  m.offer(0, 3); m.offer(1, 1); m.offer(2, 1); m.offer(3, 5);
  EXPECT(m.pick() == 1);  // least loaded, lowest index
  EXPECT(m.pick() == 2);
  EXPECT(m.pick() == -1);  // two picks per round
  m.reset();
  m.offer(5, 0);
  EXPECT(m.pick() == 5 && m.pick() == 5 && m.pick() == -1);  // re-offered one level up
}

// ------------------------------------------------------- buffered control socket
TEST(ctrl_buffer_coalescing) {
  int sv[2];
  EXPECT(socketpair(AF_UNIX, SOCK_STREAM, 0, sv) == 0);
  setNonBlocking(sv[0], true);
  setNonBlocking(sv[1], true);
  CtrlSendBuffer tx;
  CtrlRecvBuffer rx;
  tx.attach(sv[0]);
  rx.attach(sv[1]);
  CtrlMsg m;
  EXPECT(rx.pop(&m) == kInProgress);
  for (uint32_t i = 0; i < 8; ++i) {
    CtrlMsg c = {kCtrlNormal, (uint16_t)i, 1000 + i, i * 1000, 8000};
    EXPECT(tx.push(c) == kSuccess);
  }
  EXPECT(tx.full() && tx.pending());
  EXPECT(rx.pop(&m) == kInProgress);  // nothing on the wire before the flush
  EXPECT(tx.flush() == kSuccess && !tx.pending());
  for (uint32_t i = 0; i < 8; ++i) {
    EXPECT(rx.pop(&m) == kSuccess);
    EXPECT(m.index == i && m.size == 1000 + i && m.offset == i * 1000 && m.total == 8000);
  }
  // a 9th push flushes by itself; an inline payload behind a record is drained raw
  CtrlMsg in = {kCtrlInline, 0, 5, 0, 5};
  EXPECT(tx.push(in) == kSuccess && tx.flush() == kSuccess);
  EXPECT(send(sv[0], "hello", 5, 0) == 5);
  EXPECT(rx.pop(&m) == kSuccess && m.type == kCtrlInline && m.size == 5);
  char buf[8] = {0};
  int got = rx.drain(buf, 5);
  if (got < 5) got += (int)recv(sv[1], buf + got, (size_t)(5 - got), 0);
  EXPECT(got == 5 && memcmp(buf, "hello", 5) == 0);
  close(sv[0]);
  EXPECT(rx.pop(&m) == kRemoteError);  // peer gone is an error, not a hang
  close(sv[1]);
}

// --------------------------------------------------------------- stall detector
TEST(stall_detector_fake_clock) {
  StallDetector d;
  g_fake_now = 1000;
  d.configure(/*threshold*/ 10000, /*frequency*/ 30000, fakeClock);
  uint64_t ns = 0;
  EXPECT(!d.shouldWarn(&ns));  // first poll only starts the clock
  g_fake_now += 9999;
  EXPECT(!d.shouldWarn(&ns));
  g_fake_now += 1;
  EXPECT(d.shouldWarn(&ns) && ns == 10000);  // first warning at the threshold
  g_fake_now += 29999;
  EXPECT(!d.shouldWarn(&ns));
  g_fake_now += 1;
  EXPECT(d.shouldWarn(&ns) && ns == 40000);  // then every `frequency`
  d.reset();
  EXPECT(!d.shouldWarn(&ns) && d.polls() == 1);
  g_fake_now += 5000;
  EXPECT(!d.shouldWarn(&ns));
}

// ------------------------------------------------------------------------ flags
TEST(flags_defaults_and_ranges) {
  unsetenv("NCCL_DYNAMIC_CHUNK_SIZE");
  unsetenv("NCCL_INLINE_THRESHOLD");
  Flags f;
  loadFlags(&f);
  EXPECT(f.dynamic_chunk_size == 128 * 1024);  // unset means the documented default, never 0
  EXPECT(f.inline_threshold == 0 && f.connection_retry == 3 && f.enable == 1);
  EXPECT(f.timeout_threshold_ns == 10000000000ll && f.timeout_frequency_ns == 30000000000ll);
  setenv("NCCL_DYNAMIC_CHUNK_SIZE", "0", 1);      // out of range: ignored
  setenv("NCCL_INLINE_THRESHOLD", "4096", 1);     // above the 2048 maximum: ignored
  setenv("NCCL_GPUDIRECTTCPX_CONNECTION_RETRY", "0x10", 1);  // base detection like strtoll(.., 0)
  setenv("NCCL_GPUDIRECTTCPX_SCHED_ALG", "katy", 1);
  setenv("NCCL_GPUDIRECTTCPX_SLOWNESS_SWITCH", "TX_COMP,RX_CTRL", 1);
  setenv("NCCL_GPUDIRECTTCPX_SLOWNESS_REPORT", "ALL", 1);
  setenv("NCCL_GPUDIRECTTCPX_TELEMETRY_SAMPLING_FACTOR", "banana", 1);
  loadFlags(&f);
  EXPECT(f.dynamic_chunk_size == 128 * 1024 && f.inline_threshold == 0);
  EXPECT(f.connection_retry == 16 && f.sched_alg == kSchedKaty && f.sampling_factor == 1);
  EXPECT(f.slow_switch[kSlowTxComp] && !f.slow_switch[kSlowSendRecv] && f.slow_switch[kSlowRxCtrl]);
  EXPECT(f.slow_report[0] && f.slow_report[1] && f.slow_report[2]);
  setenv("NCCL_INLINE_THRESHOLD", "2048", 1);
  setenv("NCCL_DYNAMIC_CHUNK_SIZE", "1024", 1);
  loadFlags(&f);
  EXPECT(f.inline_threshold == 1024);  // never above the chunk size
  for (const char* e : {"NCCL_DYNAMIC_CHUNK_SIZE", "NCCL_INLINE_THRESHOLD", "NCCL_GPUDIRECTTCPX_CONNECTION_RETRY",
                        "NCCL_GPUDIRECTTCPX_SCHED_ALG", "NCCL_GPUDIRECTTCPX_SLOWNESS_SWITCH",
                        "NCCL_GPUDIRECTTCPX_SLOWNESS_REPORT", "NCCL_GPUDIRECTTCPX_TELEMETRY_SAMPLING_FACTOR"})
    unsetenv(e);
  // the stand-alone prefix is an alias of the plugin's own family; the NCCL-style name wins
  setenv("NET_TCPX_CONNECTION_RETRY", "7", 1);
  setenv("NET_TCPX_SCHED_ALG", "KATY", 1);
  loadFlags(&f);
  EXPECT(f.connection_retry == 7 && f.sched_alg == kSchedKaty);
  setenv("NCCL_GPUDIRECTTCPX_CONNECTION_RETRY", "5", 1);
  loadFlags(&f);
  EXPECT(f.connection_retry == 5);
  setenv("NET_TCPX_DYNAMIC_CHUNK_SIZE", "4096", 1);  // not in that family: no alias
  loadFlags(&f);
  EXPECT(f.dynamic_chunk_size == 128 * 1024);
  for (const char* e : {"NET_TCPX_CONNECTION_RETRY", "NET_TCPX_SCHED_ALG", "NCCL_GPUDIRECTTCPX_CONNECTION_RETRY", "NET_TCPX_DYNAMIC_CHUNK_SIZE"})
    unsetenv(e);
  bool sw[kSlowKinds];
  EXPECT(!parseSlownessList("SENDRECV,bogus", sw) && sw[kSlowSendRecv] && !sw[kSlowTxComp]);
  EXPECT(flagDocs().size() > 50);
  // socket buffers: off by default, taken as given, and raised when too small to keep a loopback stream moving
  EXPECT(f.socket_sndbuf == 0 && f.socket_rcvbuf == 0);
  setenv("NCCL_GPUDIRECTTCPX_SOCKET_SNDBUF", "262144", 1);
  setenv("NCCL_GPUDIRECTTCPX_SOCKET_RCVBUF", "4096", 1);
  loadFlags(&f);
  EXPECT(f.socket_sndbuf == 262144 && f.socket_rcvbuf == 65536);
  unsetenv("NCCL_GPUDIRECTTCPX_SOCKET_SNDBUF");
  unsetenv("NCCL_GPUDIRECTTCPX_SOCKET_RCVBUF");
}

TEST(page_allocator_random_walk) {
  // thousands of random allocations, promises and releases: a page is never out twice,
  // the counts always add up, and a promise can always be drawn
  for (int variant = 0; variant < 3; ++variant) {
    const uint32_t total = 777;
    PageAllocator a(total, variant > 0, 12345 + (uint64_t)variant, variant == 2 ? 8 : 1);
    std::vector<std::vector<PageRun>> held;
    std::vector<uint8_t> out(total, 0);
    uint32_t in_use = 0, promised = 0;
    uint64_t x = 88172645463325252ull + (uint64_t)variant;
    auto rnd = [&x]() { x ^= x << 13; x ^= x >> 7; x ^= x << 17; return x; };
    bool ok = true;
    for (int step = 0; step < 20000 && ok; ++step) {
      const uint32_t op = (uint32_t)(rnd() % 4);
      if (op == 0 || op == 1) {  // allocate, sometimes out of a promise
        const uint32_t n = 1 + (uint32_t)(rnd() % 40);
        const bool from_promise = op == 1 && promised >= n;
        std::vector<PageRun> runs;
        const bool got = a.alloc(n, &runs, from_promise);
        const bool should = from_promise ? true : (total - in_use - promised >= n);
        ok = ok && got == should;
        if (got) {
          uint32_t count = 0;
          for (const PageRun& r : runs)
            for (uint32_t i = 0; i < r.count; ++i) { ok = ok && r.first + i < total && !out[r.first + i]; out[r.first + i] = 1; ++count; }
          ok = ok && count == n;
          in_use += n;
          if (from_promise) promised -= n;
          held.push_back(runs);
        } else {
          ok = ok && runs.empty();
        }
      } else if (op == 2) {  // promise
        const uint32_t n = 1 + (uint32_t)(rnd() % 60);
        const bool got = a.reserve(n);
        ok = ok && got == (total - in_use - promised >= n);
        if (got) promised += n;
      } else if (!held.empty()) {  // release one allocation, now and then also give a promise back
        const size_t k = (size_t)(rnd() % held.size());
        for (const PageRun& r : held[k]) {
          a.release(r.first, r.count);
          for (uint32_t i = 0; i < r.count; ++i) out[r.first + i] = 0;
          in_use -= r.count;
        }
        held.erase(held.begin() + (long)k);
        if (promised > 0 && rnd() % 3 == 0) { const uint32_t back = 1 + (uint32_t)(rnd() % promised); a.unreserve(back); promised -= back; }
      }
      ok = ok && a.freePages() == total - in_use && a.reservedPages() == promised;
    }
    EXPECT(ok);
  }
}

// ---------------------------------------------------------------- interface lists
TEST(interface_list_syntax) {
  IfList l = parseIfList("eth,ib0");
  EXPECT(!l.exclude && !l.exact && l.specs.size() == 2);
  EXPECT(matchIfList(l, "eth0") && matchIfList(l, "eth12") && matchIfList(l, "ib0") && !matchIfList(l, "lo"));
  l = parseIfList("^docker,lo");
  EXPECT(l.exclude && !matchIfList(l, "docker0") && !matchIfList(l, "lo") && matchIfList(l, "eth0"));
  l = parseIfList("=eth0");
  EXPECT(l.exact && matchIfList(l, "eth0") && !matchIfList(l, "eth01"));
  l = parseIfList("mlx5_0:1,mlx5_1:2");
  EXPECT(l.specs[0].port == 1 && l.specs[1].port == 2);
  EXPECT(matchIfList(l, "mlx5_0", 1) && !matchIfList(l, "mlx5_0", 2) && matchIfList(l, "mlx5_1", 2));
  std::vector<NetIf> lo = findInterfaces("lo", AF_INET, nullptr);
  EXPECT(lo.size() == 1 && lo[0].loopback);
  if (!lo.empty()) {
    std::vector<NetIf> v = expandVirtual(lo[0], 3);
    EXPECT(v.size() == 3 && std::string(v[2].name) == "lo#2");
    EXPECT(addressToString(v[0].addr, false) == "127.0.0.1" && addressToString(v[2].addr, false) == "127.0.0.3");
  }
  EXPECT(envSocketFamily("AF_INET6") == AF_INET6 && envSocketFamily("") == AF_UNSPEC);
}

TEST(core_range_bindings) {
  CpuBindings b;
  std::vector<std::string> ifs = {"eth1", "eth2", "lo#0", "lo#1"};
  EXPECT(parseCoreRanges("eth1:8-21,112-125;eth2:30-31", ifs, &b));
  EXPECT(b.n_ranges[0] == 2 && b.lo[0][0] == 8 && b.hi[0][0] == 21 && b.lo[0][1] == 112 && b.hi[0][1] == 125);
  EXPECT(b.n_ranges[1] == 1 && b.lo[1][0] == 30 && b.hi[1][0] == 31 && b.n_ranges[2] == 0);
  EXPECT(parseCoreRanges("lo:0-3", ifs, &b) && b.n_ranges[2] == 1 && b.n_ranges[3] == 1);  // physical name covers its virtual devices
  EXPECT(!parseCoreRanges("eth9:1-2", ifs, &b));
  EXPECT(!parseCoreRanges("eth1:5-2", ifs, &b));
  EXPECT(parseCoreRanges("", ifs, &b) && b.n_ranges[0] == 0);
}

// --------------------------------------------------------------- page allocator
TEST(page_allocator) {
  PageAllocator a(64, /*scatter=*/false);
  std::vector<PageRun> runs;
  EXPECT(a.alloc(32, &runs) && runs.size() == 1 && runs[0].first == 0 && runs[0].count == 32);
  std::vector<PageRun> more;
  EXPECT(!a.alloc(33, &more) && more.empty() && a.freePages() == 32);
  a.release(runs[0].first, runs[0].count);
  EXPECT(a.freePages() == 64);
  more.clear();
  EXPECT(a.alloc(32, &more) && more.size() == 1 && more[0].first == 0);  // a released run comes back contiguous
  // promises: all or nothing, and nobody else may eat into them
  PageAllocator pr(100, /*scatter=*/false);
  std::vector<PageRun> held, other;
  EXPECT(pr.reserve(60) && pr.reservedPages() == 60);
  EXPECT(!pr.reserve(41) && pr.reservedPages() == 60);      // 40 are left to promise
  EXPECT(!pr.alloc(41, &other) && other.empty());            // an unpromised taker sees only those 40
  EXPECT(pr.alloc(40, &other) && pr.freePages() == 60);
  EXPECT(pr.alloc(25, &held, /*from_reservation=*/true) && pr.reservedPages() == 35 && pr.freePages() == 35);
  pr.unreserve(35);                                          // the message turned out smaller
  EXPECT(pr.reservedPages() == 0 && pr.reserve(35));
  pr.unreserve(1000);                                        // never below zero
  EXPECT(pr.reservedPages() == 0);
  PageAllocator s(1024, /*scatter=*/true);
  std::vector<PageRun> sr;
  EXPECT(s.alloc(256, &sr));
  std::set<uint32_t> pages;
  uint32_t total = 0;
  for (auto& r : sr) for (uint32_t i = 0; i < r.count; ++i) { pages.insert(r.first + i); ++total; }
  EXPECT(total == 256 && pages.size() == 256);   // exact count, no duplicates
  EXPECT(sr.size() > 128);                       // and really scattered
  for (auto& r : sr) s.release(r.first, r.count);
  EXPECT(s.freePages() == 1024);
  // groups of 8 pages scattered as units: 256 pages come out as 32 runs of 8
  PageAllocator g(1024, /*scatter=*/true, 7, /*run_pages=*/8);
  std::vector<PageRun> gr;
  EXPECT(g.alloc(256, &gr) && gr.size() <= 32 && gr.size() >= 28);
  std::set<uint32_t> gp;
  for (auto& r : gr) { EXPECT(r.first % 8 == 0 && r.count % 8 == 0); for (uint32_t i = 0; i < r.count; ++i) gp.insert(r.first + i); }
  EXPECT(gp.size() == 256);
  for (auto& r : gr) g.release(r.first, r.count);
  std::vector<PageRun> again;
  EXPECT(g.alloc(5, &again) && again.size() == 1 && again[0].count == 5);  // a partial group stays contiguous
  s.release(sr[0].first, 1);                     // double release is refused
  EXPECT(s.freePages() == 1024);
}

TEST(rx_buf_mgr_host_pool) {
  RxBufMgr* m = newHostRxBufMgr(1 << 20, true);
  EXPECT(m != nullptr);
  if (m == nullptr) return;
  EXPECT(m->bytes() == (1 << 20) && m->hostBase() != nullptr && m->devBase() == m->hostBase() && !m->deviceResident());
  std::vector<PageRun> runs;
  EXPECT(m->allocPages(256, &runs) && m->freePages() == 0);
  std::vector<PageRun> none;
  EXPECT(!m->allocPages(1, &none));
  m->releasePages(runs.data(), runs.size());
  EXPECT(m->freePages() == 256);
  EXPECT(m->registerApplication(1234) == kSuccess && m->deregisterApplication(1234) == kSuccess);
  int sv[2];
  EXPECT(socketpair(AF_UNIX, SOCK_STREAM, 0, sv) == 0);
  EXPECT(m->installFlowRule(sv[0], "0000:1b:00.0") == kSuccess && m->flowRules().size() == 1);
  EXPECT(m->removeFlowRule(sv[0]) == kSuccess && m->flowRules().empty());
  close(sv[0]);
  close(sv[1]);
  delete m;
}

// Needs a running tcpxb_rxdm; the Python test-suite starts one and names its
// directory in TCPXB_TEST_RXDM_PREFIX.  Without it the test is a no-op.
TEST(rxdm_daemon_roundtrip) {
  const char* prefix = getenv("TCPXB_TEST_RXDM_PREFIX");
  if (prefix == nullptr) { printf("  (no daemon: skipped)\n"); return; }
  setenv("NCCL_GPUDIRECTTCPX_RX_BUF_MGR", "daemon", 1);
  setenv("NCCL_GPUDIRECTTCPX_UNIX_CLIENT_PREFIX", prefix, 1);
  // the daemon under test may speak the reference's protobuf wire format instead of the native one
  const bool proto = getenv("TCPXB_TEST_RXDM_WIRE") != nullptr && !strcmp(getenv("TCPXB_TEST_RXDM_WIRE"), "proto");
  if (proto) setenv("NCCL_GPUDIRECTTCPX_RXDM_WIRE", "proto", 1);
  reloadFlags();
  auto status = [&](uint64_t* rules, uint64_t* apps, uint64_t* pools) {
    RxdmMessage q, rep;
    memset(&q, 0, sizeof q);
    q.magic = kRxdmMagic;
    q.type = kRxdmStatus;
    EXPECT(rxdmCall(prefix, "rxdm_status", q, &rep, nullptr) == kSuccess);
    *rules = rep.reply.a; *apps = rep.reply.b; *pools = rep.reply.c;
  };
  uint64_t rules = 9, apps = 9, pools = 9;
  status(&rules, &apps, &pools);
  EXPECT(rules == 0 && apps == 0);
  RxBufMgr* m = rxBufMgrFor(-1);  // imports the "host" pool: memfd over SCM_RIGHTS, mapped here
  EXPECT(m != nullptr);
  if (m == nullptr) return;
  EXPECT(m->bytes() == (8u << 20) && m->hostBase() != nullptr && m->freePages() == 2048);
  std::vector<PageRun> runs;
  EXPECT(m->allocPages(4, &runs));
  memset(m->hostBase() + (uint64_t)runs[0].first * kRxPageBytes, 0x5a, kRxPageBytes);
  // a second mapping of the same pool sees the bytes: the pool really is shared
  int fd = -1;
  if (proto) {
    rxproto::Message pq;
    pq.kind = rxproto::kRawBytes;
    pq.raw_bytes = "host";
    EXPECT(rxproto::call(prefix, "get_gpu_fd_host", pq, nullptr, &fd) == kSuccess && fd >= 0);
    // a request that names another GPU than the socket gets words back, not a descriptor
    rxproto::Message bad = pq, words;
    bad.raw_bytes = "0000:ff:00.0";
    int none = -1;
    EXPECT(rxproto::call(prefix, "get_gpu_fd_host", bad, &words, &none) == kSuccess && none < 0 && words.kind == rxproto::kRawBytes &&
           words.raw_bytes.find("Invalid argument") == 0);
  } else {
    RxdmMessage q, rep;
    memset(&q, 0, sizeof q);
    q.magic = kRxdmMagic;
    q.type = kRxdmGetGpuFd;
    snprintf(q.gpu.gpu_pci, sizeof q.gpu.gpu_pci, "host");
    EXPECT(rxdmCall(prefix, "get_gpu_fd", q, &rep, &fd) == kSuccess && fd >= 0 && rep.reply.a == (8u << 20));
  }
  if (fd >= 0) {
    uint8_t probe = 0;
    EXPECT(pread(fd, &probe, 1, (off_t)runs[0].first * kRxPageBytes + 100) == 1 && probe == 0x5a);
    close(fd);
  }
  m->releasePages(runs.data(), runs.size());
  // flow-steering rule for a real TCP connection, then its removal
  std::vector<NetIf> lo = findInterfaces("lo", AF_INET, nullptr);
  SocketAddress a = lo[0].addr;
  setAddressPort(&a, 0);
  int lfd = -1, cfd = -1, sfd = -1;
  EXPECT(createListenSocket(&lfd, &a) == kSuccess);
  EXPECT(connectAddress(&cfd, a, nullptr) == kSuccess);
  EXPECT(acceptSocket(lfd, &sfd, 2000) == kSuccess);
  EXPECT(m->installFlowRule(sfd, "0000:1b:00.0") == kSuccess && m->flowRules().size() == 1);
  status(&rules, &apps, &pools);
  EXPECT(rules == 1 && pools == 1);
  EXPECT(m->removeFlowRule(sfd) == kSuccess && m->flowRules().empty());
  status(&rules, &apps, &pools);
  EXPECT(rules == 0);
  // lifecycle: registered while the connection lives
  EXPECT(m->registerApplication(4242) == kSuccess);
  status(&rules, &apps, &pools);
  EXPECT(apps == 1);
  EXPECT(m->deregisterApplication(4242) == kSuccess);
  for (int i = 0; i < 100 && apps != 0; ++i) { usleep(20000); status(&rules, &apps, &pools); }
  EXPECT(apps == 0);
  close(cfd); close(sfd); close(lfd);
  unsetenv("NCCL_GPUDIRECTTCPX_RX_BUF_MGR");
  unsetenv("NCCL_GPUDIRECTTCPX_UNIX_CLIENT_PREFIX");
  unsetenv("NCCL_GPUDIRECTTCPX_RXDM_WIRE");
  reloadFlags();
}

// The protobuf bytes of the daemon protocol, against encodings worked out from the schema
// by hand (and cross-checked against the protobuf library by the Python tests).
TEST(rxdm_proto_wire_bytes) {
  using namespace rxproto;
  auto hex = [](const std::string& b) {
    std::string h;
    char t[4];
    for (unsigned char c : b) { snprintf(t, sizeof t, "%02x", c); h += t; }
    return h;
  };
  Message ok;
  ok.kind = kRawBytes;
  ok.raw_bytes = "Ok.";
  EXPECT(hex(encode(ok)) == "0a034f6b2e");
  Message rule;
  rule.kind = kFlowSteerRule;
  rule.has_ntuple = true;
  rule.flow_type = kFlowTcpV4;
  rule.src.present = rule.dst.present = true;
  rule.src.ip = "10.0.0.1"; rule.src.port = 5000;
  rule.dst.ip = "10.0.0.2"; rule.dst.port = 6000;
  rule.has_queue_id = true; rule.queue_id = 3;
  rule.gpu_pci_addr = "0000:1b:00.0";
  const std::string rule_hex =
      "1232" "0a20" "0801" "120d" "0a08" "31302e302e302e31" "108827" "1a0d" "0a08" "31302e302e302e32" "10f02e"
      "1003" "1a0c" "303030303a31623a30302e30";
  EXPECT(hex(encode(rule)) == rule_hex);
  Message back;
  const std::string wire = encode(rule);
  EXPECT(decode(wire.data(), wire.size(), &back) && back.kind == kFlowSteerRule && back.has_ntuple && back.flow_type == 1 &&
         back.src.ip == "10.0.0.1" && back.src.port == 5000 && back.dst.ip == "10.0.0.2" && back.dst.port == 6000 && back.has_queue_id &&
         back.queue_id == 3 && back.gpu_pci_addr == "0000:1b:00.0");
  Message reg;
  reg.kind = kAppRegister;
  reg.register_client = true;
  EXPECT(hex(encode(reg)) == "32020801");
  Message query;
  query.kind = kQueueIdQuery;
  query.gpu_pci_addr = "0000:1b:00.0";
  EXPECT(hex(encode(query)) == "1a0e0a0c303030303a31623a30302e30");
  Message resp;
  resp.kind = kQueueIdResponse;
  resp.queue_ids = {8, 9, 300};
  EXPECT(hex(encode(resp)) == "22070808" "0809" "08ac02");
  // both encodings of a repeated int32 decode: one tag per element, and packed
  const unsigned char packed[] = {0x22, 0x06, 0x0a, 0x04, 0x08, 0x09, 0xac, 0x02};
  EXPECT(decode(packed, sizeof packed, &back) && back.kind == kQueueIdResponse && back.queue_ids.size() == 3 && back.queue_ids[2] == 300);
  EXPECT(decode(encode(resp).data(), encode(resp).size(), &back) && back.queue_ids.size() == 3 && back.queue_ids[0] == 8);
  // a negative int32 takes ten bytes on the wire and comes back negative
  Message neg;
  neg.kind = kFlowSteerRule;
  neg.has_queue_id = true;
  neg.queue_id = -1;
  EXPECT(hex(encode(neg)) == "120b10ffffffffffffffffff01");
  EXPECT(decode(encode(neg).data(), encode(neg).size(), &back) && back.queue_id == -1);
  // unknown fields are skipped, whatever their wire type; truncated input is refused
  const unsigned char with_unknown[] = {0x38, 0x05, 0x0a, 0x03, 'O', 'k', '.', 0x45, 1, 2, 3, 4, 0x49, 1, 2, 3, 4, 5, 6, 7, 8};
  EXPECT(decode(with_unknown, sizeof with_unknown, &back) && back.kind == kRawBytes && back.raw_bytes == "Ok.");
  EXPECT(!decode(with_unknown, 4, &back));
  const unsigned char endless_varint[] = {0x0a, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff, 0xff};
  EXPECT(!decode(endless_varint, sizeof endless_varint, &back));
  EXPECT(decode(nullptr, 0, &back) && back.kind == kNone);
  // pool metadata: the daemon's struct {int fd; size_t size; size_t align} as raw bytes
  GpuMemMetadata md, md2;
  md.fd = 17; md.size = 1ull << 30; md.align = 2 << 20;
  const std::string raw = encodeMetadata(md);
  EXPECT(raw.size() == 24 && decodeMetadata(raw, &md2) && md2.fd == 17 && md2.size == (1ull << 30) && md2.align == (2u << 20));
  EXPECT(!decodeMetadata(raw.substr(0, 20), &md2));
  // framing over a socket pair: message, descriptor, message
  int sv[2];
  EXPECT(socketpair(AF_UNIX, SOCK_STREAM, 0, sv) == 0);
  {
    Connection a(sv[0]), b(sv[1]);
    EXPECT(a.sendMessage(rule) == kSuccess && a.sendFd(sv[0]) == kSuccess && a.sendMessage(ok) == kSuccess);
    int fd = -1;
    EXPECT(b.recv(&back, &fd) == kSuccess && fd < 0 && back.kind == kFlowSteerRule && back.dst.port == 6000);
    EXPECT(b.recv(&back, &fd) == kSuccess && fd >= 0);
    if (fd >= 0) close(fd);
    EXPECT(b.recv(&back, &fd) == kSuccess && fd < 0 && back.kind == kRawBytes && back.raw_bytes == "Ok.");
    EXPECT(b.recv(&back, &fd, 50) == kInProgress);
  }
}

TEST(memory_handles_on_standin_device) {
  if (!cu::available()) { printf("  skipped: no device (set TCPXB_FAKE_GPU=1)\n"); return; }
  cu::IpcAllocation mine, theirs;
  unsigned char handle[cu::kIpcHandleBytes];
  EXPECT(cu::ipcCreate(0, 1 << 20, &mine, handle) == kSuccess && mine.dptr != nullptr && mine.bytes == (1u << 20) && !mine.opened);
  // as with the real driver, the process that made a handle cannot open it
  EXPECT(cu::ipcOpen(0, handle, &theirs) != kSuccess && theirs.dptr == nullptr);
  // another process can, and sees the owner's bytes
  memset(mine.dptr, 0x6b, 4096);
  const pid_t child = fork();
  if (child == 0) {
    cu::IpcAllocation c;
    int rc = 1;
    if (cu::ipcOpen(0, handle, &c) == kSuccess && c.opened && c.bytes == (1u << 20) && static_cast<unsigned char*>(c.dptr)[4095] == 0x6b) {
      static_cast<unsigned char*>(c.dptr)[8192] = 0x2a;
      cu::ipcRelease(&c);
      rc = 0;
    }
    _exit(rc);
  }
  int status = -1;
  EXPECT(waitpid(child, &status, 0) == child && WIFEXITED(status) && WEXITSTATUS(status) == 0);
  EXPECT(static_cast<unsigned char*>(mine.dptr)[8192] == 0x2a);
  unsigned char junk[cu::kIpcHandleBytes];
  memset(junk, 'x', sizeof junk);
  EXPECT(cu::ipcOpen(0, junk, &theirs) != kSuccess);
  cu::ipcRelease(&mine);
  EXPECT(mine.dptr == nullptr);
  cu::ipcRelease(&mine);  // twice is harmless
}

TEST(rx_pool_skip_odds) {
  setenv("NCCL_TCPX_RXMEM_IMPORT_SKIP_ODDS", "1", 1);
  setenv("NCCL_GPUDIRECTTCPX_RX_POOL_BYTES", "4194304", 1);
  reloadFlags();
  EXPECT(rxBufMgrFor(1) == nullptr && rxBufMgrFor(3) == nullptr);  // whatever devices exist: odd ones get none
  RxBufMgr* even = rxBufMgrFor(-1);  // the host-only pool is not a GPU's and is not skipped
  EXPECT(even != nullptr && even->totalPages() == 1024);
  unsetenv("NCCL_TCPX_RXMEM_IMPORT_SKIP_ODDS");
  unsetenv("NCCL_GPUDIRECTTCPX_RX_POOL_BYTES");
  reloadFlags();
}

TEST(dev_queue_fifo) {
  DevQueue q;
  EXPECT(q.init(nullptr, false) == kSuccess);
  UnpackSlot slots[kUnpackQueueDepth + 1];
  for (int i = 0; i < kUnpackQueueDepth; ++i) {
    q.nextFree(&slots[i]);
    EXPECT(slots[i].active && slots[i].index == (uint64_t)i && slots[i].mem == q.metaHost()->mem[i]);
  }
  q.nextFree(&slots[kUnpackQueueDepth]);
  EXPECT(!slots[kUnpackQueueDepth].active && q.inUse() == (uint64_t)kUnpackQueueDepth);
  EXPECT(!q.release(3));  // only the oldest may go
  EXPECT(q.release(0) && q.inUse() == (uint64_t)kUnpackQueueDepth - 1);
  q.nextFree(&slots[kUnpackQueueDepth]);
  EXPECT(slots[kUnpackQueueDepth].active && slots[kUnpackQueueDepth].index == 0);
  static_assert(sizeof(UnpackMeta) == (size_t)kUnpackQueueDepth * kUnpackMaxSlicePages * 16 + kUnpackQueueDepth * 8, "layout");
  static_assert(sizeof(UnpackDeviceHandle) == 24, "layout");
}

// -------------------------------------------------------------------- telemetry
TEST(event_log_concurrent_producers) {
  EventLog log(64, 256);
  std::vector<std::thread> producers;
  for (int p = 0; p < 3; ++p) producers.emplace_back([&log, p] { log.push("producer %d", p); });
  for (auto& t : producers) t.join();
  int n = 0;
  std::string line;
  while (log.pop(&line, 10)) { EXPECT(line.rfind("producer ", 0) == 0); ++n; }
  EXPECT(n == 3);
  // a waiting consumer is woken by a push
  std::atomic<bool> got{false};
  std::thread consumer([&] { std::string l; got = log.pop(&l, 30000); });
  usleep(20000);
  log.push("wake");
  consumer.join();
  EXPECT(got.load());
  // a full log drops and counts, it never blocks the producer
  EventLog tiny(4, 16);
  for (int i = 0; i < 10; ++i) tiny.push("line-%d-with-a-long-tail-that-is-cut", i);
  EXPECT(tiny.size() == 4 && tiny.dropped() == 6);
  EXPECT(tiny.pop(&line, 0) && line.size() == 16);
}

TEST(flow_counters_and_lines) {
  FlowStats s;
  s.flow_id = flowIdOf("a->b tx");
  EXPECT(s.flow_id == flowIdOf("a->b tx") && s.flow_id != flowIdOf("a->c tx"));
  s.tx_cnt = 7; s.tx_completion_cnt = 5; s.tx_slow_cnt = 1; s.tx_completion_slow_cnt = 2; s.rx_cnt = 9; s.rx_slow_cnt = 3;
  std::string tx = flowStatsLine(s, "a->b tx", false), rx = flowStatsLine(s, "a->b rx", true);
  EXPECT(tx.find("] = tx [5/7] tx_slow 1 tx_comp_slow 2") != std::string::npos);
  EXPECT(rx.find("] = rx 9 rx_slow 3") != std::string::npos);
  EXPECT(tx.rfind("per_flow_stats[", 0) == 0);
}

TEST(tracepoints_and_exporter) {
  char dir[] = "/tmp/tcpxb_ut_XXXXXX";
  EXPECT(mkdtemp(dir) != nullptr);
  EventLog log(1000, 256);
  TraceConfig tc;
  tc.task_level = true; tc.request_level = false; tc.to_file = true; tc.sampling = 1;
  setTraceConfig(tc);
  int obj = 0;
  traceTransition(&log, 'T', &obj, true, "ACTIVE");
  traceTransition(&log, 'R', &obj, true, "POSTED");  // request level is off
  EXPECT(log.size() == 1);
  std::string path;
  {
    Exporter ex(&log, dir, "ut", -1);
    path = ex.path();
    traceTransition(&log, 'T', &obj, false, "INACTIVE");
    ex.stop();
  }
  FILE* f = fopen(path.c_str(), "r");
  EXPECT(f != nullptr);
  int lines = 0;
  if (f != nullptr) {
    char buf[512];
    while (fgets(buf, sizeof buf, f)) {
      char kind; void* p; int passive; char state[32]; unsigned long ns;
      EXPECT(sscanf(buf, "%c %p %d %31s %lu", &kind, &p, &passive, state, &ns) == 5);
      EXPECT(kind == 'T' && p == &obj && ns > 1600000000000000000ul);
      ++lines;
    }
    fclose(f);
  }
  EXPECT(lines == 2);
  EXPECT(Exporter::writeStatsFile(Exporter::statsPath(dir, "ut"), {"a", "b"}));
  // the collector removes only exporter_*.log files that are old enough
  EXPECT(LogGarbageCollector::sweepOnce(dir, 1) == 0);
  EXPECT(LogGarbageCollector::sweepOnce(dir, 0) == 0);
  // two hours old: an exporter log goes, a file of another name stays
  const std::string old_log = std::string(dir) + "/exporter_1_old.log", other = std::string(dir) + "/notes.log";
  for (const std::string& pth : {old_log, other}) {
    FILE* of = fopen(pth.c_str(), "w");
    EXPECT(of != nullptr);
    if (of != nullptr) fclose(of);
    struct timeval tv[2];
    gettimeofday(&tv[0], nullptr);
    tv[0].tv_sec -= 7200;
    tv[1] = tv[0];
    EXPECT(utimes(pth.c_str(), tv) == 0);
  }
  EXPECT(LogGarbageCollector::sweepOnce(dir, 60) == 1);
  EXPECT(access(old_log.c_str(), F_OK) != 0 && access(other.c_str(), F_OK) == 0);
  {
    // the background collector does the same on its period
    FILE* of = fopen(old_log.c_str(), "w");
    if (of != nullptr) fclose(of);
    struct timeval tv[2];
    gettimeofday(&tv[0], nullptr);
    tv[0].tv_sec -= 7200;
    tv[1] = tv[0];
    utimes(old_log.c_str(), tv);
    LogGarbageCollector gc(dir, 60, 1, -1);
    const uint64_t until = monotonicNanos() + 3000000000ull;
    while (access(old_log.c_str(), F_OK) == 0 && monotonicNanos() < until) usleep(10000);
    EXPECT(access(old_log.c_str(), F_OK) != 0);
  }
  setTraceConfig(TraceConfig());
  std::string cmd = std::string("rm -r ") + dir;
  EXPECT(system(cmd.c_str()) == 0);
}


// ------------------------------------------------------------------ devmem-TCP
// A control buffer as recvmsg(MSG_SOCK_DEVMEM) would fill it.
struct CmsgBuilder {
  std::vector<char> buf;
  struct msghdr msg;
  size_t used = 0;
  explicit CmsgBuilder(size_t fragments) : buf(devmem::rxControlBytes(fragments) + 64) { memset(&msg, 0, sizeof msg); }
  void add(int type, uint64_t off, uint32_t size, uint32_t token, uint32_t dmabuf = 1) {
    devmem::DmabufCmsg f = {off, size, token, dmabuf, 0};
    msg.msg_control = buf.data();
    msg.msg_controllen = used + CMSG_SPACE(sizeof f);
    struct cmsghdr* cm = reinterpret_cast<struct cmsghdr*>(buf.data() + used);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = type;
    cm->cmsg_len = CMSG_LEN(sizeof f);
    memcpy(CMSG_DATA(cm), &f, sizeof f);
    used += CMSG_SPACE(sizeof f);
  }
};

TEST(devmem_recv_fragments_become_records_and_token_runs) {
  CmsgBuilder b(8);
  const uint64_t offs[5] = {81920, 4096, 1 << 20, 12288, 40960};
  const uint32_t toks[5] = {7, 8, 9, 20, 21};
  for (int i = 0; i < 5; ++i) b.add(devmem::kSoDevmemDmabuf, offs[i], i == 4 ? 1000 : 4096, toks[i]);
  LoadMeta rec[16];
  std::vector<devmem::DmabufToken> runs;
  devmem::RxSink sink;
  sink.records = rec; sink.capacity = 16; sink.tokens = &runs; sink.pool_bytes = 8 << 20; sink.dmabuf_id = 1;
  EXPECT(devmem::parseRecv(&b.msg, 4 * 4096 + 1000, 1 << 16, &sink) == kSuccess);
  EXPECT(sink.filled == 5);
  for (int i = 0; i < 5; ++i) {
    EXPECT(rec[i].src_off == offs[i] && rec[i].len == (i == 4 ? 1000u : 4096u));
    EXPECT(rec[i].dst_off == (1u << 16) + (uint64_t)i * 4096);
  }
  EXPECT(runs.size() == 2 && runs[0].token_start == 7 && runs[0].token_count == 3 && runs[1].token_start == 20 && runs[1].token_count == 2);
  // a second recvmsg of the same message appends, and its first token extends the last run
  CmsgBuilder c(2);
  c.add(devmem::kSoDevmemDmabuf, 8192, 4096, 22);
  EXPECT(devmem::parseRecv(&c.msg, 4096, (1 << 16) + 4 * 4096 + 1000, &sink) == kSuccess);
  EXPECT(sink.filled == 6 && runs.size() == 2 && runs[1].token_count == 3);
}

TEST(devmem_recv_refuses_what_the_scatter_list_cannot_describe) {
  LoadMeta rec[4];
  std::vector<devmem::DmabufToken> runs;
  auto freshSink = [&] {
    devmem::RxSink s;
    s.records = rec; s.capacity = 4; s.tokens = &runs; s.pool_bytes = 1 << 20; s.dmabuf_id = 1;
    runs.clear();
    return s;
  };
  {  // payload in the host linear buffer: the flow missed the devmem queue
    CmsgBuilder b(3);
    b.add(devmem::kSoDevmemDmabuf, 0, 4096, 1);
    b.add(devmem::kSoDevmemLinear, 0, 512, 0);
    b.add(devmem::kSoDevmemDmabuf, 4096, 4096, 2);
    devmem::RxSink s = freshSink();
    EXPECT(devmem::parseRecv(&b.msg, 8192 + 512, 0, &s) == kInternalError);
    EXPECT(runs.size() == 1 && runs[0].token_count == 2);  // both tokens can still be handed back
  }
  {  // an empty linear record is harmless (the kernel emits one for a header-only skb)
    CmsgBuilder b(2);
    b.add(devmem::kSoDevmemLinear, 0, 0, 0);
    b.add(devmem::kSoDevmemDmabuf, 0, 100, 1);
    devmem::RxSink s = freshSink();
    EXPECT(devmem::parseRecv(&b.msg, 100, 0, &s) == kSuccess && s.filled == 1);
  }
  {  // a fragment longer than a page is cut into page-sized records under one token
    CmsgBuilder b(1);
    b.add(devmem::kSoDevmemDmabuf, 65536, 10000, 5);
    devmem::RxSink s = freshSink();
    EXPECT(devmem::parseRecv(&b.msg, 10000, 300, &s) == kSuccess && s.filled == 3);
    EXPECT(rec[0].len == 4096 && rec[1].len == 4096 && rec[2].len == 10000 - 8192);
    EXPECT(rec[2].src_off == 65536 + 8192 && rec[2].dst_off == 300 + 8192 && runs.size() == 1 && runs[0].token_count == 1);
  }
  {  // more fragments than the list holds
    CmsgBuilder b(6);
    for (uint32_t i = 0; i < 6; ++i) b.add(devmem::kSoDevmemDmabuf, i * 4096, 4096, i);
    devmem::RxSink s = freshSink();
    EXPECT(devmem::parseRecv(&b.msg, 6 * 4096, 0, &s) == kInternalError);
    EXPECT(runs.size() == 1 && runs[0].token_count == 6);
  }
  {  // truncated control buffer, fragments that do not add up, a fragment outside the pool, a foreign dma-buf
    CmsgBuilder b(1);
    b.add(devmem::kSoDevmemDmabuf, 0, 4096, 1);
    devmem::RxSink s = freshSink();
    b.msg.msg_flags = MSG_CTRUNC;
    EXPECT(devmem::parseRecv(&b.msg, 4096, 0, &s) == kInternalError);
    b.msg.msg_flags = 0;
    s = freshSink();
    EXPECT(devmem::parseRecv(&b.msg, 5000, 0, &s) == kInternalError);
    CmsgBuilder o(1);
    o.add(devmem::kSoDevmemDmabuf, (1 << 20) - 100, 4096, 1);
    s = freshSink();
    EXPECT(devmem::parseRecv(&o.msg, 4096, 0, &s) == kInternalError);
    CmsgBuilder f(1);
    f.add(devmem::kSoDevmemDmabuf, 0, 4096, 1, /*dmabuf=*/9);
    s = freshSink();
    EXPECT(devmem::parseRecv(&f.msg, 4096, 0, &s) == kInternalError);
    struct msghdr none;
    memset(&none, 0, sizeof none);
    s = freshSink();
    EXPECT(devmem::parseRecv(&none, 4096, 0, &s) == kInternalError);  // bytes without any fragment record
  }
  {  // the scatter-list slot of a request holds 2048 records: fragment 2049 is refused
    std::vector<LoadMeta> big(kUnpackMaxSlicePages);
    CmsgBuilder b(kUnpackMaxSlicePages + 1);
    for (uint32_t i = 0; i <= (uint32_t)kUnpackMaxSlicePages; ++i) b.add(devmem::kSoDevmemDmabuf, (uint64_t)i * 2048, 2048, i);
    devmem::RxSink s;
    s.records = big.data(); s.capacity = big.size(); s.tokens = &runs; s.pool_bytes = 16 << 20;
    runs.clear();
    EXPECT(devmem::parseRecv(&b.msg, (kUnpackMaxSlicePages + 1) * 2048, 0, &s) == kInternalError && s.filled == big.size());
  }
}

std::vector<std::pair<int, size_t>> g_dontneed_calls;  // (fd, runs) per setsockopt
int g_dontneed_fail_at = -1;
int fakeDontneed(int fd, int level, int optname, const void* val, socklen_t len) {
  if (level != SOL_SOCKET || optname != devmem::kSoDevmemDontneed || val == nullptr || len % sizeof(devmem::DmabufToken)) { errno = EINVAL; return -1; }
  if ((int)g_dontneed_calls.size() == g_dontneed_fail_at) { errno = ENOMEM; return -1; }
  g_dontneed_calls.push_back({fd, len / sizeof(devmem::DmabufToken)});
  return 0;
}

TEST(devmem_tokens_go_back_in_batches) {
  devmem::SocketOps ops = devmem::systemOps();
  ops.setsockopt = fakeDontneed;
  std::vector<devmem::DmabufToken> runs;
  for (uint32_t i = 0; i < 300; ++i) runs.push_back({i * 10, 3});
  g_dontneed_calls.clear();
  g_dontneed_fail_at = -1;
  size_t calls = 0;
  EXPECT(devmem::recycle(ops, 42, &runs, &calls) == kSuccess && runs.empty() && calls == 3);
  EXPECT(g_dontneed_calls.size() == 3 && g_dontneed_calls[0].second == 128 && g_dontneed_calls[1].second == 128 && g_dontneed_calls[2].second == 44);
  EXPECT(g_dontneed_calls[0].first == 42);
  // a failing call keeps what was not handed back yet
  for (uint32_t i = 0; i < 200; ++i) runs.push_back({i * 10, 1});
  g_dontneed_calls.clear();
  g_dontneed_fail_at = 1;
  EXPECT(devmem::recycle(ops, 42, &runs, nullptr) == kSystemError && runs.size() == 72 && runs[0].token_start == 1280);
  g_dontneed_fail_at = -1;
}

TEST(devmem_send_message_and_completion_accounting) {
  devmem::TxMessage m;
  devmem::buildSend(&m, 77, (5ull << 30) + 12345, 262144);
  EXPECT(m.msg.msg_iovlen == 1 && (uintptr_t)m.iov.iov_base == (5ull << 30) + 12345 && m.iov.iov_len == 262144);
  struct cmsghdr* cm = CMSG_FIRSTHDR(&m.msg);
  uint32_t id = 0;
  memcpy(&id, CMSG_DATA(cm), 4);
  EXPECT(cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == devmem::kSoDevmemDmabuf && id == 77 && CMSG_NXTHDR(&m.msg, cm) == nullptr);
  // an error-queue notice as the kernel writes it: inclusive range in ee_info .. ee_data
  char control[CMSG_SPACE(sizeof(struct sock_extended_err))];
  memset(control, 0, sizeof control);
  struct msghdr em;
  memset(&em, 0, sizeof em);
  em.msg_control = control;
  em.msg_controllen = sizeof control;
  struct cmsghdr* ec = CMSG_FIRSTHDR(&em);
  ec->cmsg_level = SOL_IP;
  ec->cmsg_type = IP_RECVERR;
  ec->cmsg_len = CMSG_LEN(sizeof(struct sock_extended_err));
  struct sock_extended_err ee;
  memset(&ee, 0, sizeof ee);
  ee.ee_origin = 5;  // SO_EE_ORIGIN_ZEROCOPY
  ee.ee_info = 10;
  ee.ee_data = 14;
  memcpy(CMSG_DATA(ec), &ee, sizeof ee);
  uint32_t lo = 0, hi = 0;
  EXPECT(devmem::parseZerocopyNotice(&em, &lo, &hi) && lo == 10 && hi == 15);
  ee.ee_origin = 2;  // an ICMP error, not a completion
  memcpy(CMSG_DATA(ec), &ee, sizeof ee);
  EXPECT(!devmem::parseZerocopyNotice(&em, &lo, &hi));
  // completions: out of order, overlapping, across the 2^32 wrap
  devmem::TxCompletions tc;
  for (int i = 0; i < 10; ++i) EXPECT(tc.onSend() == (uint32_t)i);
  tc.onNotice(3, 6);
  EXPECT(tc.done() == 0 && !tc.completed(0, 1) && tc.outstanding() == 10);
  tc.onNotice(0, 3);
  EXPECT(tc.done() == 6 && tc.completed(0, 6) && !tc.completed(5, 2));
  tc.onNotice(4, 8);  // overlaps what is done
  EXPECT(tc.done() == 8 && tc.outstanding() == 2);
  // across the 2^32 wrap of the per-socket sequence numbers
  devmem::TxCompletions w(0xfffffffdu);
  uint32_t ids[6];
  for (int i = 0; i < 6; ++i) ids[i] = w.onSend();
  EXPECT(ids[0] == 0xfffffffdu && ids[3] == 0 && ids[5] == 2);
  w.onNotice(0xffffffffu, 2);            // ids 2^32 - 1, 0, 1: ahead of the frontier
  EXPECT(!w.completed(ids[0], 1) && w.outstanding() == 6);
  w.onNotice(0xfffffffdu, 0xffffffffu);  // the two before them
  EXPECT(w.completed(ids[0], 5) && !w.completed(ids[0], 6) && w.done() == 2 && w.outstanding() == 1);
}

// A model of a devmem socket for the receive loop: bytes come from a real socket, land in
// a "pool" at shuffled pages, and are reported as fragment records with tokens.
struct DevmemModel {
  std::vector<uint8_t> pool;
  std::vector<uint32_t> free_pages;
  std::map<uint32_t, uint32_t> live;  // token -> page
  uint32_t next_token = 100;
  std::vector<uint8_t> bounce;
} *g_model = nullptr;

ssize_t modelRecvmsg(int fd, struct msghdr* msg, int flags) {
  if (!(flags & devmem::kMsgSockDevmem)) { errno = EINVAL; return -1; }
  DevmemModel& m = *g_model;
  const size_t room = msg->msg_controllen / CMSG_SPACE(sizeof(devmem::DmabufCmsg));
  size_t want = std::min<size_t>(msg->msg_iov[0].iov_len, room * 4096);
  want = std::min<size_t>(want, m.free_pages.size() * 4096);
  if (want == 0) { errno = ENOBUFS; return -1; }
  m.bounce.resize(want);
  const ssize_t n = recv(fd, m.bounce.data(), want, MSG_DONTWAIT);
  if (n <= 0) return n;
  size_t used = 0;
  char* c = static_cast<char*>(msg->msg_control);
  for (size_t off = 0; off < (size_t)n; off += 4096) {
    const uint32_t len = (uint32_t)std::min<size_t>(4096, (size_t)n - off);
    const uint32_t page = m.free_pages.back();
    m.free_pages.pop_back();
    memcpy(m.pool.data() + (size_t)page * 4096, m.bounce.data() + off, len);
    const uint32_t tok = m.next_token++;
    m.live[tok] = page;
    devmem::DmabufCmsg f = {(uint64_t)page * 4096, len, tok, 1, 0};
    struct cmsghdr* cm = reinterpret_cast<struct cmsghdr*>(c + used);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = devmem::kSoDevmemDmabuf;
    cm->cmsg_len = CMSG_LEN(sizeof f);
    memcpy(CMSG_DATA(cm), &f, sizeof f);
    used += CMSG_SPACE(sizeof f);
  }
  msg->msg_controllen = used;
  msg->msg_flags = 0;
  return n;
}
int modelSetsockopt(int, int level, int optname, const void* val, socklen_t len) {
  if (level != SOL_SOCKET || optname != devmem::kSoDevmemDontneed) { errno = EINVAL; return -1; }
  const devmem::DmabufToken* t = static_cast<const devmem::DmabufToken*>(val);
  for (size_t i = 0; i < len / sizeof *t; ++i)
    for (uint32_t k = 0; k < t[i].token_count; ++k) {
      auto it = g_model->live.find(t[i].token_start + k);
      if (it == g_model->live.end()) { errno = EINVAL; return -1; }
      g_model->free_pages.push_back(it->second);
      g_model->live.erase(it);
    }
  return 0;
}

TEST(devmem_receive_loop_against_a_kernel_model) {
  int sv[2];
  EXPECT(socketpair(AF_UNIX, SOCK_STREAM, 0, sv) == 0);
  DevmemModel model;
  const uint32_t pages = 512;
  model.pool.assign((size_t)pages * 4096, 0xEE);
  for (uint32_t p = 0; p < pages; ++p) model.free_pages.push_back((p * 197) % pages);  // 197 is coprime to 512: a permutation
  g_model = &model;
  devmem::SocketOps ops = {modelRecvmsg, nullptr, modelSetsockopt};
  const size_t total = 1000000;  // not a multiple of the page size
  std::vector<uint8_t> src(total), dst(total, 0);
  for (size_t i = 0; i < total; ++i) src[i] = (uint8_t)(i * 2654435761u >> 13);
  std::thread sender([&] {
    size_t sent = 0;
    while (sent < total) {
      ssize_t n = send(sv[0], src.data() + sent, std::min<size_t>(70000, total - sent), 0);
      if (n <= 0) break;
      sent += (size_t)n;
    }
  });
  std::vector<LoadMeta> rec(kUnpackMaxSlicePages);
  std::vector<devmem::DmabufToken> runs;
  devmem::RxSink sink;
  sink.records = rec.data(); sink.capacity = rec.size(); sink.tokens = &runs; sink.pool_bytes = model.pool.size(); sink.dmabuf_id = 1;
  std::vector<char> control(devmem::rxControlBytes(64));
  size_t got = 0;
  bool ok = true;
  while (got < total && ok) {
    const ssize_t n = devmem::recvInto(ops, sv[1], total - got, control.data(), control.size(), got, &sink);
    if (n == -EAGAIN) { usleep(100); continue; }
    if (n <= 0) { ok = false; break; }
    got += (size_t)n;
  }
  sender.join();
  EXPECT(ok && got == total);
  // what a consumer does with the list: copy every record out of the pool
  uint64_t covered = 0;
  for (uint64_t i = 0; i < sink.filled; ++i) {
    memcpy(dst.data() + rec[i].dst_off, model.pool.data() + rec[i].src_off, rec[i].len);
    covered += rec[i].len;
  }
  EXPECT(covered == total && dst == src);
  EXPECT(runs.size() == 1 && runs[0].token_count == sink.filled);  // one flow: consecutive tokens, one run
  EXPECT(model.live.size() == sink.filled);
  EXPECT(devmem::recycle(ops, sv[1], &runs) == kSuccess && model.live.empty() && model.free_pages.size() == pages);
  g_model = nullptr;
  close(sv[0]);
  close(sv[1]);
}

// ------------------------------------------------- driver-API services (stand-in device)
TEST(shared_device_allocation_and_dmabuf_export_on_standin_device) {
  if (!cu::available()) { printf("  skipped: no device (set TCPXB_FAKE_GPU=1)\n"); return; }
  EXPECT(cu::deviceInit(0) == kSuccess);
  cu::SharedAllocation owner, client;
  int fd = -1;
  EXPECT(cu::sharedCreate(0, 3 << 20, &owner, &fd) == kSuccess && fd >= 0);
  EXPECT(owner.bytes % cu::sharedGranularity(0) == 0 && owner.bytes >= (3u << 20) && !owner.imported);
  EXPECT(cu::sharedImport(0, fd, owner.bytes, &client) == kSuccess && client.imported);
  close(fd);
  // the two mappings are the same memory
  memset(owner.dptr, 0x5a, 4096);
  EXPECT(static_cast<uint8_t*>(client.dptr)[4095] == 0x5a);
  static_cast<uint8_t*>(client.dptr)[8192] = 0x33;
  EXPECT(static_cast<uint8_t*>(owner.dptr)[8192] == 0x33);
  // a dma-buf of a range inside the allocation: a descriptor plus the range's offset
  int dfd = -1;
  uint64_t off = 0;
  EXPECT(cu::exportDmabuf(static_cast<uint8_t*>(client.dptr) + 12288, 65536, &dfd, &off) == kSuccess && dfd >= 0 && off == 12288);
  if (dfd >= 0) close(dfd);
  EXPECT(cu::exportDmabuf(static_cast<uint8_t*>(client.dptr) + client.bytes - 100, 4096, &dfd, &off) != kSuccess);  // leaves the allocation
  int stack_var = 0;
  EXPECT(cu::exportDmabuf(&stack_var, 4, &dfd, &off) != kSuccess);
  {
    cu::ScopedContext ctx(0);
    EXPECT(ctx.ok());
  }
  cu::sharedRelease(&client);
  cu::sharedRelease(&owner);
  EXPECT(owner.dptr == nullptr && client.dptr == nullptr);
}

TEST(chunk_size_follows_the_sockets) {
  // one chunk per socket and message, page-rounded, never below the striping quantum and
  // never above 4 MiB; ADAPTIVE_CHUNK=0 keeps the fixed quantum
  unsetenv("NCCL_GPUDIRECTTCPX_ADAPTIVE_CHUNK");
  setenv("NCCL_DYNAMIC_CHUNK_SIZE", "131072", 1);
  reloadFlags();
  EXPECT(chunkBytesFor(4 << 20, 1) == 4 << 20);
  EXPECT(chunkBytesFor(4 << 20, 4) == 1 << 20);
  EXPECT(chunkBytesFor(1 << 20, 8) == 131072);          // size / sockets is the quantum itself
  EXPECT(chunkBytesFor(300000, 2) == 151552);           // 150000 rounded up to whole pages
  EXPECT(chunkBytesFor(100000, 4) == 131072);           // small messages: one chunk of at most the quantum
  EXPECT(chunkBytesFor(64 << 20, 2) == kMaxAdaptiveChunk);
  EXPECT(chunkBytesFor(0, 4) == 131072);
  setenv("NCCL_GPUDIRECTTCPX_ADAPTIVE_CHUNK", "0", 1);
  reloadFlags();
  EXPECT(chunkBytesFor(4 << 20, 1) == 131072);
  unsetenv("NCCL_GPUDIRECTTCPX_ADAPTIVE_CHUNK");
  unsetenv("NCCL_DYNAMIC_CHUNK_SIZE");
  reloadFlags();
}

TEST(stream_counter_on_standin_device) {
  if (!gpu::available()) { printf("  skipped: no device (set TCPXB_FAKE_GPU=1)\n"); return; }
  gpu::StreamCounter c;
  EXPECT(c.init() == kSuccess && c.ready() && c.issued() == 0);
  EXPECT(c.reached(0) && !c.reached(1));
  uint32_t a = 0, b = 0;
  EXPECT(c.mark(nullptr, &a) == kSuccess && a == 1);
  EXPECT(c.mark(nullptr, &b) == kSuccess && b == 2 && c.issued() == 2);
  EXPECT(c.reached(1) && c.reached(2) && !c.reached(3));  // the stand-in's streams run everything at once
}

TEST(result_strings_and_handle_layout) {
  EXPECT(std::string(resultString(kSuccess)) == "success" && std::string(resultString(kRemoteError)) == "remote error");
  EXPECT(sizeof(Handle) <= 128 && sizeof(CtrlMsg) == 16 && sizeof(LoadMeta) == 16);
  EXPECT(sizeof(SocketAddress) == sizeof(struct sockaddr_in6));
}

}  // namespace

int main(int argc, char** argv) {
  const char* filter = argc > 1 ? argv[1] : "";
  int ran = 0;
  for (const Test& t : tests()) {
    if (*filter && strstr(t.name, filter) == nullptr) continue;
    g_current_ok = true;
    t.fn();
    printf("%s %s\n", g_current_ok ? "ok" : "FAIL", t.name);
    fflush(stdout);
    if (!g_current_ok) ++g_failures;
    ++ran;
  }
  printf("%d test(s), %d failure(s)\n", ran, g_failures);
  return g_failures == 0 && ran > 0 ? 0 : 1;
}
