// Hierarchical collective engine; see tcpxb/engine.h for the algorithms.
#include "tcpxb/engine.h"

#include <poll.h>
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/eventfd.h>
#include <sys/prctl.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#ifndef TCPXB_NO_CUDA
#include <nvtx3/nvToolsExt.h>
#endif

#include "tcpxb/kernels.h"
#include "tcpxb/transport.h"

using namespace tcpxb;

namespace {

thread_local char g_err[512] = "";
int fail(const char* fmt, const char* a = "", long b = 0) {
  snprintf(g_err, sizeof g_err, fmt, a, b);
  return -1;
}
#define ENG_NET(expr)                                                           \
  do {                                                                          \
    Result r_ = (expr);                                                         \
    if (r_ != kSuccess) return fail("%s -> %ld", #expr, (long)r_);              \
  } while (0)
#define ENG_K(expr)                                                             \
  do {                                                                          \
    ++e->stats.kernel_launches;                                                 \
    if ((expr) != 0) {                                                          \
      snprintf(g_err, sizeof g_err, "%s: %s", #expr, tcpxb_kernel_last_error()); \
      return -1;                                                                \
    }                                                                           \
  } while (0)
#define ENG_TRY(expr)                                                           \
  do {                                                                          \
    if ((expr) != 0) return -1;                                                 \
  } while (0)

double nowSec() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}

// NVTX range for the lifetime of a scope; costs nothing unless a tool is attached.
#ifndef TCPXB_NO_CUDA
struct Range {
  explicit Range(const char* name) { nvtxRangePushA(name); }
  ~Range() { nvtxRangePop(); }
};
#else
struct Range {
  explicit Range(const char*) {}
  ~Range() {}
};
#endif

struct Rail {
  ListenComm* listen = nullptr;
  Comm* send = nullptr;
  Comm* recv = nullptr;
};

// What to do with the bytes that arrive in one exchange.
struct RecvSpec {
  uint64_t bytes = 0;
  uint8_t* dst = nullptr;        // local destination of the region
  const uint8_t* acc = nullptr;  // addend region; null = plain copy
  int dtype = TCPXB_U8;
  bool fanout = false;           // also store into the local peers' output buffers
  uint64_t out_offset = 0;       // offset of `dst` inside the output buffer (for the peer addresses)
  bool last = false;             // the final kernel publishes the fan-out flags
};
struct SendSpec {
  uint64_t bytes = 0;
  const uint8_t* src = nullptr;
};

struct PendingUnpack {
  Request* req;
  uint32_t mark;  // value of the engine's stream counter once the request's kernel has finished
};

struct Engine {
  tcpxbEngineConfig cfg;
  int nodes = 1, node = 0, local = 0, G = 1;
  bool twin = false;  // world == 1: the rank is its own network peer
  std::vector<Rail> rails;
  bool connected = false;
  // intra-node mappings
  std::vector<uint8_t*> work, out;
  std::vector<uint32_t*> flags;
  uint8_t* mc_out = nullptr;
  uint64_t buffer_bytes = 0;
  uint32_t epoch = 0;
  // device scratch
  uint8_t* scratch = nullptr;
  uint64_t scratch_bytes = 0;
  uint32_t* ticket = nullptr;       // fan-out completion counter (device)
  uint32_t* status_host = nullptr;  // kernel status block (pinned, device-mapped)
  uint32_t* status_dev = nullptr;
  gpu::StreamCounter kernel_marks;  // advanced on the caller's stream behind every unpack launch
  gpu::Event dep_event = nullptr;
  tcpxbEngineStats stats;
  int req_bytes = 1 << 20, inflight = 4, ctas = 16;
  bool yield_when_idle = false;
  // idle policy of the driving thread
  Notifier notifier;
  int idle_spin_us = 20, idle_sleep_us = 30;
  bool wake_on_events = false;  // sleep in ppoll on the control sockets and an eventfd instead of napping
  // asynchronous calls: jobs run in order on a thread and a stream of the engine's own
  struct Job {
    uint64_t ticket = 0;
    std::function<int(void* stream)> run;
    gpu::Event after = nullptr;  // the engine's stream waits for this before the job (caller's event, may be null)
    gpu::Event done = nullptr;   // recorded on the engine's stream behind the job's last kernel
    int rc = 0;
    bool finished = false;
    std::string error;
  };
  std::thread worker;
  std::mutex job_mu;
  std::condition_variable job_cv;
  std::deque<Job*> job_queue;
  std::map<uint64_t, Job*> jobs;  // every job not yet released, by ticket
  uint64_t next_ticket = 0;
  bool worker_stop = false;
  gpu::Stream async_stream = nullptr;
};

constexpr double kSmallExchangeSpinUs = 250.0;

// One look at every receive comm's control socket: a single poll() with no wait, then a
// hint to the comms whose socket has data.  Replaces one recv() attempt per comm and
// progress round.
void pollCtrlSockets(Engine* e) {
  struct pollfd pfds[TCPXB_ENGINE_MAX_RAILS];
  Comm* owner[TCPXB_ENGINE_MAX_RAILS];
  int n = 0;
  for (Rail& r : e->rails) {
    const int fd = netCtrlPollFd(r.recv);
    if (fd >= 0) { pfds[n] = {fd, POLLIN, 0}; owner[n] = r.recv; ++n; }
  }
  if (n == 0 || poll(pfds, (nfds_t)n, 0) <= 0) return;
  for (int i = 0; i < n; ++i)
    if (pfds[i].revents & (POLLIN | POLLHUP | POLLERR)) netHintCtrlReadable(owner[i]);
}

// Blocks the driving thread until a helper thread finishes a task, a control record
// arrives, or `timeout_us` passes (GPU events have no descriptor: the timeout bounds
// how late their completion is noticed).
void sleepUntilWork(Engine* e, bool want_ctrl, int timeout_us) {
  struct pollfd pfds[1 + TCPXB_ENGINE_MAX_RAILS];
  Comm* owner[1 + TCPXB_ENGINE_MAX_RAILS] = {};
  int n = 0;
  pfds[n++] = {e->notifier.event_fd, POLLIN, 0};
  if (want_ctrl) {
    for (Rail& r : e->rails) {
      const int fd = netCtrlPollFd(r.recv);
      if (fd >= 0) { pfds[n] = {fd, POLLIN, 0}; owner[n] = r.recv; ++n; }
    }
  }
  struct timespec ts = {0, (long)timeout_us * 1000};
  const int rc = ppoll(pfds, (nfds_t)n, &ts, nullptr);
  e->notifier.armed.store(0, std::memory_order_release);
  for (int i = 1; i < n && rc > 0; ++i)
    if (pfds[i].revents & (POLLIN | POLLHUP | POLLERR)) netHintCtrlReadable(owner[i]);
  if (rc > 0 && (pfds[0].revents & POLLIN)) {
    uint64_t v;
    ssize_t got = read(e->notifier.event_fd, &v, sizeof v);
    (void)got;
  }
  ++e->stats.sleeps;
}

int ensureScratch(Engine* e, uint64_t bytes) {
  if (e->scratch_bytes >= bytes) return 0;
  gpu::deviceFree(e->scratch);
  e->scratch = nullptr;
  void* p = nullptr;
  ENG_NET(gpu::deviceAlloc(bytes, &p));
  e->scratch = static_cast<uint8_t*>(p);
  e->scratch_bytes = bytes;
  return 0;
}

// The kernels report into a pinned status block; a non-zero first word means a
// record was skipped or a bounded wait ran out, and the collective's result is not
// to be trusted.  Checked whenever the host learns that kernels have finished.
int checkDeviceStatus(Engine* e) {
  const uint32_t code = e->status_host[0];
  if (code == 0) return 0;
  snprintf(g_err, sizeof g_err, "device status %u (%s) at record %u, %u report(s)", code,
           code == TCPXB_ST_BOUNDS ? "record out of bounds" : code == TCPXB_ST_ALIGN ? "misaligned reduce record"
           : code == TCPXB_ST_TIMEOUT ? "a bounded device wait ran out" : "unknown",
           e->status_host[1], e->status_host[2]);
  return -1;
}

// Launches the unpack kernel for one finished receive request.
int launchUnpack(Engine* e, Request* req, const RecvSpec& rs, uint64_t region_off, uint64_t len, bool publish,
                 void* stream) {
  ScatterList sl;
  ENG_NET(netRequestScatterList(req, &sl));
  e->stats.fragments += sl.count;
  ++e->stats.unpack_launches;
  tcpxbUnpackOpts opts;
  memset(&opts, 0, sizeof opts);
  opts.max_ctas = e->ctas;
  uint8_t* dst = rs.dst + region_off;
  const uint8_t* acc = rs.acc ? rs.acc + region_off : nullptr;
  const tcpxbLoadMeta* descs = reinterpret_cast<const tcpxbLoadMeta*>(sl.dev);
  const uint32_t count = (uint32_t)sl.count;
  void* peers[TCPXB_MAX_PEERS];
  int npeers = 0;
  const bool fan = rs.fanout && e->G > 1;
  if (fan) {
    for (int l = 0; l < e->G; ++l) {
      if (l == e->local) continue;
      peers[npeers] = e->out[l] + rs.out_offset + region_off;
      if (publish) opts.peer_flags[npeers] = e->flags[l] + 32 + e->local;  // block B, my slot
      ++npeers;
    }
    if (publish) {
      opts.flag_value = e->epoch;
      opts.ticket = e->ticket;
    }
  }
  if (e->cfg.plain_mode) {
    // Baseline: unpack to a bounce buffer, add in a second pass, copy to the peers.
    // the last req_bytes of the scratch are the bounce buffer of the two-pass reduce
    uint8_t* bounce = nullptr;
    if (acc != nullptr) {
      ENG_TRY(ensureScratch(e, std::max<uint64_t>(e->scratch_bytes, (uint64_t)e->req_bytes)));
      if (e->scratch == nullptr) return fail("no scratch for the unfused reduce%s", "");
      bounce = e->scratch + e->scratch_bytes - (uint64_t)e->req_bytes;
    }
    // the unpack kernel must not publish completion here: the add and the peer copies come after it
    tcpxbUnpackOpts copy_opts;
    memset(&copy_opts, 0, sizeof copy_opts);
    copy_opts.max_ctas = opts.max_ctas;
    ENG_K(tcpxb_unpack_copy(sl.pool_dev, sl.pool_bytes, acc ? bounce : dst, len, descs, count, e->status_dev, &copy_opts, stream));
    if (acc) {
      void* srcs[2] = {const_cast<uint8_t*>(acc), bounce};
      ENG_K(tcpxb_peer_reduce(dst, srcs, 2, 0, len & ~15ull, rs.dtype, stream));
    }
    for (int i = 0; i < npeers; ++i) ENG_NET(gpu::copyDeviceToDeviceAsync(peers[i], dst, len, stream));
    if (fan && publish) {
      uint32_t* pf[TCPXB_MAX_PEERS];
      for (int i = 0; i < npeers; ++i) pf[i] = opts.peer_flags[i];
      ENG_K(tcpxb_signal_flags(pf, npeers, e->epoch, stream));
    }
    return 0;
  }
  const bool nvls = fan && e->cfg.use_nvls && e->mc_out != nullptr;
  if (acc == nullptr) {
    if (!fan) ENG_K(tcpxb_unpack_copy(sl.pool_dev, sl.pool_bytes, dst, len, descs, count, e->status_dev, &opts, stream));
    else if (nvls)
      ENG_K(tcpxb_unpack_fanout_nvls(sl.pool_dev, sl.pool_bytes, dst, e->mc_out + rs.out_offset + region_off, len, peers,
                                     npeers, descs, count, e->status_dev, &opts, stream));
    else
      ENG_K(tcpxb_unpack_fanout(sl.pool_dev, sl.pool_bytes, dst, len, peers, npeers, descs, count, e->status_dev, &opts, stream));
  } else {
    if (!fan)
      ENG_K(tcpxb_unpack_reduce(sl.pool_dev, sl.pool_bytes, acc, dst, len, descs, count, rs.dtype,
                                acc == dst ? e->cfg.reduce_impl : TCPXB_REDUCE_SM, e->status_dev, &opts, stream));
    else if (nvls)
      ENG_K(tcpxb_unpack_reduce_fanout_nvls(sl.pool_dev, sl.pool_bytes, acc, dst, e->mc_out + rs.out_offset + region_off, len,
                                            peers, npeers, descs, count, rs.dtype, e->status_dev, &opts, stream));
    else
      ENG_K(tcpxb_unpack_reduce_fanout(sl.pool_dev, sl.pool_bytes, acc, dst, len, peers, npeers, descs, count, rs.dtype,
                                       TCPXB_REDUCE_SM, e->status_dev, &opts, stream));
  }
  return 0;
}

// One simultaneous send + receive with the ring neighbours, in requests of
// req_bytes striped over the rails.  Request k of a direction uses rail k % rails
// on both ends, so the two sides agree without talking about it.
int exchange(Engine* e, const SendSpec& ss, const RecvSpec& rs, void* stream) {
  Range range("tcpxb exchange");
  const int R = (int)e->rails.size();
  const uint64_t rb = (uint64_t)e->req_bytes;
  const uint64_t n_send = (ss.bytes + rb - 1) / rb, n_recv = (rs.bytes + rb - 1) / rb;
  uint64_t post_s = 0, post_r = 0, done_s = 0, launched_r = 0;
  std::vector<std::deque<Request*>> sq(R), rq(R);
  std::vector<std::deque<uint64_t>> rq_idx(R);
  std::vector<std::deque<PendingUnpack>> uq(R);
  if (ss.bytes > 0) {
    // sends may read only what the stream has produced so far
    ENG_NET(gpu::eventRecord(e->dep_event, stream));
    for (int r = 0; r < R; ++r) netSetSendDependency(e->rails[r].send, e->dep_event);
  }
  MemHandle send_mh{const_cast<uint8_t*>(ss.src), ss.bytes, kPtrCuda, e->cfg.gpu_dev};
  MemHandle recv_mh{rs.dst, rs.bytes, kPtrCuda, e->cfg.gpu_dev};
  const double t0 = nowSec();
  double tp = t0;
  auto lap = [&tp](double& acc) { const double n = nowSec(); acc += n - tp; tp = n; };
  double idle_since = 0;
  bool armed = false;
  // Small exchanges are latency-bound: spin a little before sleeping.  Large ones have
  // requests queued on every rail, and every microsecond of spinning is taken from the
  // helper threads when cores are scarce: sleep at once.
  // A small exchange is over in one round trip of the sockets, some tens of microseconds: a nap (which
  // lasts 50 us and more once the timer and the scheduler are through) would double its time, so the
  // driving thread spins through it.
  const double spin_us = (ss.bytes + rs.bytes <= (1u << 20)) ? std::max((double)e->idle_spin_us, kSmallExchangeSpinUs) : 0.0;
  while (done_s < n_send || launched_r < n_recv) {
    bool moved = false;
    if (launched_r < n_recv) pollCtrlSockets(e);  // which control sockets have records: one system call for all rails
    // post receives (they claim pool pages as control records arrive)
    while (post_r < n_recv) {
      const int r = (int)(post_r % R);
      // Requests whose kernel is queued no longer need the network: they do not count
      // against the window, so that receiving goes on while kernels run.  They still
      // hold pool pages and a scatter-list slot each, hence the second bound.
      if ((int)rq[r].size() >= e->inflight || (int)(rq[r].size() + uq[r].size()) >= 2 * e->inflight) break;
      const uint64_t off = post_r * rb;
      void* data = rs.dst + off;
      int sz = (int)std::min<uint64_t>(rb, rs.bytes - off), tag = 0;
      MemHandle* mh = &recv_mh;
      Request* req = nullptr;
      ENG_NET(netIrecv(e->rails[r].recv, 1, &data, &sz, &tag, &mh, &req));
      if (req == nullptr) break;
      rq[r].push_back(req);
      rq_idx[r].push_back(post_r);
      ++post_r;
      moved = true;
    }
    lap(e->stats.t_post_recv);
    while (post_s < n_send) {
      const int r = (int)(post_s % R);
      if ((int)sq[r].size() >= e->inflight) break;
      const uint64_t off = post_s * rb;
      const int sz = (int)std::min<uint64_t>(rb, ss.bytes - off);
      Request* req = nullptr;
      ENG_NET(netIsend(e->rails[r].send, const_cast<uint8_t*>(ss.src) + off, sz, 0, &send_mh, &req));
      if (req == nullptr) break;
      sq[r].push_back(req);
      ++post_s;
      moved = true;
    }
    lap(e->stats.t_post_send);
    for (int r = 0; r < R; ++r) {
      while (!rq[r].empty()) {
        int done = 0, sz = 0;
        ENG_NET(netTest(rq[r].front(), &done, &sz));
        if (!done) break;
        const uint64_t k = rq_idx[r].front();
        const uint64_t off = k * rb;
        const uint64_t want = std::min<uint64_t>(rb, rs.bytes - off);
        if ((uint64_t)sz != want) return fail("received %s bytes short: request size %ld", "", (long)sz);
        // Whichever request is launched last runs last on the stream, so it is the
        // one that publishes completion.
        const bool publish = rs.last && (launched_r + 1 == n_recv);
        lap(e->stats.t_test_recv);
        ENG_TRY(launchUnpack(e, rq[r].front(), rs, off, want, publish, stream));
        uint32_t done_mark = 0;
        ENG_NET(e->kernel_marks.mark(stream, &done_mark));
        uq[r].push_back({rq[r].front(), done_mark});
        rq[r].pop_front();
        rq_idx[r].pop_front();
        ++launched_r;
        ++e->stats.requests;
        e->stats.bytes_received += want;
        moved = true;
        lap(e->stats.t_launch);
      }
      lap(e->stats.t_test_recv);
      while (!uq[r].empty()) {
        if (!e->kernel_marks.reached(uq[r].front().mark)) break;
        ENG_TRY(checkDeviceStatus(e));
        ENG_NET(netIrecvConsumed(e->rails[r].recv, 1, uq[r].front().req));
        uq[r].pop_front();
        moved = true;
      }
      lap(e->stats.t_consume);
      while (!sq[r].empty()) {
        int done = 0, sz = 0;
        ENG_NET(netTest(sq[r].front(), &done, &sz));
        if (!done) break;
        e->stats.bytes_sent += (uint64_t)sz;
        sq[r].pop_front();
        ++done_s;
        moved = true;
      }
      lap(e->stats.t_test_send);
    }
    if (moved) {
      idle_since = 0;
      if (armed) { e->notifier.armed.store(0, std::memory_order_release); armed = false; }
      continue;
    }
    // Nothing moved.  Spin briefly (the next event is usually microseconds away when
    // messages are small), then sleep: on a box where helper threads outnumber the
    // cores, a spinning driver takes a core away from the threads that move the bytes.
    if (idle_since == 0) idle_since = tp;
    const bool may_sleep = e->idle_sleep_us > 0;
    if (!may_sleep || (tp - idle_since) * 1e6 < spin_us) {
      if (e->yield_when_idle) sched_yield();
      else for (int i = 0; i < 64; ++i) __builtin_ia32_pause();
      lap(e->stats.t_idle);
    } else if (!e->wake_on_events) {
      // Nap: a fixed short sleep that nobody has to end.  With several requests queued on
      // every rail, looking again after a few tens of microseconds loses nothing, and the
      // helper threads never pay a system call to wake this thread.
      struct timespec ts = {0, (long)e->idle_sleep_us * 1000};
      nanosleep(&ts, nullptr);
      ++e->stats.sleeps;
      lap(e->stats.t_sleep);
    } else if (!armed) {
      // arm, then look once more: a completion between the last look and the arming is not lost
      e->notifier.armed.store(1, std::memory_order_seq_cst);
      armed = true;
    } else {
      // kernels or staging copies in flight complete without a wake-up: look again sooner
      bool gpu_pending = false;
      for (int r = 0; r < R; ++r) gpu_pending = gpu_pending || !uq[r].empty();
      sleepUntilWork(e, launched_r < n_recv, gpu_pending ? std::min(e->idle_sleep_us, 50) : e->idle_sleep_us);
      armed = false;
      lap(e->stats.t_sleep);
    }
  }
  if (armed) e->notifier.armed.store(0, std::memory_order_release);
  // pool pages go back once the kernels that read them have finished
  bool any_left = false;
  for (int r = 0; r < R; ++r) any_left = any_left || !uq[r].empty();
  if (any_left) ENG_NET(gpu::streamSynchronize(stream));
  for (int r = 0; r < R; ++r) {
    while (!uq[r].empty()) {
      if (!e->kernel_marks.reached(uq[r].front().mark)) return fail("unpack completion mark missing after a stream synchronize%s", "");
      ENG_NET(netIrecvConsumed(e->rails[r].recv, 1, uq[r].front().req));
      uq[r].pop_front();
    }
  }
  e->stats.seconds_net_wait += nowSec() - t0;
  ENG_TRY(checkDeviceStatus(e));  // every unpack kernel of this exchange has finished
  return 0;
}

int checkReady(Engine* e) {
  if (e == nullptr) return fail("null engine%s", "");
  if (!e->connected) return fail("engine is not connected%s", "");
  if (e->G > 1 && e->out.empty()) return fail("set_peers was not called%s", "");
  ENG_NET(gpu::setDevice(e->cfg.gpu_dev));
  // an earlier call's last kernels (e.g. its final flag wait) may have failed after it returned
  return checkDeviceStatus(e);
}

// "Inputs staged" barrier among the local GPUs: block A of the flag pages.
int barrierInputs(Engine* e, void* stream) {
  if (e->G <= 1) return 0;
  uint32_t* pf[TCPXB_MAX_PEERS + 1];
  int n = 0;
  for (int l = 0; l < e->G; ++l) pf[n++] = e->flags[l] + e->local;  // my slot in everybody's block A
  ENG_K(tcpxb_signal_flags(pf, n, e->epoch, stream));
  ENG_K(tcpxb_wait_flags(e->flags[e->local], e->G, e->epoch, 0, e->status_dev, stream));
  return 0;
}

// Waits until every local peer has finished storing into this GPU's output.
int waitFanout(Engine* e, void* stream) {
  if (e->G <= 1) return 0;
  // my own slot of block B is written here, the peers' slots by their last kernel
  uint32_t* own[1] = {e->flags[e->local] + 32 + e->local};
  ENG_K(tcpxb_signal_flags(own, 1, e->epoch, stream));
  ENG_K(tcpxb_wait_flags(e->flags[e->local] + 32, e->G, e->epoch, 0, e->status_dev, stream));
  return 0;
}

// ---- worker thread of the asynchronous calls

void workerMain(Engine* e) {
  prctl(PR_SET_NAME, "tcpxb-engine", 0, 0, 0);
  prctl(PR_SET_TIMERSLACK, 1, 0, 0, 0);
  gpu::setDevice(e->cfg.gpu_dev);
  for (;;) {
    Engine::Job* job = nullptr;
    {
      std::unique_lock<std::mutex> l(e->job_mu);
      e->job_cv.wait(l, [e] { return e->worker_stop || !e->job_queue.empty(); });
      if (e->job_queue.empty()) return;  // stop requested and nothing left
      job = e->job_queue.front();
      e->job_queue.pop_front();
    }
    int rc = 0;
    if (job->after != nullptr && gpu::streamWaitEvent(e->async_stream, job->after) != kSuccess) rc = fail("waiting for the caller's event failed%s", "");
    if (rc == 0) rc = job->run(e->async_stream);
    if (rc == 0 && gpu::eventRecord(job->done, e->async_stream) != kSuccess) rc = fail("recording the completion event failed%s", "");
    {
      std::lock_guard<std::mutex> l(e->job_mu);
      job->rc = rc;
      if (rc != 0) job->error = g_err;  // g_err belongs to this thread: hand the text over
      job->finished = true;
    }
    e->job_cv.notify_all();
  }
}

uint64_t submit(Engine* e, std::function<int(void*)> fn, void* after_event) {
  std::lock_guard<std::mutex> l(e->job_mu);
  if (e->async_stream == nullptr) {
    if (gpu::setDevice(e->cfg.gpu_dev) != kSuccess || gpu::streamCreate(&e->async_stream) != kSuccess) { fail("engine stream: %s", gpu::lastError()); return 0; }
    e->worker = std::thread(workerMain, e);
  }
  auto* job = new Engine::Job();
  if (gpu::eventCreate(&job->done) != kSuccess) { delete job; fail("event: %s", gpu::lastError()); return 0; }
  job->ticket = ++e->next_ticket;
  job->run = std::move(fn);
  job->after = after_event;
  e->jobs[job->ticket] = job;
  e->job_queue.push_back(job);
  e->job_cv.notify_all();
  return job->ticket;
}

void stopWorker(Engine* e) {
  {
    std::lock_guard<std::mutex> l(e->job_mu);
    e->worker_stop = true;
  }
  e->job_cv.notify_all();
  if (e->worker.joinable()) e->worker.join();
  for (auto& kv : e->jobs) { gpu::eventDestroy(kv.second->done); delete kv.second; }
  e->jobs.clear();
  gpu::streamDestroy(e->async_stream);
  e->async_stream = nullptr;
}


}  // namespace

extern "C" {

const char* tcpxb_engine_last_error(void) { return g_err; }

void* tcpxb_engine_create(const tcpxbEngineConfig* cfg) {
  if (cfg == nullptr || cfg->world < 1 || cfg->rank < 0 || cfg->rank >= cfg->world || cfg->gpus_per_node < 1 ||
      cfg->world % cfg->gpus_per_node != 0 || cfg->gpus_per_node > TCPXB_MAX_PEERS) {
    fail("bad engine configuration%s", "");
    return nullptr;
  }
  if (cfg->world > 1 && cfg->world / cfg->gpus_per_node < 2) {
    fail("the engine needs at least two emulated nodes%s", "");
    return nullptr;
  }
  if (netInit(nullptr) != kSuccess) { fail("transport init failed%s", ""); return nullptr; }
  if (!gpu::available() || gpu::setDevice(cfg->gpu_dev) != kSuccess) { fail("CUDA device unavailable%s", ""); return nullptr; }
  Engine* e = new Engine();
  e->cfg = *cfg;
  e->G = cfg->gpus_per_node;
  e->nodes = cfg->world / e->G;
  e->node = cfg->rank / e->G;
  e->local = cfg->rank % e->G;
  if (cfg->world == 1) { e->twin = true; e->nodes = 2; }
  if (cfg->request_bytes > 0) e->req_bytes = std::min(cfg->request_bytes, 4 << 20) / 4096 * 4096;
  if (e->req_bytes < 4096) e->req_bytes = 4096;
  if (cfg->max_inflight > 0) e->inflight = std::min(cfg->max_inflight, 12);
  if (cfg->unpack_ctas > 0) e->ctas = cfg->unpack_ctas;
  memset(&e->stats, 0, sizeof e->stats);
  e->yield_when_idle = getenv("TCPXB_ENGINE_YIELD") != nullptr;
  if (cfg->idle_spin_us > 0) e->idle_spin_us = cfg->idle_spin_us;
  if (cfg->idle_sleep_us != 0) e->idle_sleep_us = cfg->idle_sleep_us;
  e->wake_on_events = cfg->wake_on_events != 0;
  if (e->wake_on_events) e->notifier.event_fd = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  prctl(PR_SET_TIMERSLACK, 1, 0, 0, 0);  // naps are tens of microseconds: no 50 us default slack on this thread
  int ndev = 0;
  netDevices(&ndev);
  e->rails.resize((size_t)std::min(ndev, TCPXB_ENGINE_MAX_RAILS));
  void* h = nullptr;
  void* d = nullptr;
  void* t = nullptr;
  if (gpu::hostAllocMapped(64, &h, &d) != kSuccess || gpu::deviceAlloc(64, &t) != kSuccess ||
      gpu::memsetAsync(t, 0, 64, nullptr) != kSuccess || gpu::streamSynchronize(nullptr) != kSuccess ||
      gpu::eventCreate(&e->dep_event) != kSuccess || e->kernel_marks.init() != kSuccess) {
    fail("engine device allocations failed: %s", gpu::lastError());
    delete e;
    return nullptr;
  }
  memset(h, 0, 64);
  e->status_host = static_cast<uint32_t*>(h);
  e->status_dev = static_cast<uint32_t*>(d);
  e->ticket = static_cast<uint32_t*>(t);
  return e;
}

void tcpxb_engine_destroy(void* engine) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr) return;
  stopWorker(e);
  for (Rail& r : e->rails) {
    if (r.send) netClose(r.send);
    if (r.recv) netClose(r.recv);
    if (r.listen) netCloseListen(r.listen);
  }
  if (e->notifier.event_fd >= 0) close(e->notifier.event_fd);
  gpu::eventDestroy(e->dep_event);
  gpu::deviceFree(e->scratch);
  gpu::deviceFree(e->ticket);
  gpu::hostFreeMapped(e->status_host);
  delete e;
}

int tcpxb_engine_rails(void* engine) { return engine ? (int)static_cast<Engine*>(engine)->rails.size() : 0; }

int tcpxb_engine_listen(void* engine, void* handles_out) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr || handles_out == nullptr) return fail("null argument%s", "");
  ENG_NET(gpu::setDevice(e->cfg.gpu_dev));
  char* out = static_cast<char*>(handles_out);
  for (size_t r = 0; r < e->rails.size(); ++r) {
    memset(out + r * TCPXB_ENGINE_HANDLE_BYTES, 0, TCPXB_ENGINE_HANDLE_BYTES);
    ENG_NET(netListen((int)r, out + r * TCPXB_ENGINE_HANDLE_BYTES, &e->rails[r].listen));
    netSetAcceptRecvMode(e->rails[r].listen, kRecvModeUnpack);
  }
  return 0;
}

int tcpxb_engine_connect(void* engine, const void* next_handles) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr || next_handles == nullptr) return fail("null argument%s", "");
  ENG_NET(gpu::setDevice(e->cfg.gpu_dev));
  std::vector<char> handles(e->rails.size() * TCPXB_ENGINE_HANDLE_BYTES);
  memcpy(handles.data(), next_handles, handles.size());
  const double deadline = nowSec() + 60.0;
  for (;;) {
    bool all = true;
    for (size_t r = 0; r < e->rails.size(); ++r) {
      Rail& rail = e->rails[r];
      if (rail.send == nullptr) ENG_NET(netConnect((int)r, handles.data() + r * TCPXB_ENGINE_HANDLE_BYTES, &rail.send));
      if (rail.recv == nullptr) ENG_NET(netAccept(rail.listen, &rail.recv));
      all = all && rail.send != nullptr && rail.recv != nullptr;
    }
    if (all) break;
    if (nowSec() > deadline) return fail("connection setup timed out%s", "");
    sched_yield();
  }
  for (Rail& rail : e->rails) {
    // staging no larger than what can be in flight: a small ring stays cache-resident
    const uint64_t want = (uint64_t)(e->inflight + 1) * (uint64_t)e->req_bytes;
    netSetTxStagingBytes(rail.send, std::min<uint64_t>(want, (uint64_t)flags().tx_staging_bytes));
    ENG_NET(netPrepareCuda(rail.send, e->cfg.gpu_dev));
    ENG_NET(netPrepareCuda(rail.recv, e->cfg.gpu_dev));
    // a handful of busy comms per process: napping helpers beat a futex call per task
    if (flags().helper_nap_us == 0) {
      netSetHelperNap(rail.send, 20, 50);
      netSetHelperNap(rail.recv, 20, 50);
    }
    if (e->wake_on_events) {
      netSetNotifier(rail.send, &e->notifier);
      netSetNotifier(rail.recv, &e->notifier);
    }
  }
  e->connected = true;
  return 0;
}

int tcpxb_engine_set_peers(void* engine, void* const* work_ptrs, void* const* out_ptrs, uint32_t* const* flag_ptrs,
                           void* mc_out, uint64_t buffer_bytes) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr || work_ptrs == nullptr || out_ptrs == nullptr || flag_ptrs == nullptr) return fail("null argument%s", "");
  e->work.clear(); e->out.clear(); e->flags.clear();
  for (int l = 0; l < e->G; ++l) {
    if (work_ptrs[l] == nullptr || out_ptrs[l] == nullptr || flag_ptrs[l] == nullptr) return fail("null peer mapping%s", "");
    e->work.push_back(static_cast<uint8_t*>(work_ptrs[l]));
    e->out.push_back(static_cast<uint8_t*>(out_ptrs[l]));
    e->flags.push_back(flag_ptrs[l]);
  }
  e->mc_out = static_cast<uint8_t*>(mc_out);
  e->buffer_bytes = buffer_bytes;
  return 0;
}

int tcpxb_engine_all_reduce(void* engine, const void* in_, void* out_, uint64_t bytes, int dtype, void* stream) {
  Range range("tcpxb all_reduce");
  Engine* e = static_cast<Engine*>(engine);
  ENG_TRY(checkReady(e));
  if (dtype != TCPXB_BF16 && dtype != TCPXB_F32) return fail("all_reduce needs bf16 or f32%s", "");
  const uint64_t unit = (uint64_t)e->G * (uint64_t)(e->nodes > 2 ? e->nodes : 1) * 16;
  if (bytes == 0 || bytes % unit != 0) return fail("all_reduce size must be a multiple of %s%ld bytes", "", (long)unit);
  const uint8_t* in = static_cast<const uint8_t*>(in_);
  uint8_t* out = static_cast<uint8_t*>(out_);
  if (e->G > 1 && bytes > e->buffer_bytes) return fail("all_reduce of %s%ld bytes does not fit the symmetric buffers", "", (long)bytes);
  // Several GPUs per node: peers read the input and write the output through the
  // symmetric buffers.  Tensors that live elsewhere are staged in and out by device
  // copies on the caller's stream.  The previous call ended with every local peer's
  // fan-out signal, which those peers sent after their last read of this GPU's work
  // buffer, so the buffer is free to overwrite here.
  uint8_t* user_out = nullptr;
  if (e->G > 1 && in != e->work[e->local]) {
    ENG_NET(gpu::copyDeviceToDeviceAsync(e->work[e->local], in, bytes, stream));
    in = e->work[e->local];
  }
  if (e->G > 1 && out != e->out[e->local]) {
    user_out = out;
    out = e->out[e->local];
  }
  ++e->epoch;
  const uint64_t shard = bytes / (uint64_t)e->G;
  const uint64_t shard_off = shard * (uint64_t)e->local;
  // 1. intra-node reduce-scatter into `red`
  const uint8_t* red = in;
  if (e->G > 1) {
    ENG_TRY(ensureScratch(e, shard + (uint64_t)e->req_bytes));
    ENG_TRY(barrierInputs(e, stream));
    std::vector<void*> srcs;
    for (int l = 0; l < e->G; ++l) srcs.push_back(e->work[l]);
    ENG_K(tcpxb_peer_reduce(e->scratch, srcs.data(), e->G, shard_off, shard, dtype, stream));
    red = e->scratch;
  } else if (e->nodes == 2 && in == out) {
    // In place between two nodes: shards are swapped request by request, and a request
    // summed into `out` would overwrite input that a later request has yet to send.
    // Sends and addends therefore come from a copy of the input.
    ENG_TRY(ensureScratch(e, bytes + (uint64_t)e->req_bytes));
    ENG_NET(gpu::copyDeviceToDeviceAsync(e->scratch, in, bytes, stream));
    red = e->scratch;
  } else if (e->cfg.plain_mode) {
    ENG_TRY(ensureScratch(e, (uint64_t)e->req_bytes));
  }
  uint8_t* out_shard = out + shard_off;
  if (e->nodes == 2) {
    // 2a. two nodes: swap whole shards, add on arrival, fan out
    SendSpec ss{shard, red};
    RecvSpec rs;
    rs.bytes = shard; rs.dst = out_shard; rs.acc = red; rs.dtype = dtype; rs.fanout = true; rs.out_offset = shard_off; rs.last = true;
    ENG_TRY(exchange(e, ss, rs, stream));
  } else {
    // 2b. ring over the nodes on this rail.  Pieces of the shard; piece p ends up
    // fully reduced on node (p - 1) mod nodes after the reduce-scatter half.
    const int N = e->nodes;
    const uint64_t piece = shard / (uint64_t)N;
    // the running sums live in scratch (G > 1) or in a copy of the input (G == 1)
    uint8_t* acc;
    if (e->G > 1) {
      acc = e->scratch;
    } else {
      ENG_TRY(ensureScratch(e, shard + (uint64_t)e->req_bytes));
      ENG_NET(gpu::copyDeviceToDeviceAsync(e->scratch, in, shard, stream));
      acc = e->scratch;
    }
    auto mod = [N](int x) { return ((x % N) + N) % N; };
    for (int s = 0; s < N - 1; ++s) {
      const int sp = mod(e->node - s), rp = mod(e->node - s - 1);
      SendSpec ss{piece, acc + (uint64_t)sp * piece};
      RecvSpec rs;
      rs.bytes = piece; rs.dtype = dtype; rs.acc = acc + (uint64_t)rp * piece;
      if (s == N - 2) {  // final sum of piece rp: write it to the output and fan it out
        rs.dst = out_shard + (uint64_t)rp * piece; rs.fanout = true; rs.out_offset = shard_off + (uint64_t)rp * piece;
      } else {
        rs.dst = acc + (uint64_t)rp * piece;
      }
      ENG_TRY(exchange(e, ss, rs, stream));
    }
    for (int s = 0; s < N - 1; ++s) {
      const int sp = mod(e->node + 1 - s), rp = mod(e->node - s);
      SendSpec ss{piece, out_shard + (uint64_t)sp * piece};
      RecvSpec rs;
      rs.bytes = piece; rs.dst = out_shard + (uint64_t)rp * piece; rs.fanout = true;
      rs.out_offset = shard_off + (uint64_t)rp * piece; rs.last = (s == N - 2);
      ENG_TRY(exchange(e, ss, rs, stream));
    }
  }
  ENG_TRY(waitFanout(e, stream));
  if (user_out != nullptr) ENG_NET(gpu::copyDeviceToDeviceAsync(user_out, out, bytes, stream));
  return 0;
}

int tcpxb_engine_all_gather(void* engine, const void* in_, void* out_, uint64_t B, void* stream) {
  Range range("tcpxb all_gather");
  Engine* e = static_cast<Engine*>(engine);
  ENG_TRY(checkReady(e));
  if (B == 0 || B % 16 != 0) return fail("all_gather block must be a multiple of 16 bytes%s", "");
  uint8_t* out = static_cast<uint8_t*>(out_);
  const int world_blocks = e->nodes * e->G;
  if (e->G > 1 && (out != e->out[e->local] || B * (uint64_t)world_blocks > e->buffer_bytes))
    return fail("with several GPUs per node, out must be the registered output buffer%s", "");
  ++e->epoch;
  const int me = e->twin ? 0 : e->cfg.rank;
  // own block into every local GPU's output
  ENG_TRY(barrierInputs(e, stream));  // the peers' outputs may be overwritten from here on
  for (int l = 0; l < e->G; ++l) {
    uint8_t* dst = (l == e->local ? out : e->out[l]) + (uint64_t)me * B;
    ENG_NET(gpu::copyDeviceToDeviceAsync(dst, in_, B, stream));
  }
  const int N = e->nodes;
  auto mod = [N](int x) { return ((x % N) + N) % N; };
  for (int s = 0; s < N - 1; ++s) {
    const int sn = mod(e->node - s), rn = mod(e->node - s - 1);
    const uint64_t soff = (uint64_t)((e->twin ? rn : sn) * e->G + e->local) * B;  // the twin sends what its peer would
    const uint64_t roff = (uint64_t)(rn * e->G + e->local) * B;
    SendSpec ss{B, e->twin ? static_cast<const uint8_t*>(in_) : out + soff};
    RecvSpec rs;
    rs.bytes = B; rs.dst = out + roff; rs.fanout = true; rs.out_offset = roff; rs.last = (s == N - 2);
    ENG_TRY(exchange(e, ss, rs, stream));
  }
  ENG_TRY(waitFanout(e, stream));
  return 0;
}

int tcpxb_engine_reduce_scatter(void* engine, const void* in_, void* out_, uint64_t B, int dtype, void* stream) {
  Range range("tcpxb reduce_scatter");
  Engine* e = static_cast<Engine*>(engine);
  ENG_TRY(checkReady(e));
  if (dtype != TCPXB_BF16 && dtype != TCPXB_F32) return fail("reduce_scatter needs bf16 or f32%s", "");
  if (B == 0 || B % 16 != 0) return fail("reduce_scatter block must be a multiple of 16 bytes%s", "");
  const uint8_t* in = static_cast<const uint8_t*>(in_);
  uint8_t* out = static_cast<uint8_t*>(out_);
  const int N = e->nodes;
  if (e->G > 1 && (in != e->work[e->local] || B * (uint64_t)(N * e->G) > e->buffer_bytes))
    return fail("with several GPUs per node, in must be the registered work buffer%s", "");
  ++e->epoch;
  // 1. per node-block j: sum over the local GPUs of block (j, local) -> tmp[j]
  ENG_TRY(ensureScratch(e, (uint64_t)N * B + (uint64_t)e->req_bytes));
  uint8_t* tmp = e->scratch;
  if (e->G > 1) {
    ENG_TRY(barrierInputs(e, stream));
    std::vector<void*> srcs;
    for (int l = 0; l < e->G; ++l) srcs.push_back(e->work[l]);
    for (int j = 0; j < N; ++j)
      ENG_K(tcpxb_peer_reduce(tmp + (uint64_t)j * B, srcs.data(), e->G, (uint64_t)(j * e->G + e->local) * B, B, dtype, stream));
  } else {
    for (int j = 0; j < N; ++j) {
      const int blk = e->twin ? 0 : j;  // the twin's input has one block per real rank
      ENG_NET(gpu::copyDeviceToDeviceAsync(tmp + (uint64_t)j * B, in + (uint64_t)blk * B, B, stream));
    }
  }
  // 2. ring reduce-scatter over the nodes; the last step writes the result
  auto mod = [N](int x) { return ((x % N) + N) % N; };
  for (int s = 0; s < N - 1; ++s) {
    const int sp = mod(e->node - s - 1), rp = mod(e->node - s - 2);
    SendSpec ss{B, tmp + (uint64_t)(e->twin ? rp : sp) * B};
    RecvSpec rs;
    rs.bytes = B; rs.dtype = dtype; rs.acc = tmp + (uint64_t)rp * B;
    rs.dst = (s == N - 2) ? out : tmp + (uint64_t)rp * B;
    ENG_TRY(exchange(e, ss, rs, stream));
  }
  if (e->G > 1) {
    // peers may not restage inputs before everyone has read them
    uint32_t* pf[TCPXB_MAX_PEERS + 1];
    int n = 0;
    for (int l = 0; l < e->G; ++l) pf[n++] = e->flags[l] + 32 + e->local;
    ENG_K(tcpxb_signal_flags(pf, n, e->epoch, stream));
    ENG_K(tcpxb_wait_flags(e->flags[e->local] + 32, e->G, e->epoch, 0, e->status_dev, stream));
  }
  return 0;
}

int tcpxb_engine_send_next(void* engine, const void* buf, uint64_t bytes, void* stream) {
  Engine* e = static_cast<Engine*>(engine);
  ENG_TRY(checkReady(e));
  SendSpec ss{bytes, static_cast<const uint8_t*>(buf)};
  RecvSpec rs;
  return exchange(e, ss, rs, stream);
}

int tcpxb_engine_recv_prev(void* engine, void* buf, uint64_t bytes, void* stream) {
  Engine* e = static_cast<Engine*>(engine);
  ENG_TRY(checkReady(e));
  SendSpec ss;
  RecvSpec rs;
  rs.bytes = bytes; rs.dst = static_cast<uint8_t*>(buf);
  return exchange(e, ss, rs, stream);
}

// ---- asynchronous calls ----------------------------------------------------------------
uint64_t tcpxb_engine_all_reduce_async(void* engine, const void* in, void* out, uint64_t bytes, int dtype, void* after_event) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr) { fail("null engine%s", ""); return 0; }
  return submit(e, [=](void* stream) { return tcpxb_engine_all_reduce(e, in, out, bytes, dtype, stream); }, after_event);
}

uint64_t tcpxb_engine_all_gather_async(void* engine, const void* in, void* out, uint64_t bytes_per_rank, void* after_event) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr) { fail("null engine%s", ""); return 0; }
  return submit(e, [=](void* stream) { return tcpxb_engine_all_gather(e, in, out, bytes_per_rank, stream); }, after_event);
}

uint64_t tcpxb_engine_reduce_scatter_async(void* engine, const void* in, void* out, uint64_t bytes_per_rank, int dtype, void* after_event) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr) { fail("null engine%s", ""); return 0; }
  return submit(e, [=](void* stream) { return tcpxb_engine_reduce_scatter(e, in, out, bytes_per_rank, dtype, stream); }, after_event);
}

int tcpxb_engine_test(void* engine, uint64_t ticket, int* done) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr || done == nullptr) return fail("null argument%s", "");
  std::lock_guard<std::mutex> l(e->job_mu);
  auto it = e->jobs.find(ticket);
  if (it == e->jobs.end()) return fail("unknown ticket%s", "");
  *done = it->second->finished ? 1 : 0;
  if (it->second->finished && it->second->rc != 0) { snprintf(g_err, sizeof g_err, "%s", it->second->error.c_str()); return -1; }
  return 0;
}

int tcpxb_engine_wait(void* engine, uint64_t ticket) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr) return fail("null engine%s", "");
  std::unique_lock<std::mutex> l(e->job_mu);
  auto it = e->jobs.find(ticket);
  if (it == e->jobs.end()) return fail("unknown ticket%s", "");
  Engine::Job* job = it->second;
  e->job_cv.wait(l, [job] { return job->finished; });
  if (job->rc != 0) { snprintf(g_err, sizeof g_err, "%s", job->error.c_str()); return -1; }
  return 0;
}

int tcpxb_engine_stream_wait(void* engine, uint64_t ticket, void* stream) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr) return fail("null engine%s", "");
  gpu::Event done = nullptr;
  {
    std::lock_guard<std::mutex> l(e->job_mu);
    auto it = e->jobs.find(ticket);
    if (it == e->jobs.end()) return fail("unknown ticket%s", "");
    if (!it->second->finished) return fail("the job has not finished queueing its kernels: call tcpxb_engine_wait first%s", "");
    done = it->second->done;
  }
  ENG_NET(gpu::streamWaitEvent(stream, done));
  return 0;
}

int tcpxb_engine_release(void* engine, uint64_t ticket) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr) return fail("null engine%s", "");
  std::lock_guard<std::mutex> l(e->job_mu);
  auto it = e->jobs.find(ticket);
  if (it == e->jobs.end()) return fail("unknown ticket%s", "");
  if (!it->second->finished) return fail("the job is still running%s", "");
  gpu::eventDestroy(it->second->done);
  delete it->second;
  e->jobs.erase(it);
  return 0;
}

int tcpxb_engine_stats(void* engine, tcpxbEngineStats* out) {
  if (engine == nullptr || out == nullptr) return -1;
  Engine* e = static_cast<Engine*>(engine);
  uint64_t ti = 0, tb = 0, ri = 0, rb = 0;
  for (Rail& r : e->rails) {
    uint64_t a = 0, b = 0;
    netCommHelperWaits(r.send, &a, &b); ti += a; tb += b;
    netCommHelperWaits(r.recv, &a, &b); ri += a; rb += b;
  }
  e->stats.tx_idle = ti * 1e-9; e->stats.tx_blocked = tb * 1e-9;
  e->stats.rx_idle = ri * 1e-9; e->stats.rx_blocked = rb * 1e-9;
  *out = e->stats;
  return 0;
}

int tcpxb_engine_device_status(void* engine, uint32_t* words4) {
  Engine* e = static_cast<Engine*>(engine);
  if (e == nullptr || words4 == nullptr) return -1;
  for (int i = 0; i < 4; ++i) words4[i] = e->status_host[i];
  return 0;
}

}  // extern "C"
