// Core transport: init, memory registration, the progress engine, helper threads,
// completion and teardown.  See transport.h for the overall contract.
#include "tcpxb/transport.h"

#include <linux/errqueue.h>
#include <poll.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <sys/prctl.h>
#include <unistd.h>

#include <algorithm>

#include "tcpxb/cu_driver.h"
#include "tcpxb/kernels.h"

#ifndef SO_EE_ORIGIN_ZEROCOPY
#define SO_EE_ORIGIN_ZEROCOPY 5
#endif
#ifndef MSG_ZEROCOPY
#define MSG_ZEROCOPY 0x4000000
#endif

namespace tcpxb {

namespace {

struct CoreGlobal {
  std::mutex mu;
  bool inited = false;
  CpuBindings tx_bind, rx_bind, tx_irq_bind, rx_irq_bind;
  std::unique_ptr<LogGarbageCollector> gc;
  bool registered_app = false;
};
CoreGlobal cg;

const char* kTaskStageName[] = {"FREE", "ACTIVE", "COMPLETING", "INACTIVE"};
const char* kReqStageName[] = {"FREE", "POSTED", "ACTIVE", "TRANSMITTING", "INACTIVE"};

inline void traceTask(Comm* c, const Task* t, int stage) {
  if (traceConfig().task_level) traceTransition(c->events.get(), 'T', t, c->passive, kTaskStageName[stage]);
}
inline void traceReq(Comm* c, const Request* r, int stage) {
  if (traceConfig().request_level) traceTransition(c->events.get(), 'R', r, c->passive, kReqStageName[stage]);
}

// Debug watchdog (TCPXB_WATCHDOG_SECS=n): a thread that prints, every n seconds,
// the last checkpoint of every comm whose API thread has been inside a call for
// more than n seconds.  Finds calls that never return.
std::mutex g_wd_mu;
std::vector<Comm*> g_wd_comms;
bool g_wd_started = false;
std::atomic<bool> g_wd_on{false};  // checkpoints cost a clock read each: taken only while the watchdog runs
inline void mark(Comm* c, const char* where) {
  if (!g_wd_on.load(std::memory_order_relaxed)) return;
  c->where.store(where, std::memory_order_relaxed);
  c->where_ns.store(monotonicNanos(), std::memory_order_relaxed);
}
void watchdogRegister(Comm* c) {
  const char* v = getenv("TCPXB_WATCHDOG_SECS");
  if (v == nullptr) return;
  const int secs = std::max(1, atoi(v));
  std::lock_guard<std::mutex> l(g_wd_mu);
  g_wd_comms.push_back(c);
  g_wd_on.store(true, std::memory_order_relaxed);
  if (g_wd_started) return;
  g_wd_started = true;
  std::thread([secs] {
    for (;;) {
      sleep((unsigned)secs);
      std::lock_guard<std::mutex> guard(g_wd_mu);
      const uint64_t now = monotonicNanos();
      for (Comm* wc : g_wd_comms) {
        const char* w = wc->where.load();
        const uint64_t t = wc->where_ns.load();
        if (strcmp(w, "idle") != 0 && now - t > (uint64_t)secs * 1000000000ull)
          WARN("watchdog: %s comm %lx has been at '%s' for %lu ms", wc->passive ? "recv" : "send", (unsigned long)wc->id, w,
               (unsigned long)((now - t) / 1000000));
      }
    }
  }).detach();
}
void watchdogForget(Comm* c) {
  std::lock_guard<std::mutex> l(g_wd_mu);
  g_wd_comms.erase(std::remove(g_wd_comms.begin(), g_wd_comms.end(), c), g_wd_comms.end());
}

void setError(Comm* c, Result r) {
  int expected = kSuccess;
  c->error.compare_exchange_strong(expected, (int)r);
}

}  // namespace

// ------------------------------------------------------------------ CPU bindings
bool parseCoreRanges(const char* text, const std::vector<std::string>& if_names, CpuBindings* out) {
  *out = CpuBindings();
  if (text == nullptr || *text == 0) return true;
  bool ok = true;
  std::string s(text);
  size_t pos = 0;
  while (pos <= s.size()) {
    size_t end = s.find(';', pos);
    if (end == std::string::npos) end = s.size();
    std::string item = s.substr(pos, end - pos);
    pos = end + 1;
    if (item.empty()) continue;
    size_t colon = item.find(':');
    if (colon == std::string::npos) { ok = false; continue; }
    const std::string nic = item.substr(0, colon);
    int idx = -1;
    for (size_t i = 0; i < if_names.size() && i < (size_t)kMaxIfs; ++i) {
      std::string base = if_names[i].substr(0, if_names[i].find('#'));
      if (if_names[i] == nic || base == nic) { idx = (int)i;
        // a physical name binds every virtual device carved out of it
        std::string ranges = item.substr(colon + 1);
        size_t rp = 0;
        out->n_ranges[idx] = 0;
        while (rp <= ranges.size() && out->n_ranges[idx] < kMaxRanges) {
          size_t re = ranges.find(',', rp);
          if (re == std::string::npos) re = ranges.size();
          std::string r = ranges.substr(rp, re - rp);
          rp = re + 1;
          if (r.empty()) continue;
          int lo = 0, hi = 0;
          int got = sscanf(r.c_str(), "%d-%d", &lo, &hi);
          if (got == 1) hi = lo;
          if (got < 1 || lo < 0 || hi < lo) { ok = false; continue; }
          out->lo[idx][out->n_ranges[idx]] = lo;
          out->hi[idx][out->n_ranges[idx]] = hi;
          ++out->n_ranges[idx];
        }
      }
    }
    if (idx < 0) ok = false;
  }
  return ok;
}

namespace {

void applyAffinity(Comm* comm, int tid) {
  const CpuBindings& b = comm->passive ? cg.rx_bind : cg.tx_bind;
  const int dev = comm->dev;
  if (dev < 0 || dev >= kMaxIfs || b.n_ranges[dev] == 0) return;
  const long ncpu = sysconf(_SC_NPROCESSORS_ONLN);
  std::vector<int> cores;
  for (int r = 0; r < b.n_ranges[dev]; ++r)
    for (int c = b.lo[dev][r]; c <= b.hi[dev][r] && c < ncpu; ++c) cores.push_back(c);
  if (cores.empty()) return;
  cpu_set_t set;
  CPU_ZERO(&set);
  const Flags& f = flags();
  if (f.worker_pin_threads) {
    // one core per helper: comms are strided so that neighbours do not collide
    size_t pick = ((size_t)f.worker_spray_stride * comm->num_threads * comm->stride + (size_t)tid) % cores.size();
    for (int j = 0; j < (int)f.worker_spray_count; ++j)
      CPU_SET(cores[(pick + (size_t)j * (size_t)comm->num_threads) % cores.size()], &set);
  } else {
    for (int c : cores) CPU_SET(c, &set);
  }
  pthread_setaffinity_np(pthread_self(), sizeof set, &set);
}

// ------------------------------------------------------------- zero-copy notices
// Reads completion notifications from the socket's error queue; returns how many
// sendmsg calls completed, or -1 on a socket error.
int readZerocopyCompletions(SocketCtx* s, bool devmem_path = false) {
  int completed = 0;
  for (;;) {
    char control[128];
    struct msghdr msg;
    memset(&msg, 0, sizeof msg);
    msg.msg_control = control;
    msg.msg_controllen = sizeof control;
    ssize_t rc = devmem_path ? devmem::activeOps().recvmsg(s->fd, &msg, MSG_ERRQUEUE | MSG_DONTWAIT)
                             : recvmsg(s->fd, &msg, MSG_ERRQUEUE | MSG_DONTWAIT);
    if (rc < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return completed;
      return -1;
    }
    for (struct cmsghdr* cm = CMSG_FIRSTHDR(&msg); cm != nullptr; cm = CMSG_NXTHDR(&msg, cm)) {
      if (!((cm->cmsg_level == SOL_IP && cm->cmsg_type == IP_RECVERR) ||
            (cm->cmsg_level == SOL_IPV6 && cm->cmsg_type == IPV6_RECVERR)))
        continue;
      struct sock_extended_err* ee = (struct sock_extended_err*)CMSG_DATA(cm);
      if (ee->ee_errno != 0 || ee->ee_origin != SO_EE_ORIGIN_ZEROCOPY) continue;
      // ids [ee_info, ee_data] completed; sequence numbers wrap at 2^32
      completed += (int)(ee->ee_data - ee->ee_info + 1);
    }
  }
}

// Tells the thread that drives this comm (if it sleeps between polls) that a task
// changed state.  One system call at most per sleep of that thread.
inline void notifyDriver(Comm* comm) {
  Notifier* n = comm->notifier;
  if (n != nullptr && n->armed.load(std::memory_order_acquire) != 0 && n->armed.exchange(0, std::memory_order_acq_rel) != 0) {
    const uint64_t one = 1;
    ssize_t rc = write(n->event_fd, &one, sizeof one);
    (void)rc;
  }
}

// ------------------------------------------------------------------ helper thread
// Moves bytes for the oldest active task of socket `s`.  Returns 1 when the task
// finished its I/O, 0 when the socket would block, -1 on error.
int progressTask(Comm* comm, SocketCtx* s, Task* t) {
  const bool slow_on = flags().slow_switch[kSlowSendRecv];
  while (t->offset < t->size) {
    ssize_t n;
    if (t->devmem) {
      // devmem-TCP: no payload passes through this process, only its description
      if (t->op == kSockSend) {
        devmem::TxMessage m;
        devmem::buildSend(&m, t->dmabuf_id, t->dmabuf_off + (uint64_t)t->offset, (size_t)(t->size - t->offset));
        n = devmem::sendFrom(devmem::activeOps(), s->fd, &m);
        if (n > 0) {
          s->stats.tx_cnt.fetch_add(1, std::memory_order_relaxed);
          if (t->zc_count++ == 0) t->zc_first = s->zc_next;
          ++s->zc_next;
        }
      } else {
        devmem::RxSink sink;
        sink.records = t->records.data();
        sink.capacity = t->records.size();
        sink.filled = t->records_filled;
        sink.tokens = &t->tokens;
        sink.pool_bytes = comm->rxmgr->bytes();
        sink.dmabuf_id = comm->rxmgr->rxDmabufId();
        n = devmem::recvInto(devmem::activeOps(), s->fd, (size_t)(t->size - t->offset), s->devmem_control.data(), s->devmem_control.size(),
                             (uint64_t)t->msg_offset + (uint64_t)t->offset, &sink);
        t->records_filled = sink.filled;
        if (n > 0) s->stats.rx_cnt.fetch_add(1, std::memory_order_relaxed);
      }
      if (n < 0) {  // the helpers below speak errno
        if (n == -EPROTO) {
          WARN("%s: unusable devmem control messages", s->flow.c_str());
          setError(comm, kInternalError);
          return -1;
        }
        errno = (int)-n;
        n = -1;
      }
    } else if (t->op == kSockSend) {
      int fl = MSG_DONTWAIT | MSG_NOSIGNAL;
      if (t->zerocopy) fl |= MSG_ZEROCOPY;
      n = send(s->fd, t->host_ptr + t->offset, (size_t)(t->size - t->offset), fl);
      if (n > 0) {
        s->stats.tx_cnt.fetch_add(1, std::memory_order_relaxed);
        if (t->zerocopy) { if (t->zc_count++ == 0) t->zc_first = s->zc_next; ++s->zc_next; }
      }
    } else if (t->host_ptr != nullptr) {
      n = recv(s->fd, t->host_ptr + t->offset, (size_t)(t->size - t->offset), MSG_DONTWAIT);
      if (n > 0) s->stats.rx_cnt.fetch_add(1, std::memory_order_relaxed);
    } else {
      // scattered landing: one recvmsg fills as many pool pages as have data
      struct msghdr msg;
      memset(&msg, 0, sizeof msg);
      msg.msg_iov = t->iov.data() + t->iov_pos;
      msg.msg_iovlen = std::min<size_t>(t->iov.size() - t->iov_pos, 512);
      n = recvmsg(s->fd, &msg, MSG_DONTWAIT);
      if (n > 0) {
        s->stats.rx_cnt.fetch_add(1, std::memory_order_relaxed);
        size_t left = (size_t)n;
        while (left > 0) {
          struct iovec& v = t->iov[t->iov_pos];
          if (left >= v.iov_len) { left -= v.iov_len; ++t->iov_pos; }
          else { v.iov_base = (char*)v.iov_base + left; v.iov_len -= left; left = 0; }
        }
      }
    }
    if (n > 0) {
      t->offset += (int)n;
      s->stats.bytes_posted.fetch_add((uint64_t)n, std::memory_order_relaxed);
      if (slow_on) s->stall.reset();
      continue;
    }
    if (n == 0 && t->op == kSockRecv) {
      WARN("%s: peer closed the connection in mid-message", s->flow.c_str());
      setError(comm, kRemoteError);
      return -1;
    }
    if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) {
      if (slow_on) {
        uint64_t ns = 0;
        if (s->stall.shouldWarn(&ns)) {
          (t->op == kSockSend ? s->stats.tx_slow_cnt : s->stats.rx_slow_cnt).fetch_add(1);
          if (flags().slow_report[kSlowSendRecv])
            WARN("%s: %s stalled for %lu ms at %d/%d bytes", s->flow.c_str(), t->op == kSockSend ? "send" : "recv",
                 (unsigned long)(ns / 1000000), t->offset, t->size);
        }
      }
      return 0;
    }
    if (n < 0 && t->zerocopy && errno == ENOBUFS) { t->zerocopy = false; continue; }  // optmem exhausted: copy instead
    WARN("%s: %s failed: %s", s->flow.c_str(), t->op == kSockSend ? "send" : "recv", strerror(errno));
    setError(comm, (errno == ECONNRESET || errno == EPIPE) ? kRemoteError : kSystemError);
    return -1;
  }
  return 1;
}

void helperMain(Comm* comm, int tid) {
  char name[16];
  snprintf(name, sizeof name, "tcpxb-%s%d", comm->passive ? "rx" : "tx", tid);
  prctl(PR_SET_NAME, name, 0, 0, 0);
  prctl(PR_SET_TIMERSLACK, 1, 0, 0, 0);  // naps of tens of microseconds must not be rounded up to the default 50 us slack
  applyAffinity(comm, tid);
  HelperThread& me = comm->helpers[tid];
  const Flags& f = flags();
  const bool spin = f.thread_spin != 0;
  const bool slow_txc = f.slow_switch[kSlowTxComp];
  int idle_rounds = 0;
  while (!comm->stop.load(std::memory_order_acquire)) {
    bool moved = false, blocked = false, finished = false, staging = false;
    struct pollfd pfds[kMaxSockets];
    int npfd = 0;
    for (int idx = tid; idx < comm->num_socks; idx += comm->num_threads) {
      SocketCtx* s = &comm->sock[idx];
      // Completion stage: a task whose bytes have all moved (and, for zero-copy sends,
      // whose notices have all come back) is handed back to the progress engine.
      auto retireCompleted = [&] {
        while (s->tasks.has(kTaskCompleting)) {
          Task* t = &s->tasks.front(kTaskCompleting);
          if (t->zerocopy && t->zc_count > 0) {
            // done once every notification id of this task is below zc_done (wrap-safe)
            const uint32_t last = t->zc_first + t->zc_count;
            if ((int32_t)(s->zc_done - last) < 0) break;
          } else if (t->op == kSockSend) {
            s->stats.tx_completion_cnt.fetch_add(1, std::memory_order_relaxed);
          }
          s->stats.bytes_done.fetch_add((uint64_t)t->size, std::memory_order_relaxed);
          traceTask(comm, t, kTaskInactive);
          s->tasks.advance(kTaskCompleting);
          moved = true;
          finished = true;
        }
      };
      while (s->tasks.has(kTaskActive)) {
        Task* t = &s->tasks.front(kTaskActive);
        if (t->wait_counter != nullptr) {
          // a send whose payload the copy engine is still staging: not ready, and nobody to wait on but time
          if (!t->wait_counter->reached(t->wait_mark)) { staging = true; break; }
          t->wait_counter = nullptr;
        }
        int rc = progressTask(comm, s, t);
        if (rc < 0) { notifyDriver(comm); return; }
        if (rc == 0) {
          blocked = true;
          pfds[npfd].fd = s->fd;
          pfds[npfd].events = (short)(t->op == kSockSend ? POLLOUT : POLLIN);
          pfds[npfd].revents = 0;
          ++npfd;
          break;
        }
        moved = true;
        traceTask(comm, t, kTaskCompleting);
        s->tasks.advance(kTaskActive);
        retireCompleted();  // at once: the next task may keep this thread busy for a long time
      }
      // zero-copy sends wait for the kernel's notification
      if (s->zc_done != s->zc_next) {
        int c = readZerocopyCompletions(s, comm->devmem);
        if (c < 0) { setError(comm, kSystemError); notifyDriver(comm); return; }
        if (c > 0) { s->zc_done += (uint32_t)c; s->stats.tx_completion_cnt.fetch_add((uint64_t)c); s->stall.reset(); moved = true; }
        else if (slow_txc) {
          uint64_t ns = 0;
          if (s->stall.shouldWarn(&ns)) {
            s->stats.tx_completion_slow_cnt.fetch_add(1);
            if (f.slow_report[kSlowTxComp])
              WARN("%s: no tx completion for %lu ms (%u outstanding)", s->flow.c_str(), (unsigned long)(ns / 1000000),
                   s->zc_next - s->zc_done);
          }
          if (f.tx_completion_nanosleep > 0) {
            struct timespec ts = {0, (long)f.tx_completion_nanosleep};
            nanosleep(&ts, nullptr);
          }
        }
      }
      retireCompleted();
    }
    if (finished) notifyDriver(comm);
    if (moved) { idle_rounds = 0; continue; }
    if (spin) continue;
    if (staging && !blocked) {
      // the copy engine finishes within tens of microseconds: look again soon, without a wake-up from anybody
      if (++idle_rounds > 16) {
        struct timespec ts = {0, 5000};
        nanosleep(&ts, nullptr);
      }
      continue;
    }
    if (blocked) {
      // every owned socket with work would block: sleep in the kernel until one is ready
      if (++idle_rounds > 8 && f.poll_block_us > 0) {
        const uint64_t t0 = monotonicNanos();
        poll(pfds, (nfds_t)npfd, (int)std::max<int64_t>(1, f.poll_block_us / 1000));
        me.blocked_ns.fetch_add(monotonicNanos() - t0, std::memory_order_relaxed);
      }
      continue;
    }
    if (++idle_rounds < 64) continue;  // short spin: the next chunk usually follows at once
    // No task.  Nap in short steps for a while before going to sleep for good: a nap
    // needs nobody to wake it, whereas every real sleep costs the thread that queues
    // the next task a futex system call, and with small requests that is every task.
    const int nap_us = comm->helper_nap_us.load(std::memory_order_relaxed);
    if (nap_us > 0 && idle_rounds < 64 + comm->helper_nap_rounds.load(std::memory_order_relaxed)) {
      const uint64_t t0 = monotonicNanos();
      struct timespec ts = {0, (long)nap_us * 1000};
      nanosleep(&ts, nullptr);
      me.idle_ns.fetch_add(monotonicNanos() - t0, std::memory_order_relaxed);
      continue;
    }
    const uint64_t idle_t0 = monotonicNanos();
    std::unique_lock<std::mutex> l(me.mu);
    me.sleeping.store(true, std::memory_order_seq_cst);
    me.cv.wait_for(l, std::chrono::milliseconds(50), [&] {
      return me.kicks.load(std::memory_order_seq_cst) != me.seen || comm->stop.load(std::memory_order_acquire);
    });
    me.sleeping.store(false, std::memory_order_release);
    me.idle_ns.fetch_add(monotonicNanos() - idle_t0, std::memory_order_relaxed);
    me.seen = me.kicks.load(std::memory_order_acquire);
    idle_rounds = 0;
  }
}

// A new task for socket `sock_idx`: its helper is woken once per progress round
// (flushKicks), however many tasks the round queued for it.
void kick(Comm* comm, int sock_idx) { comm->kick_mask |= 1u << (sock_idx % comm->num_threads); }

void flushKicks(Comm* comm) {
  uint32_t mask = comm->kick_mask;
  comm->kick_mask = 0;
  for (int t = 0; mask != 0; ++t, mask >>= 1) {
    if ((mask & 1u) == 0) continue;
    HelperThread& h = comm->helpers[t];
    h.kicks.fetch_add(1, std::memory_order_seq_cst);
    if (!flags().thread_spin && h.sleeping.load(std::memory_order_seq_cst)) {
      // Taking the lock after the increment closes the window in which a helper has
      // evaluated its wait predicate but is not yet blocked.
      { std::lock_guard<std::mutex> l(h.mu); }
      h.cv.notify_one();
    }
  }
}

// --------------------------------------------------------------- CUDA resources
Result ensureCudaComm(Comm* comm, int gpu_dev) {
  if (comm->stream != nullptr) return kSuccess;
  if (!gpu::available()) { WARN("CUDA buffer given but no CUDA device is usable"); return kInvalidUsage; }
  comm->gpu_dev = gpu_dev;
  int cur = -1;
  TCPXB_CHECK(gpu::currentDevice(&cur));
  if (cur != gpu_dev) TCPXB_CHECK(gpu::setDevice(gpu_dev));
  TCPXB_CHECK(gpu::streamCreate(&comm->stream));
  TCPXB_CHECK(comm->passive ? comm->unpack_marks.init() : comm->stage_marks.init());
  return kSuccess;
}

Result ensureCudaRecv(Comm* comm, int gpu_dev, bool want_device_handle = false) {
  TCPXB_CHECK(ensureCudaComm(comm, gpu_dev));
  if (comm->rxmgr == nullptr) {
    comm->rxmgr = rxBufMgrFor(gpu_dev);
    if (comm->rxmgr == nullptr) return kUnhandledCudaError;
    const std::string pci = gpu::pciBusId(gpu_dev);
    for (int i = 0; i < comm->num_socks; ++i) comm->rxmgr->installFlowRule(comm->sock[i].fd, pci);
  }
  if (comm->devq == nullptr || (want_device_handle && comm->devq->deviceHandle() == nullptr)) {
    if (comm->devq != nullptr && comm->devq->inUse() != 0) return kInvalidUsage;
    comm->devq = std::make_unique<DevQueue>();
    TCPXB_CHECK(comm->devq->init(comm->rxmgr->devBase(), want_device_handle));
  }
  if (comm->unpack_status_host == nullptr) {
    void* h = nullptr;
    void* d = nullptr;
    TCPXB_CHECK(gpu::hostAllocMapped(64, &h, &d));
    memset(h, 0, 64);
    comm->unpack_status_host = static_cast<uint32_t*>(h);
    comm->unpack_status_dev = static_cast<uint32_t*>(d);
  }
  return kSuccess;
}

Result ensureTxStage(Comm* comm) {
  if (comm->tx_stage != nullptr) return kSuccess;
  void* h = nullptr;
  void* d = nullptr;
  if (comm->tx_stage_bytes == 0) comm->tx_stage_bytes = (uint64_t)flags().tx_staging_bytes;
  TCPXB_CHECK(gpu::hostAllocMapped(comm->tx_stage_bytes, &h, &d));
  comm->tx_stage = static_cast<uint8_t*>(h);
  return kSuccess;
}

// Reserves `bytes` of the pinned tx staging ring (FIFO); false when it is full.
bool stageAlloc(Comm* comm, uint64_t bytes, uint8_t** out, uint64_t* charged) {
  const uint64_t cap = comm->tx_stage_bytes;
  if (bytes > cap) return false;
  // an empty ring restarts at offset 0, so a request as large as the ring always fits eventually
  if (comm->tx_head == comm->tx_tail) comm->tx_head = comm->tx_tail = 0;
  uint64_t head = comm->tx_head;
  uint64_t pos = head % cap;
  uint64_t skip = (pos + bytes > cap) ? cap - pos : 0;  // do not wrap inside a request
  if (head + skip + bytes - comm->tx_tail > cap) return false;
  *out = comm->tx_stage + (head + skip) % cap;
  *charged = skip + bytes;
  comm->tx_head = head + skip + bytes;
  return true;
}

Result startCudaSend(Comm* comm, Request* r, MemHandle* mh) {
  TCPXB_CHECK(ensureCudaComm(comm, mh != nullptr && mh->gpu_dev >= 0 ? mh->gpu_dev : comm->gpu_dev));
  TCPXB_CHECK(ensureTxStage(comm));
  if (r->size == 0) return kSuccess;
  if ((uint64_t)r->size > comm->tx_stage_bytes) {
    WARN("send of %d bytes from device memory is larger than the staging ring (%lu bytes); raise NCCL_GPUDIRECTTCPX_TX_STAGING_BYTES",
         r->size, (unsigned long)comm->tx_stage_bytes);
    return kInvalidArgument;
  }
  if (!stageAlloc(comm, (uint64_t)r->size, &r->stage, &r->stage_bytes)) return kInProgress;
  // One staging copy per ~2 MiB: enough to let the first chunks leave while the
  // rest is still being copied, few enough that the per-copy launch cost stays small.
  const int chunk = chunkBytesFor(r->size, comm->num_socks);
  int n_want = std::max(1, std::min(kMaxTxSegments, r->size / (2 << 20)));
  int seg = (r->size + n_want - 1) / n_want;
  seg = (seg + chunk - 1) / chunk * chunk;
  if (comm->send_dependency != nullptr) {
    TCPXB_CHECK(gpu::streamWaitEvent(comm->stream, comm->send_dependency));
    comm->send_dependency = nullptr;
  }
  r->seg_bytes = seg;
  r->n_segs = (r->size + seg - 1) / seg;
  r->segs_done = 0;
  for (int i = 0; i < r->n_segs; ++i) {
    const int off = i * seg;
    const int len = std::min(seg, r->size - off);
    TCPXB_CHECK(gpu::copyToHostAsync(r->stage + off, r->data + off, (size_t)len, comm->stream));
    TCPXB_CHECK(comm->stage_marks.mark(comm->stream, &r->seg_mark[i]));
  }
  return kSuccess;
}

// True when the staged bytes [0, upto) of a CUDA send have reached host memory.
bool stagedUpTo(Request* r, int upto) {
  const int need = (upto + r->seg_bytes - 1) / r->seg_bytes;
  while (r->segs_done < need) {
    if (!r->comm->stage_marks.reached(r->seg_mark[r->segs_done])) return false;
    ++r->segs_done;
  }
  return true;
}

void releasePages(Comm* comm, Request* r) {
  if (!r->pages.empty() && comm->rxmgr != nullptr) comm->rxmgr->releasePages(r->pages.data(), r->pages.size());
  r->pages.clear();
  if (comm->devmem) {
    // the pages go back to the NIC's pool through the socket each fragment came from
    for (int i = 0; i < comm->num_socks; ++i)
      if (!r->tokens[i].empty()) devmem::recycle(devmem::activeOps(), comm->sock[i].fd, &r->tokens[i]);
  }
}

// ------------------------------------------------------------------ task set-up
void fillSendTask(Comm* comm, Request* r, int sock_idx, int chunk) {
  SocketCtx& s = comm->sock[sock_idx];
  Task& t = s.tasks.nextFree();
  t.r = r;
  t.op = kSockSend;
  t.wait_counter = nullptr;
  t.devmem = comm->devmem && r->mem_type == kPtrCuda;
  if (t.devmem) {
    t.dmabuf_id = r->mh->dmabuf_id;
    t.dmabuf_off = r->mh->dmabuf_offset + (uint64_t)(r->data - static_cast<const uint8_t*>(r->mh->ptr)) + (uint64_t)r->offset;
  } else if (r->mem_type == kPtrCuda && r->size > 0) {
    // the helper thread itself waits for the staging copy that covers this chunk
    const int seg = (r->offset + chunk + r->seg_bytes - 1) / r->seg_bytes - 1;
    t.wait_counter = &comm->stage_marks;
    t.wait_mark = r->seg_mark[seg];
  }
  t.host_ptr = t.devmem ? nullptr : (r->mem_type == kPtrCuda ? r->stage : r->data) + r->offset;
  t.size = chunk;
  t.offset = 0;
  t.msg_offset = r->offset;
  t.pages.clear();
  t.iov.clear();
  t.iov_pos = 0;
  t.zc_first = t.zc_count = 0;
  t.zerocopy = t.devmem || (s.zerocopy_enabled && r->mem_type == kPtrHost && flags().min_zcopy_size > 0 &&
                            chunk >= flags().min_zcopy_size);
  traceTask(comm, &t, kTaskActive);
  s.tasks.admit();
  r->offset += chunk;
  kick(comm, sock_idx);
}

// Receive task into pool pages; false when the pool has no room right now.
bool fillRecvTask(Comm* comm, Request* r, int sock_idx, int chunk, int msg_offset) {
  SocketCtx& s = comm->sock[sock_idx];
  Task& t = s.tasks.nextFree();
  t.pages.clear();
  t.iov.clear();
  t.iov_pos = 0;
  t.devmem = comm->devmem && r->mem_type == kPtrCuda;
  t.wait_counter = nullptr;
  if (t.devmem) {
    // the NIC has placed (or will place) the payload in the bound pool; recvmsg only tells where
    const size_t frags = (size_t)chunk / 1024 + 64;  // fragments are MTU- to page-sized; refused beyond this
    if (t.records.size() < frags) t.records.resize(frags);
    t.records_filled = 0;
    t.tokens.clear();
    if (s.devmem_control.empty()) s.devmem_control.resize(devmem::rxControlBytes(512));
    t.host_ptr = nullptr;
  } else if (r->mem_type == kPtrCuda) {
    const uint32_t n_pages = ((uint32_t)chunk + kRxPageBytes - 1) / kRxPageBytes;
    // a sender whose chunks differ from the first one may outrun the promise; the rest is taken as it comes
    const bool promised = r->pages_reserved >= n_pages;
    if (!comm->rxmgr->allocPages(n_pages, &t.pages, promised)) return false;
    if (promised) r->pages_reserved -= n_pages;
    uint8_t* base = comm->rxmgr->hostBase();
    int left = chunk;
    for (const PageRun& run : t.pages) {
      const int run_bytes = std::min<int64_t>((int64_t)run.count * kRxPageBytes, left);
      t.iov.push_back({base + (uint64_t)run.first * kRxPageBytes, (size_t)run_bytes});
      left -= run_bytes;
    }
    t.host_ptr = nullptr;
  } else {
    t.host_ptr = r->data + msg_offset;
  }
  t.r = r;
  t.op = kSockRecv;
  t.size = chunk;
  t.offset = 0;
  t.msg_offset = msg_offset;
  t.zerocopy = false;
  t.zc_first = t.zc_count = 0;
  traceTask(comm, &t, kTaskActive);
  s.tasks.admit();
  kick(comm, sock_idx);
  return true;
}

// A finished receive task of a CUDA request: describe its pages in the request's
// slot (one record per page fragment) and keep the pages until the consumer is done.
Result describePages(Comm* comm, Request* r, Task* t, int sock_idx) {
  if (t->devmem) {
    // the kernel already wrote the list: move it into the request's slot and keep the tokens
    if (r->slot.filled + t->records_filled > (uint64_t)kUnpackMaxSlicePages) {
      WARN("receive of %d bytes arrived in more than the %d fragments a scatter-list slot holds", r->size, kUnpackMaxSlicePages);
      return kInternalError;
    }
    memcpy(&r->slot.mem[r->slot.filled], t->records.data(), t->records_filled * sizeof(LoadMeta));
    r->slot.filled += t->records_filled;
    auto& keep = r->tokens[sock_idx];
    for (const devmem::DmabufToken& run : t->tokens) {
      if (!keep.empty() && keep.back().token_start + keep.back().token_count == run.token_start) keep.back().token_count += run.token_count;
      else keep.push_back(run);
    }
    t->tokens.clear();
    t->records_filled = 0;
    return kSuccess;
  }
  int left = t->size;
  uint64_t dst = (uint64_t)t->msg_offset;
  for (const PageRun& run : t->pages) {
    r->pages.push_back(run);
    if (comm->rxmgr->deviceResident() && left > 0) {
      // device pool: the copy engine places the run (it landed in the pinned mirror)
      const uint64_t off = (uint64_t)run.first * kRxPageBytes;
      const size_t len = (size_t)std::min<int64_t>((int64_t)run.count * kRxPageBytes, left);
      TCPXB_CHECK(gpu::copyToDeviceAsync(comm->rxmgr->devBase() + off, comm->rxmgr->hostBase() + off, len, comm->stream));
    }
    for (uint32_t p = 0; p < run.count && left > 0; ++p) {
      if (r->slot.filled >= (uint64_t)kUnpackMaxSlicePages) {
        WARN("receive of %d bytes into device memory needs more than the %d page records of a scatter-list slot "
             "(%d bytes at most per receive)", r->size, kUnpackMaxSlicePages, kUnpackMaxSlicePages * (int)kRxPageBytes);
        return kInternalError;
      }
      const uint32_t len = (uint32_t)std::min<int>(left, (int)kRxPageBytes);
      LoadMeta& m = r->slot.mem[r->slot.filled++];
      m.src_off = (run.first + p) * kRxPageBytes;
      m.len = len;
      m.dst_off = dst;
      dst += len;
      left -= (int)len;
    }
  }
  t->pages.clear();
  return kSuccess;
}

Result launchUnpack(Comm* comm, Request* r) {
  // In the host-only build this is the stand-in device's unpack, done at once on this thread.
  mark(comm, "launchUnpack:kernel");
  if (r->slot.filled > 0) {
    int rc = tcpxb_unpack_copy(comm->rxmgr->devBase(), comm->rxmgr->bytes(), r->data, (uint64_t)r->size,
                               reinterpret_cast<const tcpxbLoadMeta*>(r->slot.mem_dev), (uint32_t)r->slot.filled,
                               comm->unpack_status_dev, nullptr, comm->stream);
    if (rc != 0) { WARN("unpack launch failed: %s", tcpxb_kernel_last_error()); return kUnhandledCudaError; }
  }
  mark(comm, "launchUnpack:mark");
  TCPXB_CHECK(comm->unpack_marks.mark(comm->stream, &r->unpack_mark));
  r->unpack_launched = true;
  return kSuccess;
}

// ------------------------------------------------------------- progress engine
}  // namespace

// Striping quantum of one message.  The fixed quantum (NCCL_DYNAMIC_CHUNK_SIZE) cuts a
// 4 MiB message into 32 chunks even when the comm has a single socket, and every
// chunk costs a control record, a task hand-off and a completion.  With
// ADAPTIVE_CHUNK (default) a message is cut into about one chunk per socket instead:
// the quantum grows to size / sockets, rounded up to a whole rx page, but never
// beyond kMaxAdaptiveChunk, so that large messages still pipeline through the task rings.
int chunkBytesFor(int message_bytes, int num_socks) {
  const Flags& f = flags();
  int64_t chunk = f.dynamic_chunk_size;
  if (f.adaptive_chunk != 0 && num_socks > 0) {
    int64_t per_sock = ((int64_t)message_bytes + num_socks - 1) / num_socks;
    per_sock = (per_sock + kRxPageBytes - 1) / kRxPageBytes * kRxPageBytes;
    chunk = std::max(chunk, std::min<int64_t>(per_sock, std::max<int64_t>(kMaxAdaptiveChunk, chunk)));
  }
  return (int)std::min<int64_t>(chunk, INT32_MAX);
}

namespace {

Result progressSendRequest(Comm* comm, Request* r) {
  const Flags& f = flags();
  const bool devmem_cuda = comm->devmem && r->mem_type == kPtrCuda;
  if ((r->size <= f.inline_threshold && !devmem_cuda) || r->size == 0) {
    // small message: record + payload ride the control socket
    if (!r->inline_queued) {
      if (r->mem_type == kPtrCuda && r->size > 0 && !stagedUpTo(r, r->size)) return kSuccess;
      CtrlMsg m = {kCtrlInline, 0, (uint32_t)r->size, 0, (uint32_t)r->size};
      Result pr = comm->ctrl_send.push(m);
      if (pr == kInProgress) return kSuccess;
      TCPXB_CHECK(pr);
      r->inline_queued = true;  // payload follows
    }
    Result fr = comm->ctrl_send.flush();
    if (fr == kInProgress) return kSuccess;
    TCPXB_CHECK(fr);
    if (r->size > 0) {
      uint8_t* src = r->mem_type == kPtrCuda ? r->stage : r->data;
      TCPXB_CHECK(socketProgress(kSockSend, comm->ctrl_fd, src, r->size, &r->offset));
      if (r->offset < r->size) return kSuccess;
    }
    r->offset = r->size;
    r->size_pending = 0;
    comm->ctrl_stats.tx_cnt.fetch_add(1);
    comm->ctrl_stats.bytes_done.fetch_add((uint64_t)r->size);
    traceReq(comm, r, kReqTransmitting);
    comm->rq.advance(kReqActive);
    return kSuccess;
  }
  const int chunk_size = chunkBytesFor(r->size, comm->num_socks);
  while (r->offset < r->size && comm->mapper->hasFlow()) {
    const int chunk = std::min(chunk_size, r->size - r->offset);
    // A chunk of a CUDA send is announced and queued before its staging copy has
    // finished: the control record lets the receiver set up, and the helper thread waits
    // for the copy itself (Task::wait_mark), so no progress round is spent on noticing it.
    if (comm->ctrl_send.full()) {
      Result fr = comm->ctrl_send.flush();
      if (fr == kInProgress) break;
      TCPXB_CHECK(fr);
    }
    const int s = comm->mapper->pick();
    if (s < 0) break;
    CtrlMsg m = {kCtrlNormal, (uint16_t)s, (uint32_t)chunk, (uint32_t)r->offset, (uint32_t)r->size};
    TCPXB_CHECK(comm->ctrl_send.push(m));
    fillSendTask(comm, r, s, chunk);
  }
  Result fr = comm->ctrl_send.flush();
  if (fr != kInProgress) TCPXB_CHECK(fr);
  if (r->offset == r->size) {
    traceReq(comm, r, kReqTransmitting);
    comm->rq.advance(kReqActive);
  }
  return kSuccess;
}

Result progressRecvRequest(Comm* comm, Request* r) {
  const Flags& f = flags();
  for (;;) {
    if (!comm->have_ctrl) {
      // An empty control socket costs a system call to discover; callers poll in
      // tight loops, so after one empty read the next look waits a microsecond.
      if (comm->ctrl_recv.buffered() < (int)sizeof(CtrlMsg) && comm->ctrl_quiet_until_ns != 0 && !comm->ctrl_readable_hint) {
        if (monotonicNanos() < comm->ctrl_quiet_until_ns) return kSuccess;
        comm->ctrl_quiet_until_ns = 0;
      }
      Result pr = comm->ctrl_recv.pop(&comm->ctrl);
      if (pr == kInProgress) {
        // a caller that tells us when the socket is readable (netHintCtrlReadable) needs
        // the blind retry only as a safety net
        comm->ctrl_readable_hint = false;
        comm->ctrl_quiet_until_ns = monotonicNanos() + (comm->ctrl_hinted ? 200000 : 1000);
        if (f.slow_switch[kSlowRxCtrl]) {
          uint64_t ns = 0;
          if (comm->ctrl_stall.shouldWarn(&ns) && f.slow_report[kSlowRxCtrl])
            WARN("%s: no control record for %lu ms (request %p)", comm->ctrl_flow.c_str(), (unsigned long)(ns / 1000000), (void*)r);
        }
        return kSuccess;
      }
      if (pr != kSuccess) {
        WARN("%s: control socket failed (%s)", comm->ctrl_flow.c_str(), resultString(pr));
        return pr;
      }
      if (f.slow_switch[kSlowRxCtrl]) comm->ctrl_stall.reset();
      comm->have_ctrl = true;
      comm->ctrl_stats.rx_cnt.fetch_add(1);
      const CtrlMsg& c = comm->ctrl;
      if (c.type >= kCtrlMaxType || (c.type == kCtrlNormal && c.index >= comm->num_socks) ||
          (uint64_t)c.offset + c.size > c.total) {
        WARN("%s: malformed control record type %u index %u size %u offset %u total %u", comm->ctrl_flow.c_str(), c.type,
             c.index, c.size, c.offset, c.total);
        return kRemoteError;
      }
      if (!r->size_known) {
        if ((int64_t)c.total > (int64_t)r->capacity) {
          WARN("message of %u bytes does not fit the posted receive of %d bytes", c.total, r->capacity);
          return kInvalidUsage;
        }
        r->size = (int)c.total;
        r->size_pending = r->size;
        r->size_known = true;
      }
      if (c.offset != (uint32_t)r->offset) {
        WARN("control record for offset %u arrived at offset %d", c.offset, r->offset);
        return kRemoteError;
      }
    }
    const CtrlMsg& c = comm->ctrl;
    if (r->mem_type == kPtrCuda && !comm->devmem && !r->pages_promised && r->size > 0) {
      // The first record tells the message's size and the sender's chunk size.  Every
      // page the message will need is promised now, or none: a message that waited for
      // pages while holding some could block, and be blocked by, another connection's.
      uint32_t need = 1;
      if (c.type != kCtrlInline) {
        const uint32_t chunk = c.size > 0 ? c.size : 1;
        const uint32_t per = (chunk + kRxPageBytes - 1) / kRxPageBytes;
        const uint32_t rem = (uint32_t)r->size % chunk;
        need = (uint32_t)r->size / chunk * per + (rem + kRxPageBytes - 1) / kRxPageBytes;
      }
      if (need > comm->rxmgr->totalPages()) {
        WARN("message of %d bytes needs %u rx pages but the pool has %u; raise NCCL_GPUDIRECTTCPX_RX_POOL_BYTES", r->size, need,
             comm->rxmgr->totalPages());
        return kInvalidUsage;
      }
      if (!comm->rxmgr->reservePages(need)) return kSuccess;  // pool busy: retry, holding nothing
      r->pages_promised = true;
      r->pages_reserved = need;
    }
    if (c.type == kCtrlInline) {
      if (r->size > 0) {
        uint8_t* dst = r->data;
        if (r->mem_type == kPtrCuda) {
          // land in one pool page; the unpack path then treats it like any fragment
          if (r->pages.empty()) {
            if (!comm->rxmgr->allocPages(1, &r->pages, r->pages_reserved >= 1)) return kSuccess;
            if (r->pages_reserved >= 1) --r->pages_reserved;
          }
          dst = comm->rxmgr->hostBase() + (uint64_t)r->pages[0].first * kRxPageBytes;
        }
        if (r->inline_off < r->size) r->inline_off += comm->ctrl_recv.drain(dst + r->inline_off, r->size - r->inline_off);
        if (r->inline_off < r->size) {
          Result sr = socketProgress(kSockRecv, comm->ctrl_fd, dst, r->size, &r->inline_off);
          if (sr != kSuccess) return sr;
          if (r->inline_off < r->size) return kSuccess;
        }
        if (r->mem_type == kPtrCuda) {
          if (comm->rxmgr->deviceResident()) {
            const uint64_t off = (uint64_t)r->pages[0].first * kRxPageBytes;
            TCPXB_CHECK(gpu::copyToDeviceAsync(comm->rxmgr->devBase() + off, comm->rxmgr->hostBase() + off, (size_t)r->size, comm->stream));
          }
          LoadMeta& m = r->slot.mem[r->slot.filled++];
          m.src_off = r->pages[0].first * kRxPageBytes;
          m.len = (uint32_t)r->size;
          m.dst_off = 0;
        }
        comm->ctrl_stats.bytes_done.fetch_add((uint64_t)r->size);
      }
      r->offset = r->size;
      r->size_pending = 0;
      comm->have_ctrl = false;
      traceReq(comm, r, kReqTransmitting);
      comm->rq.advance(kReqActive);
      return kSuccess;
    }
    TaskRing& tasks = comm->sock[c.index].tasks;
    if (!tasks.hasFree()) return kSuccess;  // keep the record; retry when a slot frees
    if (!fillRecvTask(comm, r, c.index, (int)c.size, (int)c.offset)) return kSuccess;  // pool full for now
    r->offset += (int)c.size;
    comm->have_ctrl = false;
    if (r->offset == r->size) {
      if (r->pages_reserved > 0) { comm->rxmgr->unreservePages(r->pages_reserved); r->pages_reserved = 0; }
      traceReq(comm, r, kReqTransmitting);
      comm->rq.advance(kReqActive);
      return kSuccess;
    }
  }
}

Result progressRound(Comm* comm) {
  mark(comm, "progress:enter");
  const int err = comm->error.load(std::memory_order_acquire);
  if (err != kSuccess) return (Result)err;
  if (comm->rq.empty()) return kSuccess;
  const Flags& f = flags();
  comm->mapper->reset();
  // 1. reap finished tasks, offer sockets with room
  for (int i = 0; i < comm->num_socks; ++i) {
    const int idx = (comm->rotate + i) % comm->num_socks;
    SocketCtx& s = comm->sock[idx];
    while (s.tasks.has(kTaskInactive)) {
      Task* t = &s.tasks.front(kTaskInactive);
      Request* r = t->r;
      r->size_pending -= t->size;
      if (t->op == kSockRecv && r->mem_type == kPtrCuda) TCPXB_CHECK(describePages(comm, r, t, idx));
      traceTask(comm, t, 0);
      s.tasks.advance(kTaskInactive);
      if (f.force_ack && t->op == kSockRecv && s.tasks.empty()) setQuickAck(s.fd);
    }
    if (s.tasks.hasFree()) comm->mapper->offer(idx, (int)(kMaxTasks - s.tasks.numFree()));
  }
  comm->rotate = (comm->rotate + 1) % comm->num_socks;
  mark(comm, "progress:posted");
  // 2. posted -> active (optionally synchronised: the receiver names the request it posted)
  while (comm->rq.has(kReqPosted)) {
    Request* r = &comm->rq.front(kReqPosted);
    if (f.recv_sync) {
      uint32_t idx = (uint32_t)comm->rq.frontIndex(kReqPosted);  // 32 bits on the wire
      if (r->op == kSockRecv) {
        Result sr = socketSend(comm->ctrl_fd, &idx, sizeof idx, 1000);
        if (sr != kSuccess) return sr == kInProgress ? kSystemError : sr;
      } else {
        // non-blocking: read what is there, finish next round
        Result sr = socketProgress(kSockRecv, comm->ctrl_fd, &r->sync_word, (int)sizeof r->sync_word, &r->sync_got);
        if (sr != kSuccess) return sr;
        if (r->sync_got < (int)sizeof r->sync_word) break;
        const uint32_t peer = r->sync_word;
        if (peer != idx) WARN("receive-sync mismatch: local request %u, peer %u", idx, peer);
      }
    }
    traceReq(comm, r, kReqActive);
    comm->rq.advance(kReqPosted);
  }
  mark(comm, "progress:schedule");
  // 3. schedule the active requests, oldest first
  if (!comm->passive && comm->ctrl_send.pending()) {
    Result fr = comm->ctrl_send.flush();
    if (fr != kInProgress) TCPXB_CHECK(fr);
  }
  while (comm->rq.has(kReqActive)) {
    Request* r = &comm->rq.front(kReqActive);
    const uint64_t before = comm->rq.frontIndex(kReqActive);
    if (r->op == kSockSend) {
      if (!comm->mapper->hasFlow() && r->size > f.inline_threshold && r->size != 0) break;
      TCPXB_CHECK(progressSendRequest(comm, r));
    } else {
      TCPXB_CHECK(progressRecvRequest(comm, r));
    }
    if (comm->rq.frontIndex(kReqActive) == before) break;  // no further progress possible now
  }
  mark(comm, "progress:finish");
  // 4. transmitting -> finished, in order
  while (comm->rq.has(kReqTransmitting)) {
    Request* r = &comm->rq.front(kReqTransmitting);
    if (!r->size_known || r->size_pending != 0) break;
    if (r->op == kSockRecv && r->mem_type == kPtrCuda) {
      if (comm->recv_mode == kRecvModeUnpack) {
        // publish the scatter list: records first, then the count
        std::atomic_thread_fence(std::memory_order_release);
        *r->slot.cnt = r->slot.filled;
        std::atomic_thread_fence(std::memory_order_seq_cst);
        if (comm->rxmgr->deviceResident()) {
          if (!r->unpack_launched) {
            TCPXB_CHECK(comm->unpack_marks.mark(comm->stream, &r->unpack_mark));  // behind the page placements
            r->unpack_launched = true;
          }
          if (!comm->unpack_marks.reached(r->unpack_mark)) break;
        }
      } else {
        if (!r->unpack_launched) TCPXB_CHECK(launchUnpack(comm, r));
        if (!comm->unpack_marks.reached(r->unpack_mark)) break;
        if (comm->unpack_status_host[0] != 0) {
          WARN("unpack kernel reported status %u at record %u", comm->unpack_status_host[0], comm->unpack_status_host[1]);
          return kInternalError;
        }
        releasePages(comm, r);
        comm->devq->release(r->slot.index);
        r->slot.active = false;
      }
    }
    if (r->op == kSockSend && r->mem_type == kPtrCuda && !comm->devmem) comm->tx_tail += r->stage_bytes;
    traceReq(comm, r, kReqFinished);
    comm->rq.advance(kReqTransmitting);
  }
  return kSuccess;
}

Result progress(Comm* comm) {
  const Result r = progressRound(comm);
  if (comm->kick_mask != 0) flushKicks(comm);  // helpers learn of this round's new tasks in one go
  return r;
}

// Frees finished requests from the head of the ring once the user has seen them
// (and, in unpack mode, has consumed the pages).
void retireRequests(Comm* comm) {
  while (comm->rq.has(kReqFinished)) {
    Request* r = &comm->rq.front(kReqFinished);
    if (!r->reported) break;
    const bool needs_consume = r->op == kSockRecv && r->mem_type == kPtrCuda && comm->recv_mode == kRecvModeUnpack;
    if (needs_consume && !r->consumed) break;
    traceReq(comm, r, 0);
    comm->rq.advance(kReqFinished);
  }
}

Result waitConnected(Comm* comm) {
  for (;;) {
    const int st = comm->conn_state.load(std::memory_order_acquire);
    if (st == kConnOk) return kSuccess;
    if (st == kConnFailed) return kRemoteError;
    if (!flags().spinwait_connect) return kInProgress;
    sched_yield();
  }
}

// A request that makes no progress for seconds gets its whole pipeline state
// logged (WARN), at most once per threshold: which ring stage it sits in, what the
// sockets' task rings hold, whether a control record is pending.
void reportStall(Comm* comm, Request* r) {
  const uint64_t now = monotonicNanos();
  const uint64_t first = (uint64_t)flags().timeout_threshold_ns, again = (uint64_t)flags().timeout_frequency_ns;
  if (now - r->posted_ns < first) return;
  if (r->last_stall_report_ns != 0 && now - r->last_stall_report_ns < again) return;
  r->last_stall_report_ns = now;
  std::string socks;
  for (int i = 0; i < comm->num_socks; ++i) {
    char b[96];
    TaskRing& t = comm->sock[i].tasks;
    snprintf(b, sizeof b, " s%d[a%u c%u i%u]", i, t.count(kTaskActive), t.count(kTaskCompleting), t.count(kTaskInactive));
    socks += b;
  }
  WARN("%s request %p (%s, %d bytes, %s memory) stalled %lu ms: offset %d pending %d size_known %d; ring posted %u active %u "
       "transmitting %u finished %u; ctrl pending %d have_ctrl %d;%s; error %d",
       comm->passive ? "recv" : "send", (void*)r, comm->ctrl_flow.c_str(), r->size, r->mem_type == kPtrCuda ? "cuda" : "host",
       (unsigned long)((now - r->posted_ns) / 1000000), r->offset, r->size_pending, (int)r->size_known,
       comm->rq.count(kReqPosted), comm->rq.count(kReqActive), comm->rq.count(kReqTransmitting), comm->rq.count(kReqFinished),
       (int)comm->ctrl_send.pending(), (int)comm->have_ctrl, socks.c_str(), comm->error.load());
}

Request* claimRequest(Comm* comm) {
  retireRequests(comm);
  if (!comm->rq.hasFree()) return nullptr;
  Request* r = &comm->rq.nextFree();
  std::vector<PageRun> pages = std::move(r->pages);
  pages.clear();
  *r = Request();
  r->pages = std::move(pages);  // keeps its capacity from one use of the slot to the next
  r->comm = comm;
  r->posted_ns = monotonicNanos();
  return r;
}

}  // namespace

// ------------------------------------------------------------------- public API
Result netInit(LoggerFn logger_fn) {
  if (logger_fn != nullptr) setLogger(logger_fn);
  std::lock_guard<std::mutex> l(cg.mu);
  reloadFlags();
  const Flags& f = flags();
  if (!f.enable) {
    INFO(kSubInit | kSubNet, "NET/GPUDirectTCPX-B200 disabled by NCCL_GPUDIRECTTCPX_SOCKET_ENABLE=0");
    return kInternalError;
  }
  if (cg.inited) return kSuccess;
  prctl(PR_SET_TIMERSLACK, 1, 0, 0, 0);
  TCPXB_CHECK(connectionInit());
  int ndev = 0;
  netDevices(&ndev);
  std::vector<std::string> names;
  for (int i = 0; i < ndev; ++i) names.push_back(netDevice(i)->nif.name);
  parseCoreRanges(f.tx_bindings.c_str(), names, &cg.tx_bind);
  parseCoreRanges(f.rx_bindings.c_str(), names, &cg.rx_bind);
  parseCoreRanges(f.tx_irq_bindings.c_str(), names, &cg.tx_irq_bind);
  parseCoreRanges(f.rx_irq_bindings.c_str(), names, &cg.rx_irq_bind);
  TraceConfig tc;
  tc.task_level = f.task_level_stats != 0;
  tc.request_level = f.request_level_stats != 0;
  tc.to_file = f.export_stats_to_file != 0;
  tc.sampling = (uint64_t)f.sampling_factor;
  setTraceConfig(tc);
  if (f.export_stats_to_file && f.file_life_min > 0)
    cg.gc = std::make_unique<LogGarbageCollector>(f.exporter_path, f.file_life_min, f.file_remove_frequency_s, (int)f.gc_core_index);
  if (f.report_lifecycle) {
    RxBufMgr* m = rxBufMgrFor(-1);
    if (m != nullptr && m->registerApplication((int)getpid()) == kSuccess) cg.registered_app = true;
  }
  INFO(kSubInit | kSubNet, "NET/GPUDirectTCPX-B200 ver. 0.1.0: %d device(s), scheduler %s, chunk %ld B, receive mode %s", ndev,
       f.sched_alg == kSchedKaty ? "KATY" : "RR", (long)f.dynamic_chunk_size, f.recv_mode == kRecvModeUnpack ? "unpack" : "host");
  cg.inited = true;
  return kSuccess;
}

Result netGetProperties(int dev, NetProperties* p) {
  const NetDevice* d = netDevice(dev);
  if (d == nullptr || p == nullptr) return kInvalidArgument;
  p->name = d->nif.name;
  p->pci_path = d->pci_path.empty() ? nullptr : d->pci_path.c_str();
  p->guid = (uint64_t)dev;
  // CUDA pointers are advertised in unpack mode (the consumer's kernel unpacks, the
  // plugin makes no CUDA call on the data path) and, on request, in host mode,
  // where the plugin itself queues copies and kernels from the caller's thread.
  const bool cuda_ptrs = gpu::devicePointersPossible() && (flags().recv_mode == kRecvModeUnpack || flags().cuda_buffers != 0);
  p->ptr_support = kPtrHost | (cuda_ptrs ? kPtrCuda : 0);
  p->speed_mbps = d->speed_mbps;
  p->port = 0;
  p->latency = 0;
  p->max_comms = 65536;
  p->max_recvs = 1;
  const bool unpack = flags().recv_mode == kRecvModeUnpack && gpu::devicePointersPossible();
  p->device_type = unpack ? 1 : 0;
  p->device_version = unpack ? kUnpackVersion : 0;
  return kSuccess;
}

Result startHelpers(Comm* comm) {
  if (comm->threads_started) return kSuccess;
  watchdogRegister(comm);
  const Flags& f = flags();
  if (traceConfig().to_file && (traceConfig().task_level || traceConfig().request_level)) {
    comm->events = std::make_unique<EventLog>(10000, (size_t)f.log_line_limit);
    char tag[32];
    snprintf(tag, sizeof tag, "%lx", (unsigned long)comm->id);
    comm->exporter = std::make_unique<Exporter>(comm->events.get(), f.exporter_path, tag, (int)f.exporter_core_index);
  }
  for (int t = 0; t < comm->num_threads; ++t) {
    comm->helpers[t].id = t;
    comm->helpers[t].thread = std::thread(helperMain, comm, t);
  }
  comm->threads_started = true;
  return kSuccess;
}

// Everything the CUDA data path needs, created while no kernel depends on this
// thread yet: stream, events of every request slot, staging or rx pool, and the
// kernels themselves (see tcpxb_kernels_preload).  Later calls are no-ops.
Result netPrepareCuda(Comm* comm, int gpu_dev) {
  if (comm == nullptr || comm->cuda_prepared) return kSuccess;
  if (gpu_dev < 0) gpu_dev = comm->gpu_dev;
  if (gpu_dev < 0 && gpu::currentDevice(&gpu_dev) != kSuccess) return kUnhandledCudaError;
  if (comm->passive) TCPXB_CHECK(ensureCudaRecv(comm, gpu_dev, comm->recv_mode == kRecvModeUnpack && comm->want_device_handle));
  else { TCPXB_CHECK(ensureCudaComm(comm, gpu_dev)); TCPXB_CHECK(ensureTxStage(comm)); }
  if (comm->passive && tcpxb_kernels_preload() != 0) {
    WARN("kernel preload failed: %s", tcpxb_kernel_last_error());
    return kUnhandledCudaError;
  }
  comm->cuda_prepared = true;
  return kSuccess;
}

Result netRegMr(Comm* comm, void* data, size_t size, int type, MemHandle** out) {
  if (out == nullptr) return kInvalidArgument;
  if (type != kPtrHost && type != kPtrCuda) { WARN("memory type %d is not supported", type); return kInvalidArgument; }
  auto* mh = new MemHandle{data, size, type, -1};
  if (type == kPtrCuda) {
    bool is_dev = false;
    gpu::pointerInfo(data, &mh->gpu_dev, &is_dev);
    if (!is_dev) {
      WARN("regMr: %p is not device memory", data);
      delete mh;
      return kInvalidArgument;
    }
    // registration happens during connection set-up, before any collective kernel
    // can be waiting on this thread: the right moment for allocations and loading
    if (comm != nullptr) TCPXB_CHECK(netPrepareCuda(comm, mh->gpu_dev));
    if (flags().rx_buf_mgr_devmem && flags().use_dma_buf != 0 && comm != nullptr && !comm->passive) {
      // devmem datapath, send side: the NIC reads transmit payload from the buffer itself, through a dma-buf
      if (flags().reg_dmabuf_use_internal_api != 0)
        WARN("NCCL_GPUDIRECTTCPX_REG_DMABUF_USE_INTERNAL_API=1 (driver procfs interface) is not offered; using the CUDA export call");
      Result er = cu::exportDmabuf(data, size, &mh->dmabuf_fd, &mh->dmabuf_offset);
      if (er != kSuccess) {
        WARN("regMr: dma-buf export of %p (+%zu) failed: %s", data, size, cu::lastError());
        delete mh;
        return er;
      }
      RxBufMgr* mgr = rxBufMgrFor(mh->gpu_dev);
      if (mgr == nullptr || mgr->bindTxDmabuf(mh->dmabuf_fd, &mh->dmabuf_id) != kSuccess) {
        WARN("regMr: the buffer manager could not bind the dma-buf for transmit");
        close(mh->dmabuf_fd);
        delete mh;
        return kSystemError;
      }
    }
  }
  *out = mh;
  return kSuccess;
}

Result netDeregMr(Comm* /*comm*/, MemHandle* mh) {
  if (mh != nullptr && mh->dmabuf_fd >= 0) close(mh->dmabuf_fd);
  delete mh;
  return kSuccess;
}

Result netIsend(Comm* comm, void* data, int size, int tag, MemHandle* mh, Request** out) {
  if (comm == nullptr || out == nullptr || size < 0) return kInvalidArgument;
  *out = nullptr;
  Result cr = waitConnected(comm);
  if (cr == kInProgress) return kSuccess;
  TCPXB_CHECK(cr);
  const int err = comm->error.load();
  if (err != kSuccess) return (Result)err;
  mark(comm, "isend:claim");
  Request* r = claimRequest(comm);
  if (r == nullptr) { mark(comm, "idle"); return kSuccess; }  // ring full: the caller retries
  r->op = kSockSend;
  r->data = static_cast<uint8_t*>(data);
  r->size = size;
  r->capacity = size;
  r->tag = tag;
  r->mem_type = mh != nullptr ? mh->type : kPtrHost;
  r->gpu_dev = mh != nullptr ? mh->gpu_dev : -1;
  r->size_pending = size;
  r->size_known = true;
  r->mh = mh;
  if (r->mem_type == kPtrCuda && comm->devmem) {
    if (mh == nullptr || mh->dmabuf_fd < 0) { WARN("devmem send of a buffer that was not registered as a dma-buf"); return kInvalidUsage; }
  } else if (r->mem_type == kPtrCuda) {
    mark(comm, "isend:startCudaSend");
    Result sr = startCudaSend(comm, r, mh);
    if (sr == kInProgress) { mark(comm, "idle"); return kSuccess; }  // staging ring full: retry later
    TCPXB_CHECK(sr);
  }
  traceReq(comm, r, kReqPosted);
  comm->rq.admit();
  *out = r;
  if (comm->api_calls++ < 3)
    TRACE(kSubNet, "send comm %lx: isend #%u of %d bytes (%s memory)", (unsigned long)comm->id, comm->api_calls, size,
         r->mem_type == kPtrCuda ? "cuda" : "host");
  Result pr = progress(comm);
  mark(comm, "idle");
  return pr;
}

Result netIrecv(Comm* comm, int n, void** data, int* sizes, int* tags, MemHandle** mhs, Request** out) {
  if (comm == nullptr || out == nullptr || n != 1) return kInvalidArgument;
  *out = nullptr;
  Result cr = waitConnected(comm);
  if (cr == kInProgress) return kSuccess;
  TCPXB_CHECK(cr);
  const int err = comm->error.load();
  if (err != kSuccess) return (Result)err;
  MemHandle* mh = mhs != nullptr ? mhs[0] : nullptr;
  const int mem_type = mh != nullptr ? mh->type : kPtrHost;
  if (mem_type == kPtrCuda) {
    TCPXB_CHECK(ensureCudaRecv(comm, mh->gpu_dev >= 0 ? mh->gpu_dev : comm->gpu_dev));
    if (comm->devq->inUse() >= (uint64_t)kUnpackQueueDepth) return kSuccess;  // consumer is behind
  }
  Request* r = claimRequest(comm);
  if (r == nullptr) return kSuccess;
  r->op = kSockRecv;
  r->data = static_cast<uint8_t*>(data[0]);
  r->capacity = sizes[0];
  r->size = sizes[0];
  r->tag = tags != nullptr ? tags[0] : 0;
  r->mem_type = mem_type;
  r->gpu_dev = mh != nullptr ? mh->gpu_dev : -1;
  r->size_pending = -1;
  r->size_known = false;
  if (mem_type == kPtrCuda) {
    comm->devq->nextFree(&r->slot);
    *r->slot.cnt = 0;
  }
  traceReq(comm, r, kReqPosted);
  comm->rq.admit();
  *out = r;
  if (comm->api_calls++ < 3)
    TRACE(kSubNet, "recv comm %lx: irecv #%u of up to %d bytes (%s memory)", (unsigned long)comm->id, comm->api_calls, sizes[0],
         mem_type == kPtrCuda ? "cuda" : "host");
  Result pr = progress(comm);
  mark(comm, "idle");
  return pr;
}

Result netIflush(Comm* /*comm*/, int /*n*/, void** /*data*/, int* /*sizes*/, MemHandle** /*mhs*/, Request** req) {
  // Data is made visible by stream order (copy engine or unpack kernel) before
  // test() reports completion; nothing is left to flush.
  if (req != nullptr) *req = nullptr;
  return kSuccess;
}

Result netTest(Request* r, int* done, int* size) {
  if (r == nullptr || done == nullptr) return kInvalidArgument;
  *done = 0;
  Comm* comm = r->comm;
  // Callers poll every outstanding request in turn (NCCL keeps up to eight per
  // comm).  Only the poll of the oldest request still unreported runs the progress
  // engine; the others just look whether they have finished.  Completion is in
  // order, so nothing a younger request could learn is missed.  A caller that keeps
  // polling a younger request alone still gets progress: every 32nd such poll drives.
  bool drives = true;
  {
    const uint32_t n = comm->rq.inFlight();
    const uint64_t base = comm->rq.frontIndex(kReqFinished);
    for (uint32_t k = 0; k < n; ++k) {
      Request* q = &comm->rq.slot(base + k);
      if (q->reported) continue;
      drives = (q == r);
      break;
    }
  }
  if (!drives && ++comm->polls_not_driving >= 32) drives = true;
  if (drives) {
    comm->polls_not_driving = 0;
    TCPXB_CHECK(progress(comm));
  } else {
    const int err = comm->error.load(std::memory_order_acquire);
    if (err != kSuccess) return (Result)err;
  }
  // finished = the request has left the transmitting stage
  bool finished = false;
  const uint32_t nfin = comm->rq.count(kReqFinished);
  for (uint32_t k = 0; k < nfin; ++k)
    if (&comm->rq.at(kReqFinished, k) == r) { finished = true; break; }
  mark(comm, "idle");
  if (!finished) {
    reportStall(comm, r);
    return kSuccess;
  }
  *done = 1;
  if (comm->done_calls++ < 3)
    TRACE(kSubNet, "%s comm %lx: request #%u done, %d bytes", comm->passive ? "recv" : "send", (unsigned long)comm->id,
         comm->done_calls, r->size);
  if (size != nullptr) *size = r->size;
  r->reported = true;
  retireRequests(comm);
  return kSuccess;
}

Result netGetDeviceHandle(Comm* comm, void** dev_handle, size_t* size) {
  if (comm == nullptr || dev_handle == nullptr) return kInvalidArgument;
  int cur = comm->gpu_dev;
  if (cur < 0 && gpu::currentDevice(&cur) != kSuccess) return kUnhandledCudaError;
  comm->want_device_handle = true;
  TCPXB_CHECK(ensureCudaRecv(comm, cur, /*want_device_handle=*/true));
  *dev_handle = comm->devq->deviceHandle();
  if (size != nullptr) *size = sizeof(UnpackDeviceHandle);
  return kSuccess;
}

Result netGetDeviceMr(Comm* /*comm*/, MemHandle* mh, void** dptr) {
  if (mh == nullptr || dptr == nullptr) return kInvalidArgument;
  *dptr = mh->ptr;  // the unpack consumer indexes the user buffer directly
  return kSuccess;
}

Result netIrecvConsumed(Comm* comm, int n, Request* r) {
  if (comm == nullptr || r == nullptr || n != 1) return kInvalidArgument;
  if (r->mem_type != kPtrCuda || comm->recv_mode != kRecvModeUnpack) { r->consumed = true; retireRequests(comm); return kSuccess; }
  if (!comm->devq->release(r->slot.index)) {
    WARN("irecvConsumed out of order: slot %lu is not the oldest", (unsigned long)r->slot.index);
    return kInvalidUsage;
  }
  releasePages(comm, r);
  r->slot.active = false;
  r->consumed = true;
  retireRequests(comm);
  return kSuccess;
}

void netSetSendDependency(Comm* comm, gpu::Event event) { comm->send_dependency = event; }

void netSetHelperNap(Comm* comm, int nap_us, int rounds) {
  if (comm == nullptr) return;
  comm->helper_nap_us.store(nap_us < 0 ? 0 : nap_us, std::memory_order_relaxed);
  comm->helper_nap_rounds.store(rounds < 0 ? 0 : rounds, std::memory_order_relaxed);
}

Result netSetTxStagingBytes(Comm* comm, uint64_t bytes) {
  if (comm == nullptr || comm->passive || bytes < 4096) return kInvalidArgument;
  if (comm->tx_stage != nullptr) return kInvalidUsage;  // already allocated
  comm->tx_stage_bytes = bytes;
  return kSuccess;
}

void netSetNotifier(Comm* comm, Notifier* notifier) {
  if (comm != nullptr) comm->notifier = notifier;
}

void netHintCtrlReadable(Comm* comm) {
  if (comm == nullptr) return;
  comm->ctrl_hinted = true;
  comm->ctrl_readable_hint = true;
}

int netCtrlPollFd(Comm* comm) {
  if (comm == nullptr || !comm->passive || comm->have_ctrl) return -1;
  if (comm->ctrl_recv.buffered() >= (int)sizeof(CtrlMsg)) return -1;
  return comm->ctrl_fd;
}

Result netRequestScatterList(Request* r, ScatterList* out) {
  if (r == nullptr || out == nullptr || r->op != kSockRecv || r->mem_type != kPtrCuda) return kInvalidArgument;
  out->host = r->slot.mem;
  out->dev = r->slot.mem_dev;
  out->count = r->slot.filled;
  out->pool_dev = r->comm->rxmgr->devBase();
  out->pool_bytes = r->comm->rxmgr->bytes();
  return kSuccess;
}

void netCommHelperWaits(Comm* comm, uint64_t* idle_ns, uint64_t* blocked_ns) {
  uint64_t idle = 0, blocked = 0;
  if (comm != nullptr) {
    for (int t = 0; t < comm->num_threads; ++t) {
      idle += comm->helpers[t].idle_ns.load(std::memory_order_relaxed);
      blocked += comm->helpers[t].blocked_ns.load(std::memory_order_relaxed);
    }
  }
  if (idle_ns != nullptr) *idle_ns = idle;
  if (blocked_ns != nullptr) *blocked_ns = blocked;
}

int netCommFlowCounters(Comm* comm, FlowCounters* out, int max) {
  int n = 0;
  for (int i = 0; i < comm->num_socks && n < max; ++i, ++n) {
    const FlowStats& s = comm->sock[i].stats;
    out[n] = {s.flow_id, s.bytes_posted.load(), s.bytes_done.load(), s.tx_cnt.load(), s.tx_completion_cnt.load(), s.rx_cnt.load()};
  }
  return n;
}

std::vector<std::string> netCommStatsLines(Comm* comm) {
  std::vector<std::string> lines;
  for (int i = 0; i < comm->num_socks; ++i) lines.push_back(flowStatsLine(comm->sock[i].stats, comm->sock[i].flow, comm->passive));
  return lines;
}

void freeComm(Comm* comm) {
  if (comm == nullptr) return;
  watchdogForget(comm);
  comm->stop.store(true, std::memory_order_release);
  if (comm->threads_started) {
    for (int t = 0; t < comm->num_threads; ++t) {
      { std::lock_guard<std::mutex> l(comm->helpers[t].mu); }
      comm->helpers[t].cv.notify_all();
      if (comm->helpers[t].thread.joinable()) comm->helpers[t].thread.join();
    }
  }
  if (comm->ctrl_fd >= 0) close(comm->ctrl_fd);
  for (int i = 0; i < kMaxSockets; ++i) {
    if (comm->sock[i].fd < 0) continue;
    if (comm->passive && comm->rxmgr != nullptr) comm->rxmgr->removeFlowRule(comm->sock[i].fd);
    close(comm->sock[i].fd);
  }
  if (comm->exporter) comm->exporter->stop();
  // anything still holding pool pages gives them back
  for (uint32_t i = 0; i < kMaxRequests; ++i) {
    Request& r = comm->rq.slot(i);
    if (comm->rxmgr != nullptr && !r.pages.empty()) comm->rxmgr->releasePages(r.pages.data(), r.pages.size());
    r.pages.clear();
    if (comm->rxmgr != nullptr && r.pages_reserved > 0) comm->rxmgr->unreservePages(r.pages_reserved);
    r.pages_reserved = 0;
  }
  for (int i = 0; i < kMaxSockets; ++i) {
    for (uint32_t k = 0; k < kMaxTasks; ++k) {
      Task& t = comm->sock[i].tasks.slot(k);
      if (comm->rxmgr != nullptr && !t.pages.empty()) comm->rxmgr->releasePages(t.pages.data(), t.pages.size());
      t.pages.clear();
    }
  }
  comm->devq.reset();
  gpu::hostFreeMapped(comm->tx_stage);
  gpu::hostFreeMapped(comm->unpack_status_host);
  gpu::streamDestroy(comm->stream);
  delete comm;
}

Result netClose(Comm* comm) {
  if (comm == nullptr) return kSuccess;
  const Flags& f = flags();
  if (comm->devq && comm->devq->inUse() != 0)
    WARN("closing a receive comm with %lu scatter lists not consumed", (unsigned long)comm->devq->inUse());
  uint64_t posted = 0, done = 0;
  for (int i = 0; i < comm->num_socks; ++i) {
    posted += comm->sock[i].stats.bytes_posted.load();
    done += comm->sock[i].stats.bytes_done.load();
  }
  INFO(kSubNet, "closing %s comm %lx: %lu bytes handed to the kernel, %lu completed, %d sockets", comm->passive ? "recv" : "send",
       (unsigned long)comm->id, (unsigned long)posted, (unsigned long)done, comm->num_socks);
  std::vector<std::string> lines = netCommStatsLines(comm);
  if (f.log_stats_to_stdout) {
    for (const auto& l : lines) printf("%s\n", l.c_str());
    fflush(stdout);
  }
  if (f.export_stats_to_file) {
    char tag[32];
    snprintf(tag, sizeof tag, "%lx", (unsigned long)comm->id);
    Exporter::writeStatsFile(Exporter::statsPath(f.exporter_path, tag), lines);
  }
  freeComm(comm);
  return kSuccess;
}

}  // namespace tcpxb
