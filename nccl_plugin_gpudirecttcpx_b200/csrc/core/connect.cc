// Connection layer: device table, listen, asynchronous connect / accept.
//
// Sequence per communicator (reference: src/connect.cc:373-506 handshake with
// retry, :600-667 and :736-817 the two asynchronous sides, :515-560 listen): the
// control socket is established first, then the data sockets from the highest
// index down.  For every socket the accepting side sends its 4-byte connection
// state and reads the connector's; once the control socket exists these exchanges
// travel on it.  The connector then names the socket's index (4 bytes, control
// socket; `num_socks` designates the control socket itself).  A failed exchange is
// retried up to CONNECTION_RETRY times.  Nothing sleeps unless CONNECT_PACING_US or
// PROGRAM_FLOW_STEERING_WAIT_MICROS ask for it.
#include <limits.h>
#include <stdio.h>
#include <stdlib.h>
#include <unistd.h>

#include <map>
#include <set>

#include "tcpxb/transport.h"

namespace tcpxb {

namespace {

struct Global {
  std::mutex mu;
  bool ready = false;
  std::vector<NetDevice> devs;
  NetDevice ctrl_dev;
  bool has_ctrl_dev = false;
  std::atomic<uint64_t> next_comm_id{1};
  std::atomic<uint32_t> tx_stride{0}, rx_stride{0};
};
Global g;

std::string pciPathOf(const char* ifname) {
  std::string name(ifname);
  if (name.find('#') != std::string::npos) return "";  // virtual devices have no PCI parent
  std::string link = "/sys/class/net/" + name + "/device";
  char buf[PATH_MAX];
  if (realpath(link.c_str(), buf) == nullptr) return "";
  return buf;
}

int pciVendorOf(const std::string& pci_path) {
  if (pci_path.empty()) return 0;
  FILE* f = fopen((pci_path + "/vendor").c_str(), "r");
  if (f == nullptr) return 0;
  int v = 0;
  if (fscanf(f, "%i", &v) != 1) v = 0;
  fclose(f);
  return v;
}

// State shared between the caller that polls and the thread that connects.
struct AsyncSetup {
  std::thread thread;
  std::atomic<bool> done{false};
  Result result = kSuccess;
  Comm* comm = nullptr;
};
std::mutex g_async_mu;
std::set<AsyncSetup*> g_async;  // live states, so a stale pointer in a handle is never trusted

void pace() {
  const int64_t us = flags().connect_pacing_us;
  if (us > 0) usleep((useconds_t)us);
}

Result exchangeStateAcceptor(int fd, int mine, int* theirs) {
  TCPXB_CHECK(socketSend(fd, &mine, sizeof mine, 10000));
  Result r = socketRecv(fd, theirs, sizeof *theirs, 10000);
  return r == kInProgress ? kSystemError : r;
}
Result exchangeStateConnector(int fd, int mine, int* theirs) {
  Result r = socketRecv(fd, theirs, sizeof *theirs, 10000);
  if (r != kSuccess) return r == kInProgress ? kSystemError : r;
  return socketSend(fd, &mine, sizeof mine, 10000);
}

// Receive-queue bookkeeping per device: which NAPI ids the accepted sockets landed
// on, to show how evenly flows spread over the NIC's receive queues
// (reference: src/connect.cc:474-486, NIC_N_RXQS).
struct NapiRecord {
  std::mutex mu;
  std::map<int, size_t> count;
};
NapiRecord g_napi[kMaxIfs];

// Where the kernel last processed this socket (diagnostics only; loopback has no
// NAPI id and reports 0).  Reference: src/connect.cc:314-336.
void logSocketLocality(Comm* comm, int index, int fd, bool is_ctrl) {
  int cpu = -1, napi = -1;
  socklen_t len = sizeof cpu;
#ifdef SO_INCOMING_CPU
  if (getsockopt(fd, SOL_SOCKET, SO_INCOMING_CPU, &cpu, &len) != 0) cpu = -1;
#endif
#ifdef SO_INCOMING_NAPI_ID
  len = sizeof napi;
  if (getsockopt(fd, SOL_SOCKET, SO_INCOMING_NAPI_ID, &napi, &len) != 0) napi = -1;
#endif
  if (comm->passive && !is_ctrl && napi > 0 && comm->dev >= 0 && comm->dev < kMaxIfs) {
    NapiRecord& rec = g_napi[comm->dev];
    std::lock_guard<std::mutex> l(rec.mu);
    const size_t n = ++rec.count[napi];
    if (rec.count.size() > (size_t)flags().nic_n_rxqs)
      INFO(kSubNet, "device %d: %zu distinct NAPI ids seen, more than NIC_N_RXQS=%ld", comm->dev, rec.count.size(),
           (long)flags().nic_n_rxqs);
    TRACE(kSubNet, "device %d: NAPI id %d now carries %zu flows", comm->dev, napi, n);
  }
  if (is_ctrl && !flags().ctrl_sockcond.empty())
    INFO(kSubNet, "comm %lx ctrl socket: incoming cpu %d napi %d (CTRL_SOCKCOND=%s: checked, not enforced)",
         (unsigned long)comm->id, cpu, napi, flags().ctrl_sockcond.c_str());
  TRACE(kSubNet, "comm %lx %s socket %d: incoming cpu %d napi %d", (unsigned long)comm->id, is_ctrl ? "ctrl" : "data", index, cpu,
        napi);
}

void attachSocket(Comm* comm, int index, int fd) {
  SocketCtx& s = comm->sock[index];
  logSocketLocality(comm, index, fd, false);
  s.fd = fd;
  // Bounded socket buffers keep the bytes a stream holds inside the kernel, and with them
  // the pages its skbs cycle through, small enough to stay in the caches.
  const int sndbuf = (int)flags().socket_sndbuf, rcvbuf = (int)flags().socket_rcvbuf;
  if (sndbuf > 0 && setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &sndbuf, sizeof sndbuf) != 0) WARN("SO_SNDBUF %d failed: %s", sndbuf, strerror(errno));
  if (rcvbuf > 0 && setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &rcvbuf, sizeof rcvbuf) != 0) WARN("SO_RCVBUF %d failed: %s", rcvbuf, strerror(errno));
  s.flow = flowString(fd, comm->passive);
  s.stats.flow_id = flowIdOf(s.flow);
  s.stall.configure((uint64_t)flags().timeout_threshold_ns, (uint64_t)flags().timeout_frequency_ns);
  s.tasks.reset();
}

void attachCtrl(Comm* comm, int fd) {
  logSocketLocality(comm, -1, fd, true);
  comm->ctrl_fd = fd;
  comm->ctrl_flow = flowString(fd, comm->passive);
  comm->ctrl_stats.flow_id = flowIdOf(comm->ctrl_flow);
  comm->ctrl_send.attach(fd);
  comm->ctrl_recv.attach(fd);
  comm->ctrl_stall.configure((uint64_t)flags().timeout_threshold_ns, (uint64_t)flags().timeout_frequency_ns);
}

void connectThread(AsyncSetup* st, Handle h, int dev) {
  Comm* comm = st->comm;
  const NetDevice& nd = g.devs[dev];
  const SocketAddress* local_data = &nd.nif.addr;
  const SocketAddress* local_ctrl = (h.redirect_ctrl && g.has_ctrl_dev) ? &g.ctrl_dev.nif.addr : local_data;
  Result res = kSuccess;
  // i == num_socks is the control socket, then data sockets num_socks-1 .. 0
  for (int i = h.num_socks; i >= 0 && res == kSuccess; --i) {
    const bool is_ctrl = (i == h.num_socks);
    int fd = -1;
    int tries = 0;
    for (;;) {
      pace();
      res = connectAddress(&fd, is_ctrl ? h.ctrl_addr : h.connect_addr, is_ctrl ? local_ctrl : local_data);
      if (res != kSuccess) break;
      int theirs = kConnFailed;
      const int xfd = is_ctrl ? fd : comm->ctrl_fd;
      res = exchangeStateConnector(xfd, kConnOk, &theirs);
      if (res == kSuccess && theirs == kConnOk) break;
      close(fd);
      fd = -1;
      if (++tries > flags().connection_retry) {
        WARN("handshake with %s failed after %d tries", addressToString(h.connect_addr).c_str(), tries);
        res = (res == kSuccess) ? kRemoteError : res;
        break;
      }
      res = kSuccess;
    }
    if (res != kSuccess) break;
    if (is_ctrl) {
      attachCtrl(comm, fd);
    } else {
      if (flags().min_zcopy_size > 0) {
        int one = 1;
        comm->sock[i].zerocopy_enabled = setsockopt(fd, SOL_SOCKET, SO_ZEROCOPY, &one, sizeof one) == 0;
      }
      attachSocket(comm, i, fd);
    }
    int index = i;
    res = socketSend(comm->ctrl_fd, &index, sizeof index, 10000);
  }
  if (res == kSuccess) {
    comm->peer_addr = h.connect_addr;
    INFO(kSubNet, "send comm %lx connected to %s: %d sockets, %d threads", (unsigned long)comm->id,
         addressToString(h.connect_addr).c_str(), comm->num_socks, comm->num_threads);
    comm->conn_state.store(kConnOk, std::memory_order_release);
  } else {
    comm->conn_state.store(kConnFailed, std::memory_order_release);
  }
  st->result = res;
  st->done.store(true, std::memory_order_release);
}

void acceptThread(AsyncSetup* st, ListenComm* l) {
  Comm* comm = st->comm;
  Result res = kSuccess;
  const int n = l->num_socks;
  for (int k = n; k >= 0 && res == kSuccess; --k) {
    const bool is_ctrl = (k == n);
    int fd = -1;
    int tries = 0;
    for (;;) {
      pace();
      do {
        res = acceptSocket(is_ctrl ? l->ctrl_fd : l->data_fd, &fd, 200);
        if (comm->stop.load()) res = kSystemError;
      } while (res == kInProgress);
      if (res != kSuccess) break;
      if (is_ctrl) setNoDelay(fd);
      Result cond = kSuccess;
      if (!is_ctrl && comm->rxmgr != nullptr)
        cond = comm->rxmgr->installFlowRule(fd, comm->gpu_dev >= 0 ? gpu::pciBusId(comm->gpu_dev) : "");
      int theirs = kConnFailed;
      const int xfd = is_ctrl ? fd : comm->ctrl_fd;
      res = exchangeStateAcceptor(xfd, cond == kSuccess ? kConnOk : kConnFailed, &theirs);
      if (res == kSuccess && cond == kSuccess && theirs == kConnOk) break;
      if (!is_ctrl && comm->rxmgr != nullptr) comm->rxmgr->removeFlowRule(fd);
      close(fd);
      fd = -1;
      if (++tries > flags().connection_retry) {
        res = (res == kSuccess) ? kRemoteError : res;
        break;
      }
      res = kSuccess;
    }
    if (res != kSuccess) break;
    if (is_ctrl) attachCtrl(comm, fd);
    int index = -1;
    res = socketRecv(comm->ctrl_fd, &index, sizeof index, 10000);
    if (res == kInProgress) res = kSystemError;
    if (res != kSuccess) break;
    if (is_ctrl) {
      if (index != n) { WARN("connector announced control index %d, expected %d", index, n); res = kRemoteError; }
    } else if (index < 0 || index >= n || comm->sock[index].fd != -1) {
      WARN("connector announced bad data socket index %d", index);
      close(fd);
      res = kRemoteError;
    } else {
      attachSocket(comm, index, fd);
    }
  }
  if (res == kSuccess) {
    const int64_t wait_us = flags().flow_steering_wait_us;
    if (wait_us > 0) usleep((useconds_t)wait_us);
    INFO(kSubNet, "recv comm %lx accepted %s: %d sockets, %d threads, gpu %d", (unsigned long)comm->id, comm->ctrl_flow.c_str(),
         comm->num_socks, comm->num_threads, comm->gpu_dev);
    comm->conn_state.store(kConnOk, std::memory_order_release);
  } else {
    comm->conn_state.store(kConnFailed, std::memory_order_release);
  }
  st->result = res;
  st->done.store(true, std::memory_order_release);
}

// Returns true when the setup finished; then *out and *res are final.
bool finishAsync(AsyncSetup* st, Comm** out, Result* res) {
  if (!st->done.load(std::memory_order_acquire)) return false;
  if (st->thread.joinable()) st->thread.join();
  *res = st->result;
  if (st->result == kSuccess) {
    *out = st->comm;
  } else {
    freeComm(st->comm);
    *out = nullptr;
  }
  {
    std::lock_guard<std::mutex> l(g_async_mu);
    g_async.erase(st);
  }
  delete st;
  return true;
}

}  // namespace

std::string handleToString(const Handle& h) {
  char buf[256];
  snprintf(buf, sizeof buf, "data %s ctrl %s%s ports %d+%d socks %d threads %d", addressToString(h.connect_addr).c_str(),
           addressToString(h.ctrl_addr).c_str(), h.redirect_ctrl ? " (redirected)" : "", h.port_start, h.port_count,
           h.num_socks, h.num_threads);
  return buf;
}

void chooseSocksThreads(int dev, int* nsocks, int* nthreads) {
  const Flags& f = flags();
  int threads = (int)f.nthreads, per_thread = (int)f.nsocks_per_thread;
  if (threads == -2 || per_thread == -2) {
    int auto_threads = 1, auto_per = 1;
    const int vendor = pciVendorOf(g.devs[dev].pci_path);
    if (vendor == 0x1d0f) { auto_threads = 2; auto_per = 8; }        // AWS
    else if (vendor == 0x1ae0) { auto_threads = 6; auto_per = 1; }   // GCP
    else if (g.devs[dev].pci_path.empty()) { auto_threads = 4; auto_per = 1; }  // loopback / veth: CPU bound
    if (threads == -2) threads = auto_threads;
    if (per_thread == -2) per_thread = auto_per;
  }
  if (threads < 0) threads = 1;
  if (threads > kMaxThreads) threads = kMaxThreads;
  if (per_thread < 0) per_thread = 1;
  // zero threads means the proxy thread drives one socket itself; keep one helper
  if (threads == 0) threads = 1;
  if (per_thread == 0) per_thread = 1;
  if (threads * per_thread > kMaxSockets) {
    if (threads > kMaxSockets) threads = kMaxSockets;
    per_thread = kMaxSockets / threads;
    if (per_thread < 1) per_thread = 1;
  }
  *nthreads = threads;
  *nsocks = threads * per_thread;
}

Result connectionInit() {
  std::lock_guard<std::mutex> l(g.mu);
  if (g.ready) return kSuccess;
  const Flags& f = flags();
  if (f.flow_steering_strategy != 3)
    WARN("FLOW_STEERING_STRATEGY=%ld is not offered; rules go through the rx buffer manager", (long)f.flow_steering_strategy);
  if (!f.port_mapping.empty())
    INFO(kSubInit, "PORT_MAPPING='%s' noted; the fixed-port strategy is not offered", f.port_mapping.c_str());
  const int family = envSocketFamily(f.socket_family);
  if (!f.ctrl_dev.empty()) {
    std::vector<NetIf> c = findInterfaces(f.ctrl_dev.c_str(), family, nullptr, 1);
    if (!c.empty()) {
      g.ctrl_dev.nif = c[0];
      g.ctrl_dev.pci_path = pciPathOf(c[0].name);
      g.has_ctrl_dev = true;
      INFO(kSubInit, "control sockets use %s (%s)", c[0].name, addressToString(c[0].addr, false).c_str());
    } else {
      WARN("control interface '%s' not found; control sockets share the data interface", f.ctrl_dev.c_str());
    }
  }
  std::vector<NetIf> ifs = findInterfaces(f.socket_ifname.c_str(), family, f.net_comm_id.c_str(), kMaxIfs);
  if (ifs.empty()) {
    WARN("no usable network interface found");
    return kInternalError;
  }
  std::vector<NetIf> all;
  if (f.virtual_nics > 0) {
    // spread the requested count over the interfaces found
    const int per = ((int)f.virtual_nics + (int)ifs.size() - 1) / (int)ifs.size();
    for (const NetIf& n : ifs)
      for (const NetIf& v : expandVirtual(n, per))
        if ((int)all.size() < (int)f.virtual_nics && (int)all.size() < kMaxIfs) all.push_back(v);
  } else {
    all = ifs;
  }
  g.devs.clear();
  for (const NetIf& n : all) {
    NetDevice d;
    d.nif = n;
    d.pci_path = pciPathOf(n.name);
    int sp = f.nic_speed_mbps > 0 ? (int)f.nic_speed_mbps : interfaceSpeedMbps(n.name);
    d.speed_mbps = sp > 0 ? sp : 10000;
    g.devs.push_back(d);
    INFO(kSubInit | kSubNet, "NET/GPUDirectTCPX-B200: device %zu = %s (%s) pci '%s' speed %d Mb/s", g.devs.size() - 1,
         n.name, addressToString(n.addr, false).c_str(), d.pci_path.c_str(), d.speed_mbps);
  }
  g.ready = true;
  return kSuccess;
}

Result netDevices(int* ndev) {
  *ndev = (int)g.devs.size();
  return kSuccess;
}

const NetDevice* netDevice(int dev) {
  if (dev < 0 || dev >= (int)g.devs.size()) return nullptr;
  return &g.devs[dev];
}

Result netListen(int dev, void* opaque, ListenComm** out) {
  if (dev < 0 || dev >= (int)g.devs.size() || opaque == nullptr || out == nullptr) return kInvalidArgument;
  Handle* h = static_cast<Handle*>(opaque);
  memset(h, 0, sizeof *h);
  auto l = std::make_unique<ListenComm>();
  l->dev = dev;
  chooseSocksThreads(dev, &l->num_socks, &l->num_threads);
  h->connect_addr = g.devs[dev].nif.addr;
  setAddressPort(&h->connect_addr, 0);
  TCPXB_CHECK(createListenSocket(&l->data_fd, &h->connect_addr));
  h->redirect_ctrl = g.has_ctrl_dev;
  h->ctrl_addr = g.has_ctrl_dev ? g.ctrl_dev.nif.addr : g.devs[dev].nif.addr;
  setAddressPort(&h->ctrl_addr, 0);
  Result r = createListenSocket(&l->ctrl_fd, &h->ctrl_addr);
  if (r != kSuccess) { close(l->data_fd); return r; }
  h->num_socks = l->num_socks;
  h->num_threads = l->num_threads;
  h->port_start = addressPort(h->connect_addr);
  h->port_count = 1;
  h->connect_args = nullptr;
  TRACE(kSubNet, "listening: %s", handleToString(*h).c_str());
  *out = l.release();
  return kSuccess;
}

Result netConnect(int dev, void* opaque, Comm** out) {
  if (dev < 0 || dev >= (int)g.devs.size() || opaque == nullptr || out == nullptr) return kInvalidArgument;
  *out = nullptr;
  Handle* h = static_cast<Handle*>(opaque);
  AsyncSetup* st = static_cast<AsyncSetup*>(h->connect_args);
  if (st != nullptr) {
    std::lock_guard<std::mutex> l(g_async_mu);
    if (g_async.count(st) == 0) st = nullptr;  // not ours: a handle copied from a peer
  }
  if (st == nullptr) {
    if (h->num_socks < 1 || h->num_socks > kMaxSockets || h->num_threads < 1 || h->num_threads > kMaxThreads) {
      WARN("connect handle carries %d sockets x %d threads", h->num_socks, h->num_threads);
      return kInvalidArgument;
    }
    st = new AsyncSetup();
    st->comm = newComm(dev, /*passive=*/false);
    st->comm->num_socks = h->num_socks;
    st->comm->num_threads = h->num_threads;
    st->comm->stride = g.tx_stride.fetch_add(1);
    {
      std::lock_guard<std::mutex> l(g_async_mu);
      g_async.insert(st);
    }
    h->connect_args = st;
    Handle copy = *h;
    st->thread = std::thread(connectThread, st, copy, dev);
    return kSuccess;
  }
  Result res = kSuccess;
  if (finishAsync(st, out, &res)) {
    h->connect_args = nullptr;
    if (res == kSuccess) res = startHelpers(*out);
    return res;
  }
  return kSuccess;
}

namespace {
struct AcceptExtras { int recv_mode = -1; };
std::mutex g_extras_mu;
std::map<ListenComm*, AcceptExtras>* g_extras = nullptr;
}  // namespace

void netSetAcceptRecvMode(ListenComm* lcomm, int recv_mode) {
  std::lock_guard<std::mutex> l(g_extras_mu);
  if (g_extras == nullptr) g_extras = new std::map<ListenComm*, AcceptExtras>();
  (*g_extras)[lcomm].recv_mode = recv_mode;
}

Result netAccept(ListenComm* l, Comm** out) {
  if (l == nullptr || out == nullptr) return kInvalidArgument;
  *out = nullptr;
  AsyncSetup* st = static_cast<AsyncSetup*>(l->accept_state);
  if (st == nullptr) {
    st = new AsyncSetup();
    st->comm = newComm(l->dev, /*passive=*/true);
    st->comm->num_socks = l->num_socks;
    st->comm->num_threads = l->num_threads;
    st->comm->stride = g.rx_stride.fetch_add(1);
    st->comm->recv_mode = flags().recv_mode;
    {
      std::lock_guard<std::mutex> lk(g_extras_mu);
      if (g_extras != nullptr) {
        auto it = g_extras->find(l);
        if (it != g_extras->end() && it->second.recv_mode >= 0) st->comm->recv_mode = it->second.recv_mode;
      }
    }
    // The rx pool belongs to the GPU that is current on the accepting thread.
    if (gpu::available()) {
      int cur = -1;
      if (gpu::currentDevice(&cur) == kSuccess) st->comm->gpu_dev = cur;
    }
    {
      std::lock_guard<std::mutex> lk(g_async_mu);
      g_async.insert(st);
    }
    l->accept_state = st;
    st->thread = std::thread(acceptThread, st, l);
    return kSuccess;
  }
  Result res = kSuccess;
  if (finishAsync(st, out, &res)) {
    l->accept_state = nullptr;
    if (res == kSuccess) res = startHelpers(*out);
    return res;
  }
  return kSuccess;
}

Result netCloseListen(ListenComm* l) {
  if (l == nullptr) return kSuccess;
  AsyncSetup* st = static_cast<AsyncSetup*>(l->accept_state);
  if (st != nullptr) {
    st->comm->stop.store(true);
    if (st->thread.joinable()) st->thread.join();
    freeComm(st->comm);
    std::lock_guard<std::mutex> lk(g_async_mu);
    g_async.erase(st);
    delete st;
  }
  {
    std::lock_guard<std::mutex> lk(g_extras_mu);
    if (g_extras != nullptr) g_extras->erase(l);
  }
  if (l->data_fd >= 0) close(l->data_fd);
  if (l->ctrl_fd >= 0) close(l->ctrl_fd);
  delete l;
  return kSuccess;
}

Comm* newComm(int dev, bool passive) {
  Comm* c = new Comm();
  c->dev = dev;
  c->passive = passive;
  c->devmem = flags().rx_buf_mgr_devmem;
  c->helper_nap_us.store((int)flags().helper_nap_us);
  c->helper_nap_rounds.store((int)flags().helper_nap_rounds);
  c->id = g.next_comm_id.fetch_add(1);
  c->mapper = makeFlowMapper(flags().sched_alg);
  c->rq.reset();
  return c;
}

void netResetForTests() {
  std::lock_guard<std::mutex> l(g.mu);
  g.ready = false;
  g.devs.clear();
  g.has_ctrl_dev = false;
}

}  // namespace tcpxb
