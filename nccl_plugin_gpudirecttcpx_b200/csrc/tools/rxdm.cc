// Receive-datapath manager daemon: owns the rx page pools and the flow-steering and
// application tables, and serves them to plugin processes over AF_UNIX sockets.
//
//   tcpxb_rxdm --prefix /tmp/tcpxb --pool-mb 1024 [--max-rules 65536] [--device-pool]
//              [--wire proto [--gpu-pci ADDR,ADDR,...]] [--legacy-ipc-files]
//
// It stands in for the external daemon the reference depends on (reference:
// README.md:14-16 names it; its clients are src/rx_buf_mgr_client/*).  One pool per
// GPU PCI address, created on first request.  By default a pool is host memory (a
// memfd the plugin maps and registers with CUDA).  With --device-pool it is device
// memory of the GPU the request names, allocated through the driver's virtual memory
// API and handed out as a shareable file descriptor that the plugin imports and maps
// (reference: src/gpu/rx_pool.cu:62-124 asks the daemon for exactly this, and
// src/gpu/common.cu:25-65 imports it); the GPU build of this tool (tcpxb_rxdm_gpu) is
// the one that can do that on real hardware.  A client that registers keeps its connection open; when
// the connection closes the client is deregistered and its flow rules are dropped,
// which is how a crashed job is cleaned up.
//
// --legacy-ipc-files also serves the reference's older import path (reference:
// src/gpu/rx_pool.cu:30-55): for every GPU the daemon allocates a pool of ordinary device
// memory and leaves its 64-byte memory handle in <prefix>/nvdma-<pci>, where a plugin started
// with NCCL_TCPX_RXMEM_IMPORT_USE_GPU_PCI_CLIENT=0 opens it.
//
// --wire proto serves the reference's own wire format instead of this repository's
// fixed structs: protobuf `UnixSocketProto` bodies, one `get_gpu_fd_<pci>` /
// `get_gpu_metadata_<pci>` socket pair per GPU, "Ok." replies as raw bytes (reference:
// src/rx_buf_mgr_client/proto/unix_socket_proto.proto:17-70, rx_rule_client.cc:38-75,
// src/gpu/rx_pool.cu:62-124).  A plugin started with NCCL_GPUDIRECTTCPX_RXDM_WIRE=proto
// talks to it, and by the same messages to the daemon the reference was written for.
#include <poll.h>
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

#include "tcpxb/cu_driver.h"
#include "tcpxb/gpu.h"
#include "tcpxb/rxdm.h"
#include "tcpxb/rxdm_proto.h"

using namespace tcpxb;

namespace {

volatile sig_atomic_t g_stop = 0;
void onSignal(int) { g_stop = 1; }

struct Rule { RxdmFlowRule r; int owner_pid; };  // owner: the requesting process, from the socket's credentials
struct App { int pid; int cred_pid; };          // the pid the client stated, and the one the kernel vouches for
struct Pool {
  int fd = -1;
  uint64_t size = 0, align = 4096;
  int kind = kRxdmPoolHost;
  cu::SharedAllocation dev;  // device pools: the daemon's own mapping keeps the allocation alive
};

struct State {
  std::string prefix;
  uint64_t pool_bytes = 1ull << 30;
  size_t max_rules = 65536;
  bool device_pool = false;
  bool proto_wire = false;
  bool legacy_ipc_files = false;
  std::map<std::string, cu::IpcAllocation> ipc_pools;  // by PCI address; the handle files name them
  std::vector<std::string> gpu_pcis;  // proto wire: the GPUs that get a socket pair of their own
  std::vector<Rule> rules;
  std::map<int, App> apps;  // keep-alive connection fd -> application
  std::map<std::string, Pool> pools;
};

int listenOn(const std::string& path) {
  unlink(path.c_str());
  int fd = socket(AF_UNIX, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  struct sockaddr_un addr;
  memset(&addr, 0, sizeof addr);
  addr.sun_family = AF_UNIX;
  snprintf(addr.sun_path, sizeof addr.sun_path, "%s", path.c_str());
  if (bind(fd, (struct sockaddr*)&addr, sizeof addr) != 0 || listen(fd, 128) != 0) {
    close(fd);
    return -1;
  }
  return fd;
}

int peerPid(int fd) {
  struct ucred cred;
  socklen_t len = sizeof cred;
  return getsockopt(fd, SOL_SOCKET, SO_PEERCRED, &cred, &len) == 0 ? (int)cred.pid : -1;
}

// An application's keep-alive connection closed (or it deregistered): forget it and
// withdraw the flow rules its process installed and did not remove, as after a crash.
void dropApplication(State* st, std::map<int, App>::iterator it, const char* how);

RxdmMessage reply(int status, const char* text, uint64_t a = 0, uint64_t b = 0, uint64_t c = 0) {
  RxdmMessage m;
  memset(&m, 0, sizeof m);
  m.magic = kRxdmMagic;
  m.type = kRxdmReply;
  m.reply.status = status;
  snprintf(m.reply.text, sizeof m.reply.text, "%s", text);
  m.reply.a = a; m.reply.b = b; m.reply.c = c;
  return m;
}

Pool* poolFor(State* st, const std::string& pci) {
  auto it = st->pools.find(pci);
  if (it != st->pools.end()) return &it->second;
  Pool p;
  if (st->device_pool) {
    // the GPU whose PCI address the client named
    int dev = -1;
    for (int d = 0; d < gpu::deviceCount(); ++d)
      if (gpu::pciBusId(d) == pci) dev = d;
    if (dev < 0) { fprintf(stderr, "[rxdm] no GPU with PCI address %s\n", pci.c_str()); return nullptr; }
    if (cu::deviceInit(dev, /*owns_its_memory=*/true) != kSuccess || cu::sharedCreate(dev, st->pool_bytes, &p.dev, &p.fd) != kSuccess) {
      fprintf(stderr, "[rxdm] device pool on GPU %s failed: %s\n", pci.c_str(), cu::lastError());
      return nullptr;
    }
    p.size = p.dev.bytes;
    p.align = cu::sharedGranularity(dev);
    p.kind = kRxdmPoolDevice;
  } else {
    std::string name = "tcpxb-rxpool-" + pci;
    p.fd = memfd_create(name.c_str(), 0);
    if (p.fd < 0) return nullptr;
    if (ftruncate(p.fd, (off_t)st->pool_bytes) != 0) { close(p.fd); return nullptr; }
    p.size = st->pool_bytes;
  }
  fprintf(stderr, "[rxdm] pool for GPU %s: %lu MiB of %s memory\n", pci.c_str(), (unsigned long)(p.size >> 20),
          p.kind == kRxdmPoolDevice ? "device" : "host");
  st->pools[pci] = p;
  return &st->pools[pci];
}

void dropApplication(State* st, std::map<int, App>::iterator it, const char* how) {
  const App app = it->second;
  st->apps.erase(it);
  size_t dropped = 0;
  bool other_registration = false;
  for (const auto& kv : st->apps) other_registration = other_registration || kv.second.cred_pid == app.cred_pid;
  if (!other_registration && app.cred_pid > 0) {
    for (size_t i = 0; i < st->rules.size();) {
      if (st->rules[i].owner_pid == app.cred_pid) { st->rules.erase(st->rules.begin() + (long)i); ++dropped; }
      else ++i;
    }
  }
  fprintf(stderr, "[rxdm] application %d %s", app.pid, how);
  if (dropped) fprintf(stderr, "; %zu flow rule(s) of process %d withdrawn", dropped, app.cred_pid);
  fprintf(stderr, "\n");
}

bool sameRule(const RxdmFlowRule& a, const RxdmFlowRule& b) {
  return strcmp(a.src_ip, b.src_ip) == 0 && a.src_port == b.src_port && strcmp(a.dst_ip, b.dst_ip) == 0 &&
         a.dst_port == b.dst_port;
}

// Handles one request on a fresh connection; returns true when the connection
// must stay open (an application registration).
bool serve(State* st, UnixSocketConnection* c, const std::string& service) {
  RxdmMessage m;
  int passed = -1;
  if (c->recv(&m, &passed, 2000) != kSuccess) return false;
  if (passed >= 0) close(passed);
  switch (m.type) {
    case kRxdmFlowRule: {
      if (st->rules.size() >= st->max_rules) { c->send(reply(8, "resource exhausted")); return false; }
      m.rule.src_ip[sizeof m.rule.src_ip - 1] = 0;
      m.rule.dst_ip[sizeof m.rule.dst_ip - 1] = 0;
      m.rule.gpu_pci[sizeof m.rule.gpu_pci - 1] = 0;
      st->rules.push_back(Rule{m.rule, peerPid(c->fd())});
      c->send(reply(0, "Ok."));
      return false;
    }
    case kRxdmFlowRuleUninstall: {
      for (size_t i = 0; i < st->rules.size(); ++i)
        if (sameRule(st->rules[i].r, m.rule)) { st->rules.erase(st->rules.begin() + (long)i); c->send(reply(0, "Ok.")); return false; }
      c->send(reply(5, "no such rule"));
      return false;
    }
    case kRxdmGetGpuFd:
    case kRxdmGetGpuMetadata: {
      m.gpu.gpu_pci[sizeof m.gpu.gpu_pci - 1] = 0;
      Pool* p = poolFor(st, m.gpu.gpu_pci);
      if (p == nullptr) { c->send(reply(13, "pool creation failed")); return false; }
      if (m.type == kRxdmGetGpuFd) c->send(reply(0, "Ok.", p->size, p->align, (uint64_t)p->kind), p->fd);
      else c->send(reply(0, "Ok.", p->size, p->align, (uint64_t)p->kind));
      return false;
    }
    case kRxdmAppRegister: {
      if (m.app.register_client) {
        st->apps[c->fd()] = App{m.app.pid, peerPid(c->fd())};
        c->send(reply(0, "Ok."));
        return true;  // keep-alive connection
      }
      for (auto it = st->apps.begin(); it != st->apps.end();) {
        auto next = std::next(it);
        if (it->second.pid == m.app.pid) dropApplication(st, it, "deregistered");
        it = next;
      }
      c->send(reply(0, "Ok."));
      return false;
    }
    case kRxdmStatus:
      c->send(reply(0, "Ok.", st->rules.size(), st->apps.size(), st->pools.size()));
      return false;
    default:
      fprintf(stderr, "[rxdm] unknown request %u on %s\n", m.type, service.c_str());
      c->send(reply(3, "unknown request"));
      return false;
  }
}

RxdmFlowRule ruleFromProto(const rxproto::Message& m) {
  RxdmFlowRule r;
  memset(&r, 0, sizeof r);
  snprintf(r.src_ip, sizeof r.src_ip, "%s", m.src.ip.c_str());
  r.src_port = (uint16_t)m.src.port;
  snprintf(r.dst_ip, sizeof r.dst_ip, "%s", m.dst.ip.c_str());
  r.dst_port = (uint16_t)m.dst.port;
  r.flow_type = m.flow_type;
  r.queue_id = m.has_queue_id ? m.queue_id : -1;
  snprintf(r.gpu_pci, sizeof r.gpu_pci, "%s", m.gpu_pci_addr.c_str());
  return r;
}

rxproto::Message rawReply(const std::string& text) {
  rxproto::Message m;
  m.kind = rxproto::kRawBytes;
  m.raw_bytes = text;
  return m;
}

// The same services in the reference's wire format.  `service` is the socket's file name;
// the per-GPU sockets carry the PCI address after their last underscore-separated stem.
bool serveProto(State* st, rxproto::Connection* c, const std::string& service) {
  rxproto::Message m;
  int passed = -1;
  if (c->recv(&m, &passed, 2000) != kSuccess) return false;
  if (passed >= 0) { close(passed); return false; }
  if (service == "rx_rule_manager" || service == "rx_rule_uninstall") {
    if (m.kind != rxproto::kFlowSteerRule || !m.has_ntuple || !m.src.present || !m.dst.present) {
      c->sendMessage(rawReply("Invalid argument: the request carries no flow-steering rule"));
      return false;
    }
    const RxdmFlowRule r = ruleFromProto(m);
    if (service == "rx_rule_manager") {
      if (st->rules.size() >= st->max_rules) { c->sendMessage(rawReply("Resource exhausted: rule table full")); return false; }
      st->rules.push_back(Rule{r, peerPid(c->fd())});
      c->sendMessage(rawReply("Ok."));
      return false;
    }
    for (size_t i = 0; i < st->rules.size(); ++i)
      if (sameRule(st->rules[i].r, r)) { st->rules.erase(st->rules.begin() + (long)i); c->sendMessage(rawReply("Ok.")); return false; }
    c->sendMessage(rawReply("Not found: no such rule"));
    return false;
  }
  const std::string fd_stem = "get_gpu_fd_", md_stem = "get_gpu_metadata_";
  if (service.compare(0, fd_stem.size(), fd_stem) == 0 || service.compare(0, md_stem.size(), md_stem) == 0) {
    const bool want_fd = service.compare(0, fd_stem.size(), fd_stem) == 0;
    const std::string pci = service.substr(want_fd ? fd_stem.size() : md_stem.size());
    if (m.kind != rxproto::kRawBytes || m.raw_bytes != pci) {
      c->sendMessage(rawReply("Invalid argument: the request names another GPU than the socket"));
      return false;
    }
    Pool* p = poolFor(st, pci);
    if (p == nullptr) { c->sendMessage(rawReply("Internal: pool creation failed")); return false; }
    if (want_fd) { c->sendFd(p->fd); return false; }
    rxproto::GpuMemMetadata md;
    md.fd = p->fd;  // the daemon's own number, as the reference's daemon sends it; meaningless to the client
    md.size = p->size;
    md.align = p->align;
    c->sendMessage(rawReply(rxproto::encodeMetadata(md)));
    return false;
  }
  if (service == "rxdm_application_registry") {
    if (m.kind != rxproto::kAppRegister) { c->sendMessage(rawReply("Invalid argument: not a registration")); return false; }
    const int pid = peerPid(c->fd());
    if (m.register_client) {
      st->apps[c->fd()] = App{pid, pid};
      c->sendMessage(rawReply("Ok."));
      return true;  // keep-alive connection
    }
    for (auto it = st->apps.begin(); it != st->apps.end();) {
      auto next = std::next(it);
      if (it->second.cred_pid == pid) dropApplication(st, it, "deregistered");
      it = next;
    }
    c->sendMessage(rawReply("Ok."));
    return false;
  }
  c->sendMessage(rawReply("Unimplemented: unknown service"));
  return false;
}

}  // namespace

int main(int argc, char** argv) {
  State st;
  st.prefix = "/tmp";
  bool status_only = false;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    if (a == "--help" || a == "-h") {
      printf("usage: tcpxb_rxdm [--prefix DIR] [--pool-mb N] [--max-rules N] [--device-pool] [--wire native|proto] [--gpu-pci A,B,...] [--legacy-ipc-files]\n"
             "       tcpxb_rxdm --status [--prefix DIR]\n"
             "Serves the rx buffer manager's UNIX sockets under DIR (default /tmp) until SIGINT or SIGTERM;\n"
             "with --status asks a running daemon under DIR for its counters and prints one JSON line.\n"
             "--wire proto speaks the protobuf messages of Google's daemon, with one get_gpu_fd_<pci> / get_gpu_metadata_<pci>\n"
             "socket pair per GPU (--gpu-pci lists them; default: every GPU of the machine, or \"host\" without one).\n");
      return 0;
    }
    if (a == "--status") { status_only = true; continue; }
    if (a == "--device-pool") { st.device_pool = true; continue; }
    if (a == "--legacy-ipc-files") { st.legacy_ipc_files = true; continue; }
    if (i + 1 >= argc) { fprintf(stderr, "%s needs a value (see --help)\n", a.c_str()); return 2; }
    const char* v = argv[++i];
    if (a == "--prefix") st.prefix = v;
    else if (a == "--pool-mb") st.pool_bytes = strtoull(v, nullptr, 0) << 20;
    else if (a == "--max-rules") st.max_rules = strtoull(v, nullptr, 0);
    else if (a == "--wire") {
      if (!strcmp(v, "proto")) st.proto_wire = true;
      else if (strcmp(v, "native")) { fprintf(stderr, "--wire takes native or proto\n"); return 2; }
    } else if (a == "--gpu-pci") {
      std::string list = v;
      for (size_t pos = 0; pos <= list.size();) {
        size_t comma = list.find(',', pos);
        if (comma == std::string::npos) comma = list.size();
        if (comma > pos) st.gpu_pcis.push_back(list.substr(pos, comma - pos));
        pos = comma + 1;
      }
    }
    else { fprintf(stderr, "unknown argument %s (see --help)\n", a.c_str()); return 2; }
  }
  if (status_only) {
    RxdmMessage req, rep;
    memset(&req, 0, sizeof req);
    req.magic = kRxdmMagic;
    req.type = kRxdmStatus;
    if (rxdmCall(st.prefix, "rxdm_status", req, &rep, nullptr) != kSuccess) {
      fprintf(stderr, "no daemon answers under %s\n", st.prefix.c_str());
      return 1;
    }
    printf("{\"tool\": \"rxdm\", \"prefix\": \"%s\", \"flow_rules\": %lu, \"applications\": %lu, \"pools\": %lu}\n", st.prefix.c_str(),
           (unsigned long)rep.reply.a, (unsigned long)rep.reply.b, (unsigned long)rep.reply.c);
    return 0;
  }
  mkdir(st.prefix.c_str(), 0755);
  signal(SIGINT, onSignal);
  signal(SIGTERM, onSignal);
  signal(SIGPIPE, SIG_IGN);
  // fixed services; the per-GPU ones share a wildcard socket each: the client names the GPU in the request
  std::vector<std::string> services = {"rx_rule_manager", "rx_rule_uninstall", "get_gpu_fd", "get_gpu_metadata",
                                       "rxdm_application_registry", "rxdm_status"};
  if (st.proto_wire) {
    if (st.gpu_pcis.empty()) {
      for (int d = 0; d < gpu::deviceCount(); ++d) {
        const std::string pci = gpu::pciBusId(d);
        st.gpu_pcis.push_back(pci.empty() ? "gpu" + std::to_string(d) : pci);
      }
      if (st.gpu_pcis.empty()) st.gpu_pcis.push_back("host");
    }
    services = {"rx_rule_manager", "rx_rule_uninstall", "rxdm_application_registry", "rxdm_status"};
    for (const auto& pci : st.gpu_pcis) {
      services.push_back("get_gpu_fd_" + pci);
      services.push_back("get_gpu_metadata_" + pci);
    }
  }
  std::vector<int> lfds;
  for (const auto& s : services) {
    int fd = listenOn(st.prefix + "/" + s);
    if (fd < 0) { fprintf(stderr, "[rxdm] cannot listen on %s/%s\n", st.prefix.c_str(), s.c_str()); return 1; }
    lfds.push_back(fd);
  }
  if (st.legacy_ipc_files) {
    for (int d = 0; d < gpu::deviceCount(); ++d) {
      std::string pci = gpu::pciBusId(d);
      if (pci.empty()) pci = "gpu" + std::to_string(d);
      cu::IpcAllocation pool;
      unsigned char handle[cu::kIpcHandleBytes];
      if (cu::deviceInit(d, /*owns_its_memory=*/true) != kSuccess || cu::ipcCreate(d, st.pool_bytes, &pool, handle) != kSuccess) {
        fprintf(stderr, "[rxdm] memory-handle pool on GPU %s failed: %s\n", pci.c_str(), cu::lastError());
        return 1;
      }
      const std::string path = st.prefix + "/nvdma-" + pci;
      FILE* f = fopen(path.c_str(), "wb");
      if (f == nullptr || fwrite(handle, 1, sizeof handle, f) != sizeof handle) { fprintf(stderr, "[rxdm] cannot write %s\n", path.c_str()); return 1; }
      fclose(f);
      st.ipc_pools[pci] = pool;
      fprintf(stderr, "[rxdm] pool for GPU %s: %lu MiB of device memory, handle in %s\n", pci.c_str(), (unsigned long)(pool.bytes >> 20), path.c_str());
    }
    if (st.ipc_pools.empty()) { fprintf(stderr, "[rxdm] --legacy-ipc-files needs a GPU\n"); return 1; }
  }
  fprintf(stderr, "[rxdm] serving under %s (%s wire format)\n", st.prefix.c_str(), st.proto_wire ? "protobuf" : "native");
  printf("ready\n");
  fflush(stdout);
  std::vector<int> keep;  // registered applications' connections
  while (!g_stop) {
    std::vector<struct pollfd> pfds;
    for (int fd : lfds) pfds.push_back({fd, POLLIN, 0});
    for (int k : keep) pfds.push_back({k, POLLIN, 0});
    int pr = poll(pfds.data(), (nfds_t)pfds.size(), 500);
    if (pr <= 0) continue;
    size_t polled = keep.size();  // connections accepted below were not part of this poll
    for (size_t i = 0; i < lfds.size(); ++i) {
      if (!(pfds[i].revents & POLLIN)) continue;
      int cfd = accept(lfds[i], nullptr, nullptr);
      if (cfd < 0) continue;
      // the status service keeps this repository's framing in both modes (the reference has no such service)
      if (st.proto_wire && services[i] != "rxdm_status") {
        rxproto::Connection c(cfd);
        if (serveProto(&st, &c, services[i])) keep.push_back(c.release());
      } else {
        UnixSocketConnection c(cfd);
        if (serve(&st, &c, services[i])) keep.push_back(c.release());
      }
    }
    for (size_t k = 0; k < polled;) {
      const struct pollfd& p = pfds[lfds.size() + k];
      if (p.revents & (POLLIN | POLLHUP | POLLERR)) {
        char b;
        ssize_t n = recv(keep[k], &b, 1, MSG_DONTWAIT);
        if (n == 0 || (n < 0 && errno != EAGAIN)) {
          auto it = st.apps.find(keep[k]);
          if (it != st.apps.end()) dropApplication(&st, it, "went away");
          close(keep[k]);
          keep.erase(keep.begin() + (long)k);
          pfds.erase(pfds.begin() + (long)(lfds.size() + k));
          --polled;
          continue;
        }
      }
      ++k;
    }
  }
  for (int k : keep) close(k);
  for (size_t i = 0; i < lfds.size(); ++i) { close(lfds[i]); unlink((st.prefix + "/" + services[i]).c_str()); }
  for (auto& p : st.pools) {
    close(p.second.fd);
    cu::sharedRelease(&p.second.dev);
  }
  for (auto& p : st.ipc_pools) {
    unlink((st.prefix + "/nvdma-" + p.first).c_str());
    cu::ipcRelease(&p.second);
  }
  return 0;
}
