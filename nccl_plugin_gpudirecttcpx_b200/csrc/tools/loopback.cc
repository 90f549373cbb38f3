// Stand-alone driver of the ncclNet table: two processes on one machine exchange
// seeded random payloads through the plugin, with no NCCL and no GPU involved.
//
//   tcpxb_loopback --plugin <libnccl-net.so | libtcpxb_host.so> [--v7]
//                  [--sizes 1024,65536,4194304,67108864] [--inflight 8] [--iters 4]
//                  [--ptr host|cuda] [--yield] [--random-sizes] [--thread-times]
//                  [--comms-per-dev N]
//
// `--random-sizes`: each listed size is the capacity of the posted receives; every message
// carries a seeded random number of bytes between 0 and that capacity (both sides derive
// it from the key), as under NCCL, which posts the largest size a step may bring.  The
// receiver checks the size test() reports and that nothing beyond it was written.
//
// `--yield` makes the polling loop call sched_yield() after a pass that neither posted
// nor finished anything, as NCCL's proxy thread does; without it the loop spins.
//
// `--ptr cuda` registers the buffers as device memory.  It is meant for the host-only
// library started with TCPXB_FAKE_GPU=1, whose stand-in device is host memory: the
// sender then goes through the staging ring and the receiver through the page pool
// and the scatter lists.  When the plugin hands out an unpack device handle
// (NCCL_GPUDIRECTTCPX_RECV_MODE=unpack) the receiver also plays the part of NCCL's
// unpack consumer: for each finished receive it advances the handle's head, reads
// that slot's count and records from the mapped block, copies the fragments out of
// the bounce buffer and only then calls irecvConsumed.
//
// The parent is the receiver, the forked child the sender.  One comm (or
// --comms-per-dev of them) is opened per device the plugin reports (set NCCL_GPUDIRECTTCPX_VIRTUAL_NICS=2 to get two
// "NICs" on lo); every comm moves `inflight` messages per iteration with tags
// 0..inflight-1.  Payload bytes are a pure function of (seed, comm, iteration,
// tag), so the receiver regenerates and compares them byte for byte.  At the end
// each side prints per-flow byte counters and one JSON line per size.
// The reference has no such tool: its only tests are two unit tests of the stats
// code (reference: src/stats/tracepoint_test.cc, src/stats/stats_buffer_test.cc).
#include <dirent.h>
#include <dlfcn.h>
#include <sched.h>
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/resource.h>
#include <sys/wait.h>
#include <time.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "tcpxb/nccl_net_abi.h"

namespace {

struct Api {
  const char* name;
  ncclResult_t (*init)(ncclDebugLogger_t);
  ncclResult_t (*devices)(int*);
  ncclResult_t (*listen)(int, void*, void**);
  ncclResult_t (*connect)(int, void*, void**, ncclNetDeviceHandle_v8_t**);
  ncclResult_t (*accept)(void*, void**, ncclNetDeviceHandle_v8_t**);
  ncclResult_t (*regMr8)(void*, void*, size_t, int, void**);
  ncclResult_t (*regMr7)(void*, void*, int, int, void**);
  ncclResult_t (*deregMr)(void*, void*);
  ncclResult_t (*isend)(void*, void*, int, int, void*, void**);
  ncclResult_t (*irecv)(void*, int, void**, int*, int*, void**, void**);
  ncclResult_t (*test)(void*, int*, int*);
  ncclResult_t (*closeSend)(void*);
  ncclResult_t (*closeRecv)(void*);
  ncclResult_t (*closeListen)(void*);
  ncclResult_t (*irecvConsumed)(void*, int, void*);
  ncclResult_t (*props8)(int, ncclNetProperties_v8_t*);
  ncclResult_t (*props7)(int, ncclNetProperties_v7_t*);
  ncclResult_t (*iflush)(void*, int, void**, int*, void**, void**);
  ncclResult_t (*getDeviceMr)(void*, void*, void**);
  void* regMrDmaBuf;
};

// What a consumer of the unpack device handle sees (NCCL's device-side layout).
constexpr int kQueueDepth = 16;
constexpr int kSlotRecords = 2048;
struct Record { uint32_t src_off, len; uint64_t dst_off; };
struct MetaBlock { Record mem[kQueueDepth][kSlotRecords]; uint64_t cnt[kQueueDepth]; };
struct DeviceHandle { MetaBlock* meta; uint8_t* bounce_buf; uint64_t head; };

int (*flow_counters)(void*, tcpxbFlowCounters*, int) = nullptr;
int (*stats_text)(void*, char*, int) = nullptr;

#define CHECK(call)                                                          \
  do {                                                                       \
    ncclResult_t r_ = (call);                                                \
    if (r_ != ncclSuccess) {                                                 \
      fprintf(stderr, "%s:%d %s -> %d\n", __FILE__, __LINE__, #call, (int)r_); \
      return 1;                                                              \
    }                                                                        \
  } while (0)

// user and system CPU seconds of the whole process (all threads) so far
void cpuSec(double* user, double* sys) {
  struct rusage ru;
  getrusage(RUSAGE_SELF, &ru);
  *user = ru.ru_utime.tv_sec + ru.ru_utime.tv_usec * 1e-6;
  *sys = ru.ru_stime.tv_sec + ru.ru_stime.tv_usec * 1e-6;
}

double nowSec() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}

// xorshift64*: payload = f(seed, comm, iter, tag)
void fillPayload(uint8_t* p, size_t n, uint64_t key) {
  uint64_t x = key * 0x9e3779b97f4a7c15ull + 0x1234567;
  if (x == 0) x = 1;
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    x ^= x >> 12; x ^= x << 25; x ^= x >> 27;
    uint64_t v = x * 0x2545f4914f6cdd1dull;
    memcpy(p + i, &v, 8);
  }
  for (; i < n; ++i) {
    x ^= x >> 12; x ^= x << 25; x ^= x >> 27;
    p[i] = (uint8_t)(x * 0x2545f4914f6cdd1dull >> 56);
  }
}
uint64_t keyOf(uint64_t seed, int comm, int size_idx, int iter, int tag) {
  return ((((seed * 131 + (uint64_t)comm) * 131 + (uint64_t)size_idx) * 131 + (uint64_t)iter) * 131) + (uint64_t)tag;
}

// Bytes message `key` really carries when sizes are random: 0..cap, with the edges likely.
size_t actualSize(bool random, size_t cap, uint64_t key) {
  if (!random || cap == 0) return cap;
  uint64_t x = key * 0xd6e8feb86659fd93ull + 0x9e3779b97f4a7c15ull;
  x ^= x >> 32; x *= 0xd6e8feb86659fd93ull; x ^= x >> 32;
  switch (x & 7) {
    case 0: return 0;
    case 1: return cap;
    case 2: return cap > 1 ? cap - 1 : cap;
    default: return (size_t)((x >> 8) % (cap + 1));
  }
}

bool loadApi(const char* path, bool v7, Api* api) {
  void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (h == nullptr) { fprintf(stderr, "dlopen(%s): %s\n", path, dlerror()); return false; }
  flow_counters = (int (*)(void*, tcpxbFlowCounters*, int))dlsym(h, "tcpxb_comm_flow_counters");
  stats_text = (int (*)(void*, char*, int))dlsym(h, "tcpxb_comm_stats_text");
  memset(api, 0, sizeof *api);
  if (v7) {
    auto* t = (ncclNet_v7_t*)dlsym(h, "ncclNetPlugin_v7");
    if (t == nullptr) return false;
    *api = {t->name, t->init, t->devices, t->listen, t->connect, t->accept, nullptr, t->regMr, t->deregMr,
            t->isend, t->irecv, t->test, t->closeSend, t->closeRecv, t->closeListen, t->irecvConsumed,
            nullptr, t->getProperties, t->iflush, t->getDeviceMr, (void*)t->regMrDmaBuf};
  } else {
    auto* t = (ncclNet_v8_t*)dlsym(h, "ncclNetPlugin_v8");
    if (t == nullptr) return false;
    *api = {t->name, t->init, t->devices, t->listen, t->connect, t->accept, t->regMr, nullptr, t->deregMr,
            t->isend, t->irecv, t->test, t->closeSend, t->closeRecv, t->closeListen, t->irecvConsumed,
            t->getProperties, nullptr, t->iflush, t->getDeviceMr, (void*)t->regMrDmaBuf};
  }
  return true;
}

ncclResult_t regMr(const Api& api, void* comm, void* data, size_t size, int type, void** mh) {
  if (api.regMr8) return api.regMr8(comm, data, size, type, mh);
  return api.regMr7(comm, data, (int)size, type, mh);
}

// One step of the unpack consumer: returns false on a malformed slot.
bool consumeSlot(DeviceHandle* h, uint8_t* dst, size_t size) {
  h->head += 1;  // starts at all-ones: the first slot is 0
  const uint64_t slot = h->head % kQueueDepth;
  const uint64_t cnt = __atomic_load_n(&h->meta->cnt[slot], __ATOMIC_ACQUIRE);
  if (cnt > (uint64_t)kSlotRecords) { fprintf(stderr, "slot %lu holds %lu records\n", (unsigned long)slot, (unsigned long)cnt); return false; }
  uint64_t covered = 0;
  for (uint64_t i = 0; i < cnt; ++i) {
    const Record& m = h->meta->mem[slot][i];
    if (m.dst_off + m.len > size) { fprintf(stderr, "record %lu leaves the buffer\n", (unsigned long)i); return false; }
    memcpy(dst + m.dst_off, h->bounce_buf + m.src_off, m.len);
    covered += m.len;
  }
  if (covered != size) { fprintf(stderr, "records cover %lu of %zu bytes\n", (unsigned long)covered, size); return false; }
  return true;
}

void printFlows(const char* side, int ci, void* comm) {
  if (flow_counters == nullptr) return;
  tcpxbFlowCounters fc[16];
  int n = flow_counters(comm, fc, 16);
  for (int i = 0; i < n; ++i)
    printf("FLOW %s comm %d sock %d id %lu bytes_posted %lu bytes_done %lu tx %lu txc %lu rx %lu\n", side, ci, i,
           (unsigned long)fc[i].flow_id, (unsigned long)fc[i].bytes_posted, (unsigned long)fc[i].bytes_done,
           (unsigned long)fc[i].tx_cnt, (unsigned long)fc[i].tx_completion_cnt, (unsigned long)fc[i].rx_cnt);
  if (stats_text != nullptr) {
    char buf[4096];
    stats_text(comm, buf, sizeof buf);
    fputs(buf, stdout);
  }
}

// CPU seconds of every thread of this process, by thread name (helper threads are named
// tcpxb-tx<i> / tcpxb-rx<i>), from /proc: shows where a core-starved box spends its time.
void printThreadTimes(const char* side) {
  DIR* d = opendir("/proc/self/task");
  if (d == nullptr) return;
  const double tick = 1.0 / (double)sysconf(_SC_CLK_TCK);
  while (struct dirent* e = readdir(d)) {
    if (e->d_name[0] == '.') continue;
    std::string path = std::string("/proc/self/task/") + e->d_name + "/stat";
    FILE* f = fopen(path.c_str(), "r");
    if (f == nullptr) continue;
    char line[1024];
    if (fgets(line, sizeof line, f) != nullptr) {
      char* open = strchr(line, '(');
      char* close = strrchr(line, ')');
      unsigned long ut = 0, st = 0;
      if (open && close && sscanf(close + 2, "%*c %*d %*d %*d %*d %*d %*u %*u %*u %*u %*u %lu %lu", &ut, &st) == 2) {
        *close = 0;
        // the cores the thread may run on (shows whether the TX/RX_BINDINGS took effect)
        char cpus[128] = "?";
        std::string spath = std::string("/proc/self/task/") + e->d_name + "/status";
        if (FILE* sf = fopen(spath.c_str(), "r")) {
          char sl[256];
          while (fgets(sl, sizeof sl, sf) != nullptr)
            if (sscanf(sl, "Cpus_allowed_list: %127s", cpus) == 1) break;
          fclose(sf);
        }
        printf("THREAD %s %s user %.3f sys %.3f cpus %s\n", side, open + 1, (double)ut * tick, (double)st * tick, cpus);
      }
    }
    fclose(f);
  }
  closedir(d);
}

struct Options {
  std::string plugin;
  bool v7 = false;
  std::vector<size_t> sizes = {1024, 65536, 4194304, 67108864};
  int inflight = 8;
  int iters = 4;
  uint64_t seed = 42;
  int ptr_type = NCCL_PTR_HOST;
  bool yield_when_idle = false;
  bool random_sizes = false;
  bool thread_times = false;
  int comms_per_dev = 1;
};

int runSide(bool receiver, const Options& opt, int rfd, int wfd) {
  Api api;
  if (!loadApi(opt.plugin.c_str(), opt.v7, &api)) return 1;
  CHECK(api.init(nullptr));
  int ndev = 0;
  CHECK(api.devices(&ndev));
  if (ndev < 1) { fprintf(stderr, "no devices\n"); return 1; }
  if (receiver) {
    // what NCCL learns about each device
    for (int d = 0; d < ndev; ++d) {
      if (api.props8 != nullptr) {
        ncclNetProperties_v8_t p;
        memset(&p, 0, sizeof p);
        CHECK(api.props8(d, &p));
        printf("PROPS dev %d name %s pci %s guid %lu ptr %d regIsGlobal %d speed %d port %d latency %.1f maxComms %d maxRecvs %d devType %d devVersion %d\n",
               d, p.name, p.pciPath ? p.pciPath : "-", (unsigned long)p.guid, p.ptrSupport, p.regIsGlobal, p.speed, p.port, p.latency,
               p.maxComms, p.maxRecvs, (int)p.netDeviceType, p.netDeviceVersion);
      } else {
        ncclNetProperties_v7_t p;
        memset(&p, 0, sizeof p);
        CHECK(api.props7(d, &p));
        printf("PROPS dev %d name %s pci %s guid %lu ptr %d speed %d port %d latency %.1f maxComms %d maxRecvs %d devType %d devVersion %d\n",
               d, p.name, p.pciPath ? p.pciPath : "-", (unsigned long)p.guid, p.ptrSupport, p.speed, p.port, p.latency, p.maxComms,
               p.maxRecvs, (int)p.netDeviceType, p.netDeviceVersion);
      }
    }
    printf("TABLE regMrDmaBuf %s\n", api.regMrDmaBuf == nullptr ? "null" : "set");
  }
  const int ncomm = ndev * opt.comms_per_dev;  // comm c lives on device c % ndev, like NCCL's channels
  std::vector<void*> comms(ncomm, nullptr), listens(ncomm, nullptr);
  std::vector<DeviceHandle*> unpack(ncomm, nullptr);
  if (receiver) {
    std::vector<char> handles((size_t)ncomm * NCCL_NET_HANDLE_MAXSIZE, 0);
    for (int c = 0; c < ncomm; ++c) CHECK(api.listen(c % ndev, &handles[(size_t)c * NCCL_NET_HANDLE_MAXSIZE], &listens[c]));
    if (write(wfd, handles.data(), handles.size()) != (ssize_t)handles.size()) return 1;
    for (int c = 0; c < ncomm; ++c)
      while (comms[c] == nullptr) {
        ncclNetDeviceHandle_v8_t* dh = nullptr;
        CHECK(api.accept(listens[c], &comms[c], &dh));
        if (comms[c] == nullptr || dh == nullptr || dh->netDeviceType != NCCL_NET_DEVICE_UNPACK) continue;
        if (opt.ptr_type != NCCL_PTR_CUDA || getenv("TCPXB_FAKE_GPU") == nullptr) {
          fprintf(stderr, "the plugin offers an unpack handle; this tool can only consume it with --ptr cuda on the stand-in device\n");
          return 1;
        }
        if (dh->size != sizeof(DeviceHandle)) { fprintf(stderr, "device handle of %zu bytes\n", dh->size); return 1; }
        unpack[c] = static_cast<DeviceHandle*>(dh->handle);
      }
  } else {
    std::vector<char> handles((size_t)ncomm * NCCL_NET_HANDLE_MAXSIZE, 0);
    size_t got = 0;
    while (got < handles.size()) {
      ssize_t n = read(rfd, handles.data() + got, handles.size() - got);
      if (n <= 0) return 1;
      got += (size_t)n;
    }
    for (int c = 0; c < ncomm; ++c)
      while (comms[c] == nullptr) {
        ncclNetDeviceHandle_v8_t* dh = nullptr;
        CHECK(api.connect(c % ndev, &handles[(size_t)c * NCCL_NET_HANDLE_MAXSIZE], &comms[c], &dh));
      }
  }
  printf("%s: %s, %d comm(s) up\n", receiver ? "receiver" : "sender", api.name, ncomm);

  int rc = 0;
  for (size_t si = 0; si < opt.sizes.size() && rc == 0; ++si) {
    const size_t size = opt.sizes[si];
    const int nbuf = ncomm * opt.inflight;
    std::vector<std::vector<uint8_t>> bufs(nbuf, std::vector<uint8_t>(size ? size : 1));
    std::vector<uint8_t> expect(size ? size : 1);
    std::vector<void*> mh(nbuf, nullptr);
    for (int b = 0; b < nbuf; ++b) CHECK(regMr(api, comms[b / opt.inflight], bufs[b].data(), size, opt.ptr_type, &mh[b]));
    if (receiver && opt.ptr_type == NCCL_PTR_CUDA && nbuf > 0 && api.getDeviceMr != nullptr) {
      // the consumer's kernels index the user buffer directly: the device view of a registration is its base
      void* dptr = nullptr;
      CHECK(api.getDeviceMr(comms[0], mh[0], &dptr));
      if (dptr != bufs[0].data()) { fprintf(stderr, "getDeviceMr returned %p for a buffer at %p\n", dptr, (void*)bufs[0].data()); return 1; }
    }
    // both sides start a size together: receiver -> sender token, sender waits
    char tok = 'g';
    if (receiver) { if (write(wfd, &tok, 1) != 1) return 1; }
    else if (read(rfd, &tok, 1) != 1) return 1;
    double dt = 0, cpu_user = 0, cpu_sys = 0, bytes = 0;
    for (int it = 0; it < opt.iters && rc == 0; ++it) {
      std::vector<void*> reqs(nbuf, nullptr);
      if (!receiver)
        for (int b = 0; b < nbuf; ++b) fillPayload(bufs[b].data(), size, keyOf(opt.seed, b / opt.inflight, (int)si, it, b % opt.inflight));
      else
        for (int b = 0; b < nbuf; ++b) memset(bufs[b].data(), 0xEE, size);
      int posted = 0, finished = 0, posted_prev = 0;
      std::vector<char> done(nbuf, 0);
      std::vector<int> got_size(nbuf, -1);
      double u0, s0, u1, s1;
      cpuSec(&u0, &s0);
      const double t0 = nowSec();  // payload generation and checking stay outside the clock
      while (finished < nbuf) {
        // post in tag order per comm; a null request means "try again"
        if (posted < nbuf) {
          const int b = posted;
          void* comm = comms[b / opt.inflight];
          if (receiver) {
            void* data = bufs[b].data();
            int sz = (int)size, tag = b % opt.inflight;
            CHECK(api.irecv(comm, 1, &data, &sz, &tag, &mh[b], &reqs[b]));
          } else {
            const size_t act = actualSize(opt.random_sizes, size, keyOf(opt.seed, b / opt.inflight, (int)si, it, b % opt.inflight));
            CHECK(api.isend(comm, bufs[b].data(), (int)act, b % opt.inflight, mh[b], &reqs[b]));
          }
          if (reqs[b] != nullptr) ++posted;
        }
        const int finished_before = finished, posted_before = posted_prev;
        posted_prev = posted;
        for (int b = 0; b < posted; ++b) {
          if (done[b]) continue;
          int d = 0, sz = -1;
          CHECK(api.test(reqs[b], &d, &sz));
          if (!d) continue;
          if (receiver && unpack[b / opt.inflight] != nullptr) {
            // requests of one comm finish in posting order, which is the FIFO order of the slots
            if (sz > 0 && !consumeSlot(unpack[b / opt.inflight], bufs[b].data(), (size_t)sz)) return 1;
            else if (sz == 0) unpack[b / opt.inflight]->head += 1;
            CHECK(api.irecvConsumed(comms[b / opt.inflight], 1, reqs[b]));
          }
          if (receiver && api.iflush != nullptr) {
            // data is visible when test() reports done, so a flush has nothing to wait for
            void* fdata = bufs[b].data();
            int fsz = sz;
            void* freq = reinterpret_cast<void*>(1);
            CHECK(api.iflush(comms[b / opt.inflight], 1, &fdata, &fsz, &mh[b], &freq));
            if (freq != nullptr) { fprintf(stderr, "iflush returned a request\n"); return 1; }
          }
          done[b] = 1;
          ++finished;
          got_size[b] = sz;
        }
        // NCCL's proxy thread gives up its core when a pass over its operations moved nothing
        if (opt.yield_when_idle && finished == finished_before && posted == posted_before) sched_yield();
      }
      dt += nowSec() - t0;
      cpuSec(&u1, &s1);
      cpu_user += u1 - u0;
      cpu_sys += s1 - s0;
      for (int b = 0; b < nbuf; ++b) {
        const uint64_t key = keyOf(opt.seed, b / opt.inflight, (int)si, it, b % opt.inflight);
        const size_t act = actualSize(opt.random_sizes, size, key);
        bytes += (double)act;
        if (got_size[b] != (int)act) { fprintf(stderr, "size mismatch: test reported %d, expected %zu\n", got_size[b], act); rc = 1; }
        if (!receiver) continue;
        fillPayload(expect.data(), size, key);
        if (memcmp(expect.data(), bufs[b].data(), act) != 0) {
          fprintf(stderr, "payload mismatch: size %zu of %zu iter %d comm %d tag %d\n", act, size, it, b / opt.inflight, b % opt.inflight);
          rc = 1;
        }
        for (size_t k = act; k < size; ++k)
          if (bufs[b][k] != 0xEE) { fprintf(stderr, "byte %zu beyond the message's %zu bytes was written\n", k, act); rc = 1; break; }
      }
    }
    // the receiver's line is the result; the sender's carries its CPU seconds for the same transfers
    printf("{\"tool\": \"%s\", \"side\": \"%s\", \"size\": %zu, \"messages\": %d, \"inflight\": %d, \"comms\": %d, "
           "\"seconds\": %.6f, \"GBps\": %.3f, \"cpu_user_s\": %.4f, \"cpu_sys_s\": %.4f, \"byte_exact\": %s}\n",
           receiver ? "loopback" : "loopback-sender", receiver ? "recv" : "send", size, nbuf * opt.iters, opt.inflight, ncomm, dt,
           bytes / dt / 1e9, cpu_user, cpu_sys, rc == 0 ? "true" : "false");
    for (int b = 0; b < nbuf; ++b) CHECK(api.deregMr(comms[b / opt.inflight], mh[b]));
  }
  for (int c = 0; c < ncomm; ++c) printFlows(receiver ? "recv" : "send", c, comms[c]);
  if (opt.thread_times) printThreadTimes(receiver ? "recv" : "send");
  fflush(stdout);
  // the sender closes after the receiver confirmed it has everything
  char tok = 'c';
  if (receiver) { if (write(wfd, &tok, 1) != 1) rc = 1; }
  else if (read(rfd, &tok, 1) != 1) rc = 1;
  for (int c = 0; c < ncomm; ++c) {
    if (receiver) { CHECK(api.closeRecv(comms[c])); CHECK(api.closeListen(listens[c])); }
    else CHECK(api.closeSend(comms[c]));
  }
  return rc;
}

}  // namespace

int main(int argc, char** argv) {
  Options opt;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--help" || a == "-h") {
      printf("usage: tcpxb_loopback --plugin LIB [--v7] [--sizes a,b,...] [--inflight 1..16] [--iters N] [--seed S]\n"
             "                      [--ptr host|cuda] [--yield] [--random-sizes] [--thread-times]\n"
             "                      [--comms-per-dev N]\n");
      return 0;
    }
    if (a == "--plugin") opt.plugin = next();
    else if (a == "--v7") opt.v7 = true;
    else if (a == "--inflight") opt.inflight = atoi(next());
    else if (a == "--iters") opt.iters = atoi(next());
    else if (a == "--seed") opt.seed = strtoull(next(), nullptr, 0);
    else if (a == "--yield") opt.yield_when_idle = true;
    else if (a == "--random-sizes") opt.random_sizes = true;
    else if (a == "--thread-times") opt.thread_times = true;
    else if (a == "--comms-per-dev") opt.comms_per_dev = atoi(next());
    else if (a == "--ptr") opt.ptr_type = std::string(next()) == "cuda" ? NCCL_PTR_CUDA : NCCL_PTR_HOST;
    else if (a == "--sizes") {
      opt.sizes.clear();
      std::string s = next();
      size_t pos = 0;
      while (pos < s.size()) {
        size_t end = s.find(',', pos);
        if (end == std::string::npos) end = s.size();
        opt.sizes.push_back(strtoull(s.substr(pos, end - pos).c_str(), nullptr, 0));
        pos = end + 1;
      }
    } else { fprintf(stderr, "unknown argument %s\n", a.c_str()); return 2; }
  }
  if (opt.plugin.empty()) { fprintf(stderr, "--plugin is required\n"); return 2; }
  if (opt.inflight < 1 || opt.inflight > 16) { fprintf(stderr, "--inflight must be 1..16\n"); return 2; }
  if (opt.comms_per_dev < 1 || opt.comms_per_dev > 64) { fprintf(stderr, "--comms-per-dev must be 1..64\n"); return 2; }
  int to_child[2], to_parent[2];
  if (pipe(to_child) != 0 || pipe(to_parent) != 0) return 1;
  fflush(stdout);
  pid_t pid = fork();
  if (pid < 0) return 1;
  if (pid == 0) {
    close(to_child[1]);
    close(to_parent[0]);
    int rc = runSide(false, opt, to_child[0], to_parent[1]);
    fflush(stdout);
    _exit(rc);
  }
  close(to_child[0]);
  close(to_parent[1]);
  int rc = runSide(true, opt, to_parent[0], to_child[1]);
  if (rc != 0) kill(pid, SIGTERM);  // the sender may be waiting for a receiver that gave up
  int status = 0;
  waitpid(pid, &status, 0);
  if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) rc = 1;
  printf("loopback %s\n", rc == 0 ? "PASSED" : "FAILED");
  return rc;
}
