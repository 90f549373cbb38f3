// Symbol tables NCCL looks up in libnccl-net.so: ncclNetPlugin_v8 and ncclNetPlugin_v7.
//
// The reference exports a single v7 table (reference: src/nccl_plugin.cc:22-42) with
// regMrDmaBuf left null and both close slots on one function; the same holds here,
// and a v8 table (size_t regMr, regIsGlobal property) is added.
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include <map>
#include <mutex>
#include <string>

#include "tcpxb/cu_driver.h"
#include "tcpxb/gpu.h"
#include "tcpxb/nccl_net_abi.h"
#include "tcpxb/transport.h"

using namespace tcpxb;

namespace {

inline ncclResult_t R(Result r) { return r == kInProgress ? ncclSuccess : static_cast<ncclResult_t>(r); }

// One device-handle descriptor per comm that asked for one; freed with the comm.
struct DevHandleBox {
  ncclNetDeviceHandle_v8_t h;
};
std::mutex g_box_mu;
std::map<void*, DevHandleBox*>* g_boxes = nullptr;

ncclResult_t attachDeviceHandle(Comm* comm, ncclNetDeviceHandle_v8_t** out) {
  if (out == nullptr) return ncclSuccess;
  *out = nullptr;
  if (comm == nullptr || comm->recv_mode != kRecvModeUnpack || !comm->passive) return ncclSuccess;
  void* dh = nullptr;
  size_t sz = 0;
  Result r = netGetDeviceHandle(comm, &dh, &sz);
  if (r != kSuccess) return R(r);
  auto* box = new DevHandleBox();
  box->h.netDeviceType = NCCL_NET_DEVICE_UNPACK;
  box->h.netDeviceVersion = kUnpackVersion;
  box->h.handle = dh;
  box->h.size = sz;
  box->h.needsProxyProgress = 1;
  {
    std::lock_guard<std::mutex> l(g_box_mu);
    if (g_boxes == nullptr) g_boxes = new std::map<void*, DevHandleBox*>();
    (*g_boxes)[comm] = box;
  }
  *out = &box->h;
  return ncclSuccess;
}

void dropDeviceHandle(void* comm) {
  std::lock_guard<std::mutex> l(g_box_mu);
  if (g_boxes == nullptr) return;
  auto it = g_boxes->find(comm);
  if (it == g_boxes->end()) return;
  delete it->second;
  g_boxes->erase(it);
}

ncclResult_t pluginInit(ncclDebugLogger_t logFunction) { return R(netInit(reinterpret_cast<LoggerFn>(logFunction))); }
ncclResult_t pluginDevices(int* ndev) { return R(netDevices(ndev)); }

ncclResult_t pluginGetProperties_v8(int dev, ncclNetProperties_v8_t* p) {
  NetProperties np;
  Result r = netGetProperties(dev, &np);
  if (r != kSuccess) return R(r);
  p->name = const_cast<char*>(np.name);
  p->pciPath = const_cast<char*>(np.pci_path);
  p->guid = np.guid;
  p->ptrSupport = np.ptr_support;
  p->regIsGlobal = 0;
  p->speed = np.speed_mbps;
  p->port = np.port;
  p->latency = np.latency;
  p->maxComms = np.max_comms;
  p->maxRecvs = np.max_recvs;
  p->netDeviceType = static_cast<ncclNetDeviceType>(np.device_type);
  p->netDeviceVersion = np.device_version;
  return ncclSuccess;
}

ncclResult_t pluginGetProperties_v7(int dev, ncclNetProperties_v7_t* p) {
  ncclNetProperties_v8_t p8;
  ncclResult_t r = pluginGetProperties_v8(dev, &p8);
  if (r != ncclSuccess) return r;
  p->name = p8.name;
  p->pciPath = p8.pciPath;
  p->guid = p8.guid;
  p->ptrSupport = p8.ptrSupport;
  p->speed = p8.speed;
  p->port = p8.port;
  p->latency = p8.latency;
  p->maxComms = p8.maxComms;
  p->maxRecvs = p8.maxRecvs;
  p->netDeviceType = p8.netDeviceType;
  p->netDeviceVersion = p8.netDeviceVersion;
  return ncclSuccess;
}

ncclResult_t pluginListen(int dev, void* handle, void** listenComm) {
  ListenComm* l = nullptr;
  Result r = netListen(dev, handle, &l);
  *listenComm = l;
  return R(r);
}

ncclResult_t pluginConnect(int dev, void* handle, void** sendComm, ncclNetDeviceHandle_v8_t** sendDevComm) {
  Comm* c = nullptr;
  Result r = netConnect(dev, handle, &c);
  *sendComm = c;
  if (sendDevComm != nullptr) *sendDevComm = nullptr;  // the sender has no device side
  return R(r);
}

ncclResult_t pluginAccept(void* listenComm, void** recvComm, ncclNetDeviceHandle_v8_t** recvDevComm) {
  Comm* c = nullptr;
  Result r = netAccept(static_cast<ListenComm*>(listenComm), &c);
  *recvComm = c;
  if (r != kSuccess) return R(r);
  if (c != nullptr) return attachDeviceHandle(c, recvDevComm);
  if (recvDevComm != nullptr) *recvDevComm = nullptr;
  return ncclSuccess;
}

ncclResult_t pluginRegMr_v8(void* comm, void* data, size_t size, int type, void** mhandle) {
  MemHandle* mh = nullptr;
  Result r = netRegMr(static_cast<Comm*>(comm), data, size, type, &mh);
  *mhandle = mh;
  return R(r);
}
ncclResult_t pluginRegMr_v7(void* comm, void* data, int size, int type, void** mhandle) {
  return pluginRegMr_v8(comm, data, (size_t)size, type, mhandle);
}
ncclResult_t pluginDeregMr(void* comm, void* mhandle) {
  return R(netDeregMr(static_cast<Comm*>(comm), static_cast<MemHandle*>(mhandle)));
}
ncclResult_t pluginIsend(void* sendComm, void* data, int size, int tag, void* mhandle, void** request) {
  Request* req = nullptr;
  Result r = netIsend(static_cast<Comm*>(sendComm), data, size, tag, static_cast<MemHandle*>(mhandle), &req);
  *request = req;
  return R(r);
}
ncclResult_t pluginIrecv(void* recvComm, int n, void** data, int* sizes, int* tags, void** mhandles, void** request) {
  Request* req = nullptr;
  Result r = netIrecv(static_cast<Comm*>(recvComm), n, data, sizes, tags, reinterpret_cast<MemHandle**>(mhandles), &req);
  *request = req;
  return R(r);
}
ncclResult_t pluginIflush(void* recvComm, int n, void** data, int* sizes, void** mhandles, void** request) {
  Request* req = nullptr;
  Result r = netIflush(static_cast<Comm*>(recvComm), n, data, sizes, reinterpret_cast<MemHandle**>(mhandles), &req);
  *request = req;
  return R(r);
}
ncclResult_t pluginTest(void* request, int* done, int* sizes) {
  return R(netTest(static_cast<Request*>(request), done, sizes));
}
ncclResult_t pluginClose(void* comm) {
  dropDeviceHandle(comm);
  return R(netClose(static_cast<Comm*>(comm)));
}
ncclResult_t pluginCloseListen(void* listenComm) { return R(netCloseListen(static_cast<ListenComm*>(listenComm))); }
ncclResult_t pluginGetDeviceMr(void* comm, void* mhandle, void** dptr_mhandle) {
  return R(netGetDeviceMr(static_cast<Comm*>(comm), static_cast<MemHandle*>(mhandle), dptr_mhandle));
}
ncclResult_t pluginIrecvConsumed(void* recvComm, int n, void* request) {
  return R(netIrecvConsumed(static_cast<Comm*>(recvComm), n, static_cast<Request*>(request)));
}

}  // namespace

extern "C" {

__attribute__((visibility("default"))) volatile ncclNet_v8_t ncclNetPlugin_v8 = {
    "GPUDirectTCPX_B200_v8",
    pluginInit,
    pluginDevices,
    pluginGetProperties_v8,
    pluginListen,
    pluginConnect,
    pluginAccept,
    pluginRegMr_v8,
    nullptr,  // regMrDmaBuf
    pluginDeregMr,
    pluginIsend,
    pluginIrecv,
    pluginIflush,
    pluginTest,
    pluginClose,
    pluginClose,
    pluginCloseListen,
    pluginGetDeviceMr,
    pluginIrecvConsumed,
};

__attribute__((visibility("default"))) volatile ncclNet_v7_t ncclNetPlugin_v7 = {
    "GPUDirectTCPX_B200_v7",
    pluginInit,
    pluginDevices,
    pluginGetProperties_v7,
    pluginListen,
    pluginConnect,
    pluginAccept,
    pluginRegMr_v7,
    nullptr,  // regMrDmaBuf
    pluginDeregMr,
    pluginIsend,
    pluginIrecv,
    pluginIflush,
    pluginTest,
    pluginClose,
    pluginClose,
    pluginCloseListen,
    pluginGetDeviceMr,
    pluginIrecvConsumed,
};

int tcpxb_comm_flow_counters(void* comm, tcpxbFlowCounters* out, int max) {
  static_assert(sizeof(tcpxbFlowCounters) == sizeof(FlowCounters), "same layout");
  return netCommFlowCounters(static_cast<Comm*>(comm), reinterpret_cast<FlowCounters*>(out), max);
}

int tcpxb_comm_stats_text(void* comm, char* buf, int len) {
  std::string all;
  for (const std::string& l : netCommStatsLines(static_cast<Comm*>(comm))) all += l + "\n";
  if (buf != nullptr && len > 0) snprintf(buf, (size_t)len, "%s", all.c_str());
  return (int)all.size() + 1;
}

int tcpxb_export_dmabuf(const void* ptr, uint64_t bytes, int* fd_out, uint64_t* offset_out) {
  if (fd_out == nullptr || offset_out == nullptr) return -1;
  return cu::exportDmabuf(ptr, (size_t)bytes, fd_out, offset_out) == kSuccess ? 0 : -1;
}

int tcpxb_shared_pool_selftest(int dev, uint64_t bytes) {
  // owner and client in one process: create, export, import, and check that both mappings are the same memory
  cu::SharedAllocation owner, client;
  int fd = -1;
  if (cu::deviceInit(dev) != kSuccess || cu::sharedCreate(dev, (size_t)bytes, &owner, &fd) != kSuccess) return -1;
  int rc = -2;
  if (cu::sharedImport(dev, fd, owner.bytes, &client) == kSuccess) {
    const uint32_t pattern = 0x5aa5c33c;
    uint32_t back = 0;
    void* tail = static_cast<uint8_t*>(owner.dptr) + owner.bytes - sizeof pattern;
    void* tail_c = static_cast<uint8_t*>(client.dptr) + owner.bytes - sizeof pattern;
    if (gpu::copyToDeviceAsync(tail, &pattern, sizeof pattern, nullptr) == kSuccess && gpu::streamSynchronize(nullptr) == kSuccess &&
        gpu::copyToHostAsync(&back, tail_c, sizeof back, nullptr) == kSuccess && gpu::streamSynchronize(nullptr) == kSuccess)
      rc = back == pattern ? 0 : -3;
    cu::sharedRelease(&client);
  }
  close(fd);
  cu::sharedRelease(&owner);
  return rc;
}

int tcpxb_flag_count(void) { return (int)flagDocs().size(); }
int tcpxb_flag_doc(int i, const char** env, const char** kind, const char** dflt, const char** doc) {
  const auto& d = flagDocs();
  if (i < 0 || i >= (int)d.size()) return -1;
  *env = d[i].env; *kind = d[i].kind; *dflt = d[i].dflt; *doc = d[i].doc;
  return 0;
}

}  // extern "C"
