#include "tcpxb/cu_driver.h"

#include <errno.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>

#include "tcpxb/flags.h"
#include "tcpxb/gpu.h"

#ifndef TCPXB_NO_CUDA
#include <cuda.h>
#include <dlfcn.h>
#endif

namespace tcpxb {
namespace cu {

namespace {
thread_local char g_err[256] = "";
Result failed(const char* what, const char* detail) {
  snprintf(g_err, sizeof g_err, "%s: %s", what, detail);
  WARN("driver call failed: %s", g_err);
  return kUnhandledCudaError;
}
constexpr int kMaxDev = 64;
}  // namespace

const char* lastError() { return g_err; }

#ifdef TCPXB_NO_CUDA
// ---------------------------------------------------------------- stand-in device
// Host memory plays device memory (see gpu.cc).  A shareable allocation is a memfd.

namespace {
bool fake() { return gpu::available(); }
std::mutex g_mu;
struct FakeAlloc { int fd; size_t bytes; };
std::map<uintptr_t, FakeAlloc> g_maps;  // mapping base -> backing memfd (kept open for dma-buf export)
bool g_own_ctx[kMaxDev] = {};
thread_local int t_ctx_depth = 0;
}  // namespace

bool available() { return fake(); }

Result deviceInit(int dev, bool owns_its_memory) {
  if (!fake() || dev != 0) return failed("deviceInit", "no such device");
  std::lock_guard<std::mutex> l(g_mu);
  g_own_ctx[0] = flags().cuda_use_primary_ctx == 0 && owns_its_memory;
  return kSuccess;
}
bool usesOwnContext(int dev) { return dev == 0 && g_own_ctx[0]; }
void deviceShutdown(int dev) { if (dev == 0) g_own_ctx[0] = false; }

ScopedContext::ScopedContext(int dev) {
  ok_ = fake() && dev == 0;
  if (ok_) { ++t_ctx_depth; pushed_ = true; }
}
ScopedContext::~ScopedContext() { if (pushed_) --t_ctx_depth; }

size_t sharedGranularity(int) { return 2u << 20; }

Result sharedCreate(int dev, size_t bytes, SharedAllocation* out, int* fd_out) {
  if (!fake() || dev != 0) return failed("sharedCreate", "no such device");
  const size_t g = sharedGranularity(dev);
  bytes = (bytes + g - 1) / g * g;
  int fd = memfd_create("tcpxb-standin-pool", MFD_CLOEXEC);
  if (fd < 0 || ftruncate(fd, (off_t)bytes) != 0) { if (fd >= 0) close(fd); return failed("memfd_create", strerror(errno)); }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) { close(fd); return failed("mmap", strerror(errno)); }
  out->dptr = p; out->bytes = bytes; out->handle = (uint64_t)fd; out->dev = dev; out->imported = false;
  { std::lock_guard<std::mutex> l(g_mu); g_maps[(uintptr_t)p] = {fd, bytes}; }
  *fd_out = dup(fd);
  return *fd_out >= 0 ? kSuccess : failed("dup", strerror(errno));
}

Result sharedImport(int dev, int fd, size_t bytes, SharedAllocation* out) {
  if (!fake() || dev != 0) return failed("sharedImport", "no such device");
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) return failed("mmap", strerror(errno));
  const int keep = dup(fd);
  out->dptr = p; out->bytes = bytes; out->handle = (uint64_t)keep; out->dev = dev; out->imported = true;
  { std::lock_guard<std::mutex> l(g_mu); g_maps[(uintptr_t)p] = {keep, bytes}; }
  return kSuccess;
}

void sharedRelease(SharedAllocation* a) {
  if (a == nullptr || a->dptr == nullptr) return;
  { std::lock_guard<std::mutex> l(g_mu); g_maps.erase((uintptr_t)a->dptr); }
  munmap(a->dptr, a->bytes);
  if ((int)a->handle >= 0) close((int)a->handle);
  *a = SharedAllocation();
}

// CUDA IPC on the stand-in: the "device memory" is a POSIX shared-memory object whose name
// travels in the handle, together with the owner's pid (a handle cannot be opened where it was made).
namespace {
struct FakeIpcHandle {
  char magic[8];
  int32_t owner_pid;
  uint32_t pad;
  uint64_t bytes;
  char name[40];
};
static_assert(sizeof(FakeIpcHandle) == kIpcHandleBytes, "handle size");
std::map<uintptr_t, std::string> g_ipc_owned;  // mapping base -> shm name to unlink
}  // namespace

Result ipcCreate(int dev, size_t bytes, IpcAllocation* out, unsigned char handle[kIpcHandleBytes]) {
  if (!fake() || dev != 0) return failed("ipcCreate", "no such device");
  static std::atomic<int> counter{0};
  FakeIpcHandle h;
  memset(&h, 0, sizeof h);
  memcpy(h.magic, "TCPXBIPC", 8);
  h.owner_pid = (int32_t)getpid();
  h.bytes = bytes;
  snprintf(h.name, sizeof h.name, "/tcpxb-ipc-%d-%d", (int)getpid(), counter.fetch_add(1));
  int fd = shm_open(h.name, O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0 || ftruncate(fd, (off_t)bytes) != 0) { if (fd >= 0) { close(fd); shm_unlink(h.name); } return failed("shm_open", strerror(errno)); }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) { shm_unlink(h.name); return failed("mmap", strerror(errno)); }
  { std::lock_guard<std::mutex> l(g_mu); g_ipc_owned[(uintptr_t)p] = h.name; }
  out->dptr = p; out->bytes = bytes; out->dev = dev; out->opened = false;
  memcpy(handle, &h, sizeof h);
  return kSuccess;
}

Result ipcOpen(int dev, const unsigned char handle[kIpcHandleBytes], IpcAllocation* out) {
  if (!fake() || dev != 0) return failed("ipcOpen", "no such device");
  FakeIpcHandle h;
  memcpy(&h, handle, sizeof h);
  h.name[sizeof h.name - 1] = 0;
  if (memcmp(h.magic, "TCPXBIPC", 8) != 0) return failed("ipcOpen", "not a memory handle");
  if (h.owner_pid == (int32_t)getpid()) return failed("ipcOpen", "a handle cannot be opened by the process that made it");
  int fd = shm_open(h.name, O_RDWR, 0);
  if (fd < 0) return failed("shm_open", strerror(errno));
  struct stat sb;
  if (fstat(fd, &sb) != 0 || (uint64_t)sb.st_size < h.bytes) { close(fd); return failed("ipcOpen", "the memory behind the handle is gone or too small"); }
  void* p = mmap(nullptr, (size_t)h.bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) return failed("mmap", strerror(errno));
  out->dptr = p; out->bytes = (size_t)h.bytes; out->dev = dev; out->opened = true;
  return kSuccess;
}

void ipcRelease(IpcAllocation* a) {
  if (a == nullptr || a->dptr == nullptr) return;
  if (!a->opened) {
    std::lock_guard<std::mutex> l(g_mu);
    auto it = g_ipc_owned.find((uintptr_t)a->dptr);
    if (it != g_ipc_owned.end()) { shm_unlink(it->second.c_str()); g_ipc_owned.erase(it); }
  }
  munmap(a->dptr, a->bytes);
  *a = IpcAllocation();
}

Result streamWriteValue32(void*, void* dev_word, uint32_t value) {
  if (!fake()) return failed("streamWriteValue32", "no device");
  __atomic_store_n(static_cast<uint32_t*>(dev_word), value, __ATOMIC_RELEASE);  // the stand-in's streams run everything at once
  return kSuccess;
}

Result exportDmabuf(const void* ptr, size_t bytes, int* fd_out, uint64_t* offset_out) {
  if (!fake()) return failed("exportDmabuf", "no device");
  std::lock_guard<std::mutex> l(g_mu);
  const uintptr_t p = (uintptr_t)ptr;
  auto it = g_maps.upper_bound(p);
  if (it == g_maps.begin()) return failed("exportDmabuf", "the range is not inside a shareable allocation of the stand-in device");
  --it;
  if (p + bytes > it->first + it->second.bytes) return failed("exportDmabuf", "the range leaves its allocation");
  *fd_out = dup(it->second.fd);
  *offset_out = p - it->first;
  return *fd_out >= 0 ? kSuccess : failed("dup", strerror(errno));
}

#else
// ---------------------------------------------------------------------- real driver

namespace {

struct Api {
  void* lib = nullptr;
  bool ok = false;
  CUresult (*Init)(unsigned) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*PrimaryCtxRetain)(CUcontext*, CUdevice) = nullptr;
  CUresult (*PrimaryCtxRelease)(CUdevice) = nullptr;
  CUresult (*CtxCreate)(CUcontext*, unsigned, CUdevice) = nullptr;
  CUresult (*CtxDestroy)(CUcontext) = nullptr;
  CUresult (*CtxPush)(CUcontext) = nullptr;
  CUresult (*CtxPop)(CUcontext*) = nullptr;
  CUresult (*CtxGetCurrent)(CUcontext*) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemGetHandleForAddressRange)(void*, CUdeviceptr, size_t, CUmemRangeHandleType, unsigned long long) = nullptr;
  CUresult (*StreamWriteValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int) = nullptr;
  CUresult (*MemAlloc)(CUdeviceptr*, size_t) = nullptr;
  CUresult (*MemFree)(CUdeviceptr) = nullptr;
  CUresult (*MemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr) = nullptr;
  CUresult (*IpcGetMemHandle)(CUipcMemHandle*, CUdeviceptr) = nullptr;
  CUresult (*IpcOpenMemHandle)(CUdeviceptr*, CUipcMemHandle, unsigned int) = nullptr;
  CUresult (*IpcCloseMemHandle)(CUdeviceptr) = nullptr;
};

template <typename F>
bool sym(void* lib, const char* name, F* out) {
  *out = reinterpret_cast<F>(dlsym(lib, name));
  return *out != nullptr;
}

// The exported names carry the ABI revision where the driver has more than one.
const Api& api() {
  static const Api a = [] {
    Api x;
    x.lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (x.lib == nullptr) return x;
    bool ok = sym(x.lib, "cuInit", &x.Init) && sym(x.lib, "cuDeviceGet", &x.DeviceGet) &&
              sym(x.lib, "cuGetErrorString", &x.GetErrorString) &&
              sym(x.lib, "cuDevicePrimaryCtxRetain", &x.PrimaryCtxRetain) &&
              sym(x.lib, "cuDevicePrimaryCtxRelease_v2", &x.PrimaryCtxRelease) &&
              sym(x.lib, "cuCtxCreate_v2", &x.CtxCreate) && sym(x.lib, "cuCtxDestroy_v2", &x.CtxDestroy) &&
              sym(x.lib, "cuCtxPushCurrent_v2", &x.CtxPush) && sym(x.lib, "cuCtxPopCurrent_v2", &x.CtxPop) &&
              sym(x.lib, "cuCtxGetCurrent", &x.CtxGetCurrent) &&
              sym(x.lib, "cuMemGetAllocationGranularity", &x.MemGetAllocationGranularity) &&
              sym(x.lib, "cuMemCreate", &x.MemCreate) && sym(x.lib, "cuMemExportToShareableHandle", &x.MemExport) &&
              sym(x.lib, "cuMemImportFromShareableHandle", &x.MemImport) &&
              sym(x.lib, "cuMemAddressReserve", &x.MemAddressReserve) && sym(x.lib, "cuMemMap", &x.MemMap) &&
              sym(x.lib, "cuMemSetAccess", &x.MemSetAccess) && sym(x.lib, "cuMemUnmap", &x.MemUnmap) &&
              sym(x.lib, "cuMemAddressFree", &x.MemAddressFree) && sym(x.lib, "cuMemRelease", &x.MemRelease);
    // optional: present from CUDA 11.7 drivers on
    sym(x.lib, "cuMemGetHandleForAddressRange", &x.MemGetHandleForAddressRange);
    sym(x.lib, "cuStreamWriteValue32_v2", &x.StreamWriteValue32);
    sym(x.lib, "cuMemAlloc_v2", &x.MemAlloc);
    sym(x.lib, "cuMemFree_v2", &x.MemFree);
    sym(x.lib, "cuMemGetAddressRange_v2", &x.MemGetAddressRange);
    sym(x.lib, "cuIpcGetMemHandle", &x.IpcGetMemHandle);
    sym(x.lib, "cuIpcOpenMemHandle_v2", &x.IpcOpenMemHandle);
    sym(x.lib, "cuIpcCloseMemHandle", &x.IpcCloseMemHandle);
    x.ok = ok && x.Init(0) == CUDA_SUCCESS;
    return x;
  }();
  return a;
}

Result cuCheck(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return kSuccess;
  const char* s = nullptr;
  if (api().GetErrorString == nullptr || api().GetErrorString(r, &s) != CUDA_SUCCESS || s == nullptr) s = "unknown error";
  return failed(what, s);
}
#define CUD(expr) cuCheck((expr), #expr)

struct DevCtx {
  CUcontext ctx = nullptr;
  bool own = false, primary_retained = false;
};
std::mutex g_mu;
DevCtx g_ctx[kMaxDev];

CUmemAllocationProp poolProp(int dev) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof prop);
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  return prop;
}

Result mapReadWrite(int dev, CUmemGenericAllocationHandle h, size_t bytes, size_t gran, CUdeviceptr* out) {
  const Api& a = api();
  CUdeviceptr va = 0;
  TCPXB_CHECK(CUD(a.MemAddressReserve(&va, bytes, gran, 0, 0)));
  Result r = CUD(a.MemMap(va, bytes, 0, h, 0));
  if (r == kSuccess) {
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof acc);
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = dev;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = CUD(a.MemSetAccess(va, bytes, &acc, 1));
    if (r != kSuccess) a.MemUnmap(va, bytes);
  }
  if (r != kSuccess) { a.MemAddressFree(va, bytes); return r; }
  *out = va;
  return kSuccess;
}

}  // namespace

bool available() { return api().ok; }

Result deviceInit(int dev, bool owns_its_memory) {
  if (!api().ok) return failed("deviceInit", "the CUDA driver library could not be loaded");
  if (dev < 0 || dev >= kMaxDev) return failed("deviceInit", "device ordinal out of range");
  std::lock_guard<std::mutex> l(g_mu);
  DevCtx& d = g_ctx[dev];
  if (d.ctx != nullptr) return kSuccess;
  const Api& a = api();
  CUdevice cd;
  TCPXB_CHECK(CUD(a.DeviceGet(&cd, dev)));
  if (flags().cuda_use_primary_ctx != 0 || !owns_its_memory) {
    if (flags().cuda_use_primary_ctx == 0)
      INFO(kSubInit, "GPU %d: NCCL_GPUDIRECTTCPX_CUDA_USE_PRIMARY_CTX=0 ignored here: the application's buffers live in the primary context", dev);
    TCPXB_CHECK(CUD(a.PrimaryCtxRetain(&d.ctx, cd)));
    d.primary_retained = true;
  } else {
    // A context of the library's own.  Memory of the application's (primary) context
    // is not reachable from it, so it serves processes that own their device memory
    // outright: the buffer-manager daemon, whose pool leaves the process as a file
    // descriptor.  cuCtxCreate makes the new context current; it is popped again.
    TCPXB_CHECK(CUD(a.CtxCreate(&d.ctx, 0, cd)));
    CUcontext popped = nullptr;
    a.CtxPop(&popped);
    d.own = true;
    INFO(kSubInit, "GPU %d: using a context of the library's own (NCCL_GPUDIRECTTCPX_CUDA_USE_PRIMARY_CTX=0)", dev);
  }
  return kSuccess;
}

bool usesOwnContext(int dev) {
  if (dev < 0 || dev >= kMaxDev) return false;
  std::lock_guard<std::mutex> l(g_mu);
  return g_ctx[dev].own;
}

void deviceShutdown(int dev) {
  if (dev < 0 || dev >= kMaxDev || !api().ok) return;
  std::lock_guard<std::mutex> l(g_mu);
  DevCtx& d = g_ctx[dev];
  if (d.ctx == nullptr) return;
  if (d.own) api().CtxDestroy(d.ctx);
  else if (d.primary_retained) { CUdevice cd; if (api().DeviceGet(&cd, dev) == CUDA_SUCCESS) api().PrimaryCtxRelease(cd); }
  d = DevCtx();
}

ScopedContext::ScopedContext(int dev) {
  if (deviceInit(dev) != kSuccess) return;
  CUcontext want;
  { std::lock_guard<std::mutex> l(g_mu); want = g_ctx[dev].ctx; }
  CUcontext cur = nullptr;
  if (api().CtxGetCurrent(&cur) == CUDA_SUCCESS && cur == want) { ok_ = true; return; }
  if (api().CtxPush(want) == CUDA_SUCCESS) { pushed_ = true; ok_ = true; }
}
ScopedContext::~ScopedContext() {
  if (pushed_) { CUcontext popped = nullptr; api().CtxPop(&popped); }
}

size_t sharedGranularity(int dev) {
  if (!api().ok) return 2u << 20;
  const CUmemAllocationProp prop = poolProp(dev);
  size_t g = 0;
  if (api().MemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0) g = 2u << 20;
  return g;
}

Result sharedCreate(int dev, size_t bytes, SharedAllocation* out, int* fd_out) {
  ScopedContext ctx(dev);
  if (!ctx.ok()) return failed("sharedCreate", "no context");
  const Api& a = api();
  const size_t g = sharedGranularity(dev);
  bytes = (bytes + g - 1) / g * g;
  const CUmemAllocationProp prop = poolProp(dev);
  CUmemGenericAllocationHandle h = 0;
  TCPXB_CHECK(CUD(a.MemCreate(&h, bytes, &prop, 0)));
  int fd = -1;
  Result r = CUD(a.MemExport(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  CUdeviceptr va = 0;
  if (r == kSuccess) r = mapReadWrite(dev, h, bytes, g, &va);
  if (r != kSuccess) { if (fd >= 0) close(fd); a.MemRelease(h); return r; }
  out->dptr = reinterpret_cast<void*>(va); out->bytes = bytes; out->handle = h; out->dev = dev; out->imported = false;
  *fd_out = fd;
  return kSuccess;
}

Result sharedImport(int dev, int fd, size_t bytes, SharedAllocation* out) {
  ScopedContext ctx(dev);
  if (!ctx.ok()) return failed("sharedImport", "no context");
  const Api& a = api();
  const size_t g = sharedGranularity(dev);
  if (bytes == 0 || bytes % g != 0) return failed("sharedImport", "size is not a multiple of the allocation granularity");
  CUmemGenericAllocationHandle h = 0;
  TCPXB_CHECK(CUD(a.MemImport(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR)));
  CUdeviceptr va = 0;
  Result r = mapReadWrite(dev, h, bytes, g, &va);
  if (r != kSuccess) { a.MemRelease(h); return r; }
  out->dptr = reinterpret_cast<void*>(va); out->bytes = bytes; out->handle = h; out->dev = dev; out->imported = true;
  return kSuccess;
}

void sharedRelease(SharedAllocation* s) {
  if (s == nullptr || s->dptr == nullptr || !api().ok) return;
  ScopedContext ctx(s->dev);
  const Api& a = api();
  const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(s->dptr);
  a.MemUnmap(va, s->bytes);
  a.MemAddressFree(va, s->bytes);
  a.MemRelease(s->handle);
  *s = SharedAllocation();
}

Result ipcCreate(int dev, size_t bytes, IpcAllocation* out, unsigned char handle[kIpcHandleBytes]) {
  const Api& a = api();
  if (!a.ok || a.MemAlloc == nullptr || a.IpcGetMemHandle == nullptr) return failed("ipcCreate", "this driver offers no memory handles");
  static_assert(sizeof(CUipcMemHandle) == kIpcHandleBytes, "handle size");
  ScopedContext ctx(dev);
  if (!ctx.ok()) return failed("ipcCreate", "no context on the device");
  CUdeviceptr p = 0;
  TCPXB_CHECK(CUD(a.MemAlloc(&p, bytes)));
  CUipcMemHandle h;
  Result r = CUD(a.IpcGetMemHandle(&h, p));
  if (r != kSuccess) { a.MemFree(p); return r; }
  memcpy(handle, &h, sizeof h);
  out->dptr = reinterpret_cast<void*>(p); out->bytes = bytes; out->dev = dev; out->opened = false;
  return kSuccess;
}

Result ipcOpen(int dev, const unsigned char handle[kIpcHandleBytes], IpcAllocation* out) {
  const Api& a = api();
  if (!a.ok || a.IpcOpenMemHandle == nullptr || a.MemGetAddressRange == nullptr) return failed("ipcOpen", "this driver offers no memory handles");
  ScopedContext ctx(dev);
  if (!ctx.ok()) return failed("ipcOpen", "no context on the device");
  CUipcMemHandle h;
  memcpy(&h, handle, sizeof h);
  CUdeviceptr p = 0;
  TCPXB_CHECK(CUD(a.IpcOpenMemHandle(&p, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS)));
  CUdeviceptr base = 0;
  size_t size = 0;
  Result r = CUD(a.MemGetAddressRange(&base, &size, p));
  if (r != kSuccess || base != p) {  // the owner exports whole allocations
    if (a.IpcCloseMemHandle != nullptr) a.IpcCloseMemHandle(p);
    return r != kSuccess ? r : failed("ipcOpen", "the handle does not name the start of an allocation");
  }
  out->dptr = reinterpret_cast<void*>(p); out->bytes = size; out->dev = dev; out->opened = true;
  return kSuccess;
}

void ipcRelease(IpcAllocation* x) {
  if (x == nullptr || x->dptr == nullptr || !api().ok) return;
  ScopedContext ctx(x->dev);
  const Api& a = api();
  const CUdeviceptr p = reinterpret_cast<CUdeviceptr>(x->dptr);
  if (x->opened) { if (a.IpcCloseMemHandle != nullptr) a.IpcCloseMemHandle(p); }
  else if (a.MemFree != nullptr) a.MemFree(p);
  *x = IpcAllocation();
}

Result streamWriteValue32(void* stream, void* dev_word, uint32_t value) {
  const Api& a = api();
  if (!a.ok || a.StreamWriteValue32 == nullptr) return kInvalidUsage;
  // default flags: the write is ordered after the memory effects of the work before it
  return a.StreamWriteValue32(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(dev_word), value, 0) == CUDA_SUCCESS
             ? kSuccess : kInvalidUsage;
}

Result exportDmabuf(const void* ptr, size_t bytes, int* fd_out, uint64_t* offset_out) {
  const Api& a = api();
  if (!a.ok || a.MemGetHandleForAddressRange == nullptr) return failed("exportDmabuf", "this driver has no dma-buf export");
  // the driver exports whole host pages only
  const uintptr_t page = (uintptr_t)sysconf(_SC_PAGESIZE);
  const uintptr_t p = reinterpret_cast<uintptr_t>(ptr);
  const uintptr_t lo = p & ~(page - 1);
  const uintptr_t hi = (p + bytes + page - 1) & ~(page - 1);
  int fd = -1;
  TCPXB_CHECK(CUD(a.MemGetHandleForAddressRange(&fd, (CUdeviceptr)lo, hi - lo, CU_MEM_RANGE_HANDLE_TYPE_DMA_BUF_FD, 0)));
  *fd_out = fd;
  *offset_out = p - lo;
  return kSuccess;
}

#endif

}  // namespace cu
}  // namespace tcpxb
