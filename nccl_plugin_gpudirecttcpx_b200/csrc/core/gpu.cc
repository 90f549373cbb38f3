#include "tcpxb/gpu.h"

#include "tcpxb/cu_driver.h"
#include "tcpxb/kernels.h"

#include <ctype.h>
#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#ifndef TCPXB_NO_CUDA
#include <cuda_runtime_api.h>
#endif

namespace tcpxb {
namespace gpu {

namespace {
thread_local char g_err[256] = "";
}
const char* lastError() { return g_err; }

#ifdef TCPXB_NO_CUDA

// Without CUDA there are two behaviours.  By default every call reports "no CUDA".
// With TCPXB_FAKE_GPU=1 in the environment the calls act on host memory instead: one
// "device" whose memory is the process's own, copies that are memcpy, streams that
// run everything at once and events that are always complete.  That lets the
// CUDA-buffer send path, the page pool, the scatter lists and the device-handle
// protocol run, and be checked by the sanitizers, on machines with no GPU.
namespace {
bool fake() {
  static const bool on = [] {
    const char* v = getenv("TCPXB_FAKE_GPU");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return on;
}
Result none() {
  snprintf(g_err, sizeof g_err, "built without CUDA");
  return kUnhandledCudaError;
}
// TCPXB_FAKE_GPU=2: the stand-in device's copies and kernels move no data, as if a
// copy engine and SMs did the work for free.  Results are then meaningless; the
// setting exists to time the host side of the data path on a machine with no GPU.
bool fakeMovesData() {
  static const bool moves = [] {
    const char* v = getenv("TCPXB_FAKE_GPU");
    return !(v != nullptr && v[0] == '2');
  }();
  return moves;
}
int g_fake_stream_tag, g_fake_event_tag;
}  // namespace

bool standinMovesData() { return fakeMovesData(); }

bool compiledWithCuda() { return false; }
bool devicePointersPossible() { return fake(); }
bool available() { return fake(); }
int deviceCount() { return fake() ? 1 : 0; }
Result currentDevice(int* dev) {
  if (!fake()) return none();
  *dev = 0;
  return kSuccess;
}
Result setDevice(int dev) { return fake() && dev == 0 ? kSuccess : none(); }
Result pointerInfo(const void*, int* device, bool* is_device) {
  // every pointer a caller declares as device memory is taken at its word
  *device = fake() ? 0 : -1;
  *is_device = fake();
  return kSuccess;
}
std::string pciBusId(int) { return fake() ? "0000:00:00.0" : ""; }
int numaNode(int) { return 0; }
Result hostAllocMapped(size_t bytes, void** host_ptr, void** dev_ptr) {
  void* p = nullptr;
  if (posix_memalign(&p, 4096, bytes ? bytes : 4096) != 0) return kSystemError;
  *host_ptr = p;
  *dev_ptr = p;
  return kSuccess;
}
void hostFreeMapped(void* p) { free(p); }
Result hostRegisterMapped(void* host_ptr, size_t, void** dev_ptr) { *dev_ptr = host_ptr; return kSuccess; }
void hostUnregister(void*) {}
Result deviceAlloc(size_t bytes, void** ptr) {
  if (!fake()) return none();
  void* p = nullptr;
  if (posix_memalign(&p, 256, bytes ? bytes : 256) != 0) return kSystemError;
  *ptr = p;
  return kSuccess;
}
void deviceFree(void* p) { free(p); }
Result streamCreate(Stream* s) {
  if (!fake()) return none();
  *s = &g_fake_stream_tag;
  return kSuccess;
}
void streamDestroy(Stream) {}
Result eventCreate(Event* e) {
  if (!fake()) return none();
  *e = &g_fake_event_tag;
  return kSuccess;
}
void eventDestroy(Event) {}
Result eventRecord(Event, Stream) { return fake() ? kSuccess : none(); }
Result eventQuery(Event) { return fake() ? kSuccess : none(); }
Result streamSynchronize(Stream) { return fake() ? kSuccess : none(); }
Result streamWaitEvent(Stream, Event) { return fake() ? kSuccess : none(); }
Result eventSynchronize(Event) { return fake() ? kSuccess : none(); }
static Result fakeCopy(void* dst, const void* src, size_t bytes) {
  if (!fake()) return none();
  if (fakeMovesData()) memmove(dst, src, bytes);
  return kSuccess;
}
Result copyDeviceToDeviceAsync(void* d, const void* s, size_t n, Stream) { return fakeCopy(d, s, n); }
Result copyToHostAsync(void* d, const void* s, size_t n, Stream) { return fakeCopy(d, s, n); }
Result copyToDeviceAsync(void* d, const void* s, size_t n, Stream) { return fakeCopy(d, s, n); }
Result memsetAsync(void* p, int value, size_t n, Stream) {
  if (!fake()) return none();
  memset(p, value, n);
  return kSuccess;
}

#else  // CUDA build

namespace {
Result check(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return kSuccess;
  snprintf(g_err, sizeof g_err, "%s: %s", what, cudaGetErrorString(e));
  WARN("CUDA call failed: %s", g_err);
  return kUnhandledCudaError;
}
#define CU(expr) check((expr), #expr)

int probeCount() {
  static int count = [] {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();  // clear the sticky "no device / no driver" state
      return 0;
    }
    return n;
  }();
  return count;
}
}  // namespace

bool compiledWithCuda() { return true; }
bool standinMovesData() { return true; }
bool devicePointersPossible() { return true; }
int deviceCount() { return probeCount(); }
bool available() { return probeCount() > 0; }

Result currentDevice(int* dev) { return CU(cudaGetDevice(dev)); }
Result setDevice(int dev) { return CU(cudaSetDevice(dev)); }

Result pointerInfo(const void* p, int* device, bool* is_device) {
  *device = -1;
  *is_device = false;
  if (!available()) return kSuccess;
  cudaPointerAttributes a;
  cudaError_t e = cudaPointerGetAttributes(&a, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return kSuccess;  // plain host memory on older runtimes
  }
  if (a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged) {
    *is_device = true;
    *device = a.device;
  }
  return kSuccess;
}

std::string pciBusId(int dev) {
  char buf[32] = "";
  if (!available() || cudaDeviceGetPCIBusId(buf, sizeof buf, dev) != cudaSuccess) return "";
  for (char* c = buf; *c; ++c) *c = (char)tolower(*c);
  return buf;
}

int numaNode(int dev) {
  std::string id = pciBusId(dev);
  if (!id.empty()) {
    std::string path = "/sys/bus/pci/devices/" + id + "/numa_node";
    if (FILE* f = fopen(path.c_str(), "r")) {
      int node = -1;
      int got = fscanf(f, "%d", &node);
      fclose(f);
      if (got == 1 && node >= 0) return node;
    }
  }
  const int n = deviceCount();
  return (n > 1 && dev >= n / 2) ? 1 : 0;
}

Result hostAllocMapped(size_t bytes, void** host_ptr, void** dev_ptr) {
  if (!available()) {
    void* p = nullptr;
    if (posix_memalign(&p, 4096, bytes ? bytes : 4096) != 0) return kSystemError;
    *host_ptr = *dev_ptr = p;
    return kSuccess;
  }
  Result r = CU(cudaHostAlloc(host_ptr, bytes, cudaHostAllocMapped | cudaHostAllocPortable));
  if (r != kSuccess) return r;
  return CU(cudaHostGetDevicePointer(dev_ptr, *host_ptr, 0));
}

void hostFreeMapped(void* p) {
  if (p == nullptr) return;
  if (!available()) { free(p); return; }
  if (cudaFreeHost(p) != cudaSuccess) (void)cudaGetLastError();
}

Result hostRegisterMapped(void* host_ptr, size_t bytes, void** dev_ptr) {
  if (!available()) { *dev_ptr = host_ptr; return kSuccess; }
  Result r = CU(cudaHostRegister(host_ptr, bytes, cudaHostRegisterMapped | cudaHostRegisterPortable));
  if (r != kSuccess) return r;
  return CU(cudaHostGetDevicePointer(dev_ptr, host_ptr, 0));
}

void hostUnregister(void* host_ptr) {
  if (host_ptr == nullptr || !available()) return;
  if (cudaHostUnregister(host_ptr) != cudaSuccess) (void)cudaGetLastError();
}

Result deviceAlloc(size_t bytes, void** ptr) { return CU(cudaMalloc(ptr, bytes)); }
void deviceFree(void* p) {
  if (p != nullptr && cudaFree(p) != cudaSuccess) (void)cudaGetLastError();
}

Result streamCreate(Stream* s) {
  cudaStream_t st;
  Result r = CU(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  *s = st;
  return r;
}
void streamDestroy(Stream s) {
  if (s != nullptr && cudaStreamDestroy((cudaStream_t)s) != cudaSuccess) (void)cudaGetLastError();
}
Result eventCreate(Event* e) {
  cudaEvent_t ev;
  Result r = CU(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  *e = ev;
  return r;
}
void eventDestroy(Event e) {
  if (e != nullptr && cudaEventDestroy((cudaEvent_t)e) != cudaSuccess) (void)cudaGetLastError();
}
Result eventRecord(Event e, Stream s) { return CU(cudaEventRecord((cudaEvent_t)e, (cudaStream_t)s)); }
Result eventQuery(Event e) {
  cudaError_t r = cudaEventQuery((cudaEvent_t)e);
  if (r == cudaSuccess) return kSuccess;
  if (r == cudaErrorNotReady) return kInProgress;
  return check(r, "cudaEventQuery");
}
Result streamSynchronize(Stream s) { return CU(cudaStreamSynchronize((cudaStream_t)s)); }
Result streamWaitEvent(Stream s, Event e) { return CU(cudaStreamWaitEvent((cudaStream_t)s, (cudaEvent_t)e, 0)); }
Result eventSynchronize(Event e) { return CU(cudaEventSynchronize((cudaEvent_t)e)); }
Result copyDeviceToDeviceAsync(void* d, const void* s_, size_t n, Stream s) {
  return CU(cudaMemcpyAsync(d, s_, n, cudaMemcpyDeviceToDevice, (cudaStream_t)s));
}
Result copyToHostAsync(void* h, const void* d, size_t n, Stream s) {
  return CU(cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, (cudaStream_t)s));
}
Result copyToDeviceAsync(void* d, const void* h, size_t n, Stream s) {
  return CU(cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, (cudaStream_t)s));
}
Result memsetAsync(void* d, int v, size_t n, Stream s) {
  return CU(cudaMemsetAsync(d, v, n, (cudaStream_t)s));
}

#endif


// ---------------------------------------------------------------- StreamCounter
StreamCounter::~StreamCounter() { hostFreeMapped(host_); }

Result StreamCounter::init() {
  if (host_ != nullptr) return kSuccess;
  void* h = nullptr;
  void* d = nullptr;
  TCPXB_CHECK(hostAllocMapped(64, &h, &d));
  memset(h, 0, 64);
  host_ = static_cast<uint32_t*>(h);
  dev_ = static_cast<uint32_t*>(d);
  return kSuccess;
}

Result StreamCounter::mark(Stream s, uint32_t* value) {
  const uint32_t v = issued_ + 1;
  if (!use_kernel_) {
    Result r = cu::streamWriteValue32(s, dev_, v);
    if (r != kSuccess) use_kernel_ = true;  // no stream memory operations here: fall back for good
  }
  if (use_kernel_) {
    uint32_t* flags[1] = {dev_};
    if (tcpxb_signal_flags(flags, 1, v, s) != 0) {
      snprintf(g_err, sizeof g_err, "stream counter: %s", tcpxb_kernel_last_error());
      return kUnhandledCudaError;
    }
  }
  issued_ = v;
  *value = v;
  return kSuccess;
}

}  // namespace gpu
}  // namespace tcpxb
