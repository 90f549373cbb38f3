// Thin, lazily initialised wrapper over the CUDA runtime for the host core.
//
// Plays the part of the reference's GPU wrapper (reference: src/gpu/cuda_wrapper.h:22-41,
// src/gpu/cuda_wrapper.cu:68-143 lazy per-GPU init and current-device lookup,
// :278-282 NUMA heuristic).  Differences: the runtime is linked statically and only
// touched when a CUDA pointer or a device handle shows up, so the host-memory path
// runs on machines with no GPU and no driver; and when the core is compiled with
// TCPXB_NO_CUDA every call reports "no CUDA" and pinned allocations fall back to
// page-aligned host memory, which keeps the buffer-manager logic testable on CPUs.
// A TCPXB_NO_CUDA build started with TCPXB_FAKE_GPU=1 goes one step further: it
// presents one stand-in device whose memory is host memory (copies are memcpy,
// events are always complete), so that the paths that take CUDA pointers can be
// driven end to end, under the sanitizers, without a GPU.
#ifndef TCPXB_GPU_H_
#define TCPXB_GPU_H_

#include <stddef.h>
#include <stdint.h>
#include <string>

#include "tcpxb/base.h"

namespace tcpxb {
namespace gpu {

bool compiledWithCuda();
// False only for the host-only build's stand-in device in its timing mode (TCPXB_FAKE_GPU=2),
// where copies and kernels are skipped so that only the host side of the data path costs time.
bool standinMovesData();
// True when a pointer handed to the transport may be device memory: always in a
// CUDA build (the runtime is not touched to answer), only with the stand-in device
// otherwise.
bool devicePointersPossible();
// True when the CUDA runtime initialises and reports at least one device.
bool available();
int deviceCount();
Result currentDevice(int* dev);
Result setDevice(int dev);
// Classifies a pointer: *is_device is true for device (and managed) memory.
Result pointerInfo(const void* p, int* device, bool* is_device);
std::string pciBusId(int dev);  // lower case, "" when unknown
int numaNode(int dev);          // sysfs, else dev < count/2 ? 0 : 1

// Pinned, portable, device-mapped host memory.  *dev_ptr receives the address the
// GPU uses (equal to the host address under unified addressing).  Without CUDA
// this is page-aligned host memory and *dev_ptr == *host_ptr.
Result hostAllocMapped(size_t bytes, void** host_ptr, void** dev_ptr);
void hostFreeMapped(void* host_ptr);
// Makes existing page-aligned host memory (e.g. a shared mapping) pinned and visible
// to the GPU; *dev_ptr is the address the GPU uses.  Without CUDA: *dev_ptr = host_ptr.
Result hostRegisterMapped(void* host_ptr, size_t bytes, void** dev_ptr);
void hostUnregister(void* host_ptr);
Result deviceAlloc(size_t bytes, void** ptr);
void deviceFree(void* ptr);

using Stream = void*;
using Event = void*;
Result streamCreate(Stream* s);      // non-blocking stream
void streamDestroy(Stream s);
Result eventCreate(Event* e);        // timing disabled
void eventDestroy(Event e);
Result eventRecord(Event e, Stream s);
// kSuccess when complete, kInProgress when not, error otherwise.
Result eventQuery(Event e);
Result streamSynchronize(Stream s);
Result streamWaitEvent(Stream s, Event e);
Result eventSynchronize(Event e);
Result copyDeviceToDeviceAsync(void* dst, const void* src, size_t bytes, Stream s);
Result copyToHostAsync(void* host_dst, const void* dev_src, size_t bytes, Stream s);
Result copyToDeviceAsync(void* dev_dst, const void* host_src, size_t bytes, Stream s);
Result memsetAsync(void* dev, int value, size_t bytes, Stream s);

// A counter in pinned, device-mapped host memory that streams advance: mark() queues
// "counter = next value" behind everything already in the stream, reached() is one plain
// load.  It stands where a CUDA event per point would: no event to create, record or
// query, which matters to a thread that tracks hundreds of copies and kernels per
// millisecond.  Marks must be issued in the order in which they will complete (one
// stream, or streams the caller orders).
class StreamCounter {
 public:
  StreamCounter() = default;
  ~StreamCounter();
  StreamCounter(const StreamCounter&) = delete;
  StreamCounter& operator=(const StreamCounter&) = delete;
  Result init();
  bool ready() const { return host_ != nullptr; }
  // Queues the next value on `s` and returns it in *value.
  Result mark(Stream s, uint32_t* value);
  bool reached(uint32_t value) const { return (int32_t)(__atomic_load_n(host_, __ATOMIC_ACQUIRE) - value) >= 0; }
  uint32_t issued() const { return issued_; }

 private:
  uint32_t* host_ = nullptr;
  uint32_t* dev_ = nullptr;
  uint32_t issued_ = 0;
  bool use_kernel_ = false;  // the driver has no stream memory operation: a one-thread kernel writes instead
};

const char* lastError();

}  // namespace gpu
}  // namespace tcpxb
#endif  // TCPXB_GPU_H_
