// CUDA driver-API services of the transport: context handling for threads the
// library creates, device memory that can be shared between processes by file
// descriptor (the rx page pool a buffer-manager daemon owns and clients import), and
// dma-buf export of registered send buffers.
//
// Counterpart of the reference's driver-API wrapper (reference:
// src/gpu/cuda_wrapper.cu:68-98 primary context retained or an own context created,
// push/pop around calls from helper threads; src/gpu/common.cu:25-65 import of a
// shareable handle: reserve, map, set access; src/gpu/tx_pool.cu:104-181 dma-buf fd
// of a registered buffer).  The driver library is loaded with dlopen at first use,
// so nothing links against it and CPU-only machines run everything else.
//
// In the host-only build (TCPXB_NO_CUDA) with the stand-in device (TCPXB_FAKE_GPU)
// the same interface is served from host memory: a "device allocation" is a memfd,
// exporting it duplicates the descriptor, importing maps it, and a dma-buf of a range
// inside such an allocation is again that descriptor plus an offset.  That keeps the
// daemon's pool hand-over and the registration path testable without a GPU.
#ifndef TCPXB_CU_DRIVER_H_
#define TCPXB_CU_DRIVER_H_

#include <stddef.h>
#include <stdint.h>

#include "tcpxb/base.h"

namespace tcpxb {
namespace cu {

// True when the driver library (or the stand-in) can be used.
bool available();
const char* lastError();

// ---- contexts ---------------------------------------------------------------------
// Chooses, once per device, the context this library's own threads use: the device's
// primary context (retained; NCCL_GPUDIRECTTCPX_CUDA_USE_PRIMARY_CTX=1, the default,
// which is also what the runtime API uses) or a context of the library's own (=0).
// An own context cannot reach memory the application allocated in the primary one, so
// it is created only for a caller that says it owns all the device memory it touches
// (`owns_its_memory`: the buffer manager daemon); everybody else gets the primary context.
Result deviceInit(int dev, bool owns_its_memory = false);
// Whether deviceInit created an own context for `dev` (false: primary, or not initialised).
bool usesOwnContext(int dev);
// Makes the chosen context current on the calling thread for the lifetime of the
// object (push in the constructor, pop in the destructor), as helper threads must
// before they touch the device.  Cheap when the context is already current.
class ScopedContext {
 public:
  explicit ScopedContext(int dev);
  ~ScopedContext();
  bool ok() const { return ok_; }
  ScopedContext(const ScopedContext&) = delete;
  ScopedContext& operator=(const ScopedContext&) = delete;
 private:
  bool pushed_ = false, ok_ = false;
};
// Releases what deviceInit took (tests; process exit does it anyway).
void deviceShutdown(int dev);

// ---- device memory shared by file descriptor ----------------------------------------
struct SharedAllocation {
  void* dptr = nullptr;    // address of the mapping in this process
  size_t bytes = 0;        // mapped size (a multiple of the granularity)
  uint64_t handle = 0;     // allocation handle (released with the mapping)
  int dev = -1;
  bool imported = false;
};
// Smallest size step of shareable allocations on `dev` (2 MiB on current GPUs).
size_t sharedGranularity(int dev);
// Owner side: allocates `bytes` (rounded up to the granularity) of device memory on
// `dev`, maps it read-write in this process and returns a POSIX file descriptor that
// another process can import.  The caller closes *fd_out when it has been sent.
Result sharedCreate(int dev, size_t bytes, SharedAllocation* out, int* fd_out);
// Client side: maps the allocation behind `fd` (as received over a UNIX socket)
// read-write on `dev`.  `bytes` is the size the owner announced.
Result sharedImport(int dev, int fd, size_t bytes, SharedAllocation* out);
void sharedRelease(SharedAllocation* a);

// ---- device memory shared by an opaque handle (CUDA IPC), the older of the two ways -------
// The reference's first import path reads a 64-byte CUipcMemHandle that the pool's owner left
// in a file and opens it (reference: src/gpu/rx_pool.cu:30-55).  Owner: ordinary device memory
// (`cuMemAlloc`) and its handle.  Client: the mapping of that memory in another process; its
// size comes from the driver's address-range query.  A handle cannot be opened by the process
// that made it.
constexpr size_t kIpcHandleBytes = 64;
struct IpcAllocation {
  void* dptr = nullptr;
  size_t bytes = 0;
  int dev = -1;
  bool opened = false;  // true: a client's mapping (closed, not freed, on release)
};
Result ipcCreate(int dev, size_t bytes, IpcAllocation* out, unsigned char handle[kIpcHandleBytes]);
Result ipcOpen(int dev, const unsigned char handle[kIpcHandleBytes], IpcAllocation* out);
void ipcRelease(IpcAllocation* a);

// ---- stream-ordered host flags -----------------------------------------------------------
// Makes `stream` write `value` to the 32-bit word at device address `dev_word` (pinned,
// device-mapped host memory) once everything queued before it has finished, with the
// driver's stream memory operation.  kInvalidUsage when the driver offers none.
Result streamWriteValue32(void* stream, void* dev_word, uint32_t value);

// ---- dma-buf export ---------------------------------------------------------------------
// A dma-buf file descriptor covering the device range [ptr, ptr + bytes): what a
// devmem-capable NIC driver binds for zero-copy transmit.  The exported range is
// widened to host-page boundaries as the driver requires; *offset_out is the
// position of `ptr` inside the exported range.  The caller owns *fd_out.
Result exportDmabuf(const void* ptr, size_t bytes, int* fd_out, uint64_t* offset_out);

}  // namespace cu
}  // namespace tcpxb
#endif  // TCPXB_CU_DRIVER_H_
