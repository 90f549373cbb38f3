// Device-visible scatter-list ring shared between the receive path (producer, on
// the host) and whoever unpacks on the GPU (NCCL's kernels in "unpack" mode, this
// library's kernels otherwise).
//
// Layout and protocol follow NCCL's device-unpack contract as the reference uses
// it (reference: src/devcomm/nccl/unpack1.cu:28-71 allocation and handle,
// src/devcomm/nccl/unpack1.h:30-65 slot allocator, src/devcomm/unpack_defs1.h:39-74):
// a pinned, device-mapped block of `depth` slots, each with room for
// kUnpackMaxSlicePages 16-byte records plus a count; the host fills a slot while a
// request is received and publishes the count last; the consumer frees slots in
// FIFO order.  The device handle is {meta, bounce_buf, head} with head starting at
// all-ones because the consumer increments it before use.
#ifndef TCPXB_DEV_QUEUE_H_
#define TCPXB_DEV_QUEUE_H_

#include <stdint.h>

#include "tcpxb/base.h"

namespace tcpxb {

constexpr int kUnpackQueueDepth = 16;       // NCCL_NET_DEVICE_UNPACK_MAX_QUEUE_DEPTH
constexpr int kUnpackSliceBytes = 4194304;  // NET_UNPACK_MAX_SLICE_SIZE
constexpr int kUnpackPageBytes = 4096;      // SLICE_PAGE_SIZE == NCCL_NET_MTU_SIZE
constexpr int kUnpackMaxSlicePages = kUnpackSliceBytes / kUnpackPageBytes * 2;
constexpr int kUnpackVersion = 0x7;         // NCCL_NET_DEVICE_UNPACK_VERSION

union alignas(16) LoadMeta {
  uint64_t r64[2];
  struct {
    uint32_t src_off;
    uint32_t len;
    uint64_t dst_off;
  };
};
static_assert(sizeof(LoadMeta) == 16, "descriptor format");

struct UnpackMeta {
  LoadMeta mem[kUnpackQueueDepth][kUnpackMaxSlicePages];
  uint64_t cnt[kUnpackQueueDepth];
};

struct UnpackDeviceHandle {
  UnpackMeta* meta;   // device address of the mapped block
  void* bounce_buf;   // device address of the rx page pool
  uint64_t head;
};

struct UnpackSlot {
  bool active = false;
  uint64_t index = 0;         // slot number = sequence % depth
  LoadMeta* mem = nullptr;    // host address of the slot's records
  LoadMeta* mem_dev = nullptr;
  uint64_t* cnt = nullptr;    // host address of the published count
  uint64_t filled = 0;        // records written so far (published at completion)
};

class DevQueue {
 public:
  ~DevQueue();
  // Allocates the mapped block; with `want_device_handle` also the small device
  // struct NCCL's kernels read.
  Result init(void* bounce_buf_dev, bool want_device_handle);
  // Takes the next slot; slot->active stays false when all `depth` are in use.
  void nextFree(UnpackSlot* slot);
  // Releases the oldest slot; false when `index` is not the oldest (FIFO contract).
  bool release(uint64_t index);
  uint64_t inUse() const { return tail_ - head_; }
  void* deviceHandle() const { return dev_handle_; }
  UnpackMeta* metaHost() const { return meta_host_; }
  UnpackMeta* metaDev() const { return meta_dev_; }

 private:
  UnpackMeta* meta_host_ = nullptr;
  UnpackMeta* meta_dev_ = nullptr;
  void* dev_handle_ = nullptr;
  uint64_t head_ = 0, tail_ = 0;
};

}  // namespace tcpxb
#endif  // TCPXB_DEV_QUEUE_H_
