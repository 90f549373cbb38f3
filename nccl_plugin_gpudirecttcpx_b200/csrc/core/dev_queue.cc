#include "tcpxb/dev_queue.h"

#include <string.h>

#include "tcpxb/gpu.h"

namespace tcpxb {

DevQueue::~DevQueue() {
  gpu::deviceFree(dev_handle_);
  gpu::hostFreeMapped(meta_host_);
}

Result DevQueue::init(void* bounce_buf_dev, bool want_device_handle) {
  void* h = nullptr;
  void* d = nullptr;
  TCPXB_CHECK(gpu::hostAllocMapped(sizeof(UnpackMeta), &h, &d));
  meta_host_ = static_cast<UnpackMeta*>(h);
  meta_dev_ = static_cast<UnpackMeta*>(d);
  memset(meta_host_->cnt, 0, sizeof meta_host_->cnt);
  if (want_device_handle) {
    UnpackDeviceHandle hd;
    hd.meta = meta_dev_;
    hd.bounce_buf = bounce_buf_dev;
    hd.head = ~0ull;
    void* p = nullptr;
    TCPXB_CHECK(gpu::deviceAlloc(sizeof hd, &p));
    dev_handle_ = p;
    TCPXB_CHECK(gpu::copyToDeviceAsync(p, &hd, sizeof hd, nullptr));
    TCPXB_CHECK(gpu::streamSynchronize(nullptr));
  }
  return kSuccess;
}

void DevQueue::nextFree(UnpackSlot* slot) {
  slot->active = false;
  if (tail_ - head_ >= (uint64_t)kUnpackQueueDepth) return;
  const uint64_t i = tail_ % kUnpackQueueDepth;
  slot->active = true;
  slot->index = i;
  slot->mem = meta_host_->mem[i];
  slot->mem_dev = meta_dev_->mem[i];
  slot->cnt = &meta_host_->cnt[i];
  slot->filled = 0;
  ++tail_;
}

bool DevQueue::release(uint64_t index) {
  if (head_ == tail_ || head_ % kUnpackQueueDepth != index) return false;
  ++head_;
  return true;
}

}  // namespace tcpxb
