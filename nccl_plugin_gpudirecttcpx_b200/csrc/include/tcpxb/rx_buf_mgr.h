// Receive buffer manager: the GPU-visible rx page pool and the services around it.
//
// In the reference these live outside the plugin: the NIC lands payload in a
// device-memory page pool owned by a separate daemon, which the plugin imports
// over UNIX sockets (reference: src/gpu/rx_pool.cu:62-124), asks for flow-steering
// rules (src/rx_buf_mgr_client/rx_rule_client.cc:38-110, called from
// src/connect.cc:564-592) and registers its pid with
// (src/rx_buf_mgr_client/application_registry_client.cc:28-73); the kernel then
// describes each received fragment as {offset, size, token} and takes pages back
// through a socket option (src/sock/tcpx.h:130-134, :299-326).
//
// Here one in-process object per GPU plays kernel + NIC + daemon ("header-split
// emulation"): payload is received straight into 4096-byte pool pages chosen by a
// page allocator, every page fragment is described with the same
// {src_off, len, dst_off} record, and page tokens return to the allocator when the
// consumer is done.  The pool is pinned host memory mapped into the GPU (default:
// recv() lands in place and the unpack kernels pull fragments over PCIe) or device
// memory fed by the copy engine from a pinned mirror.  Flow-steering and
// application-registry calls keep their call points and are recorded in a table.
#ifndef TCPXB_RX_BUF_MGR_H_
#define TCPXB_RX_BUF_MGR_H_

#include <stdint.h>

#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "tcpxb/base.h"
#include "tcpxb/socket_utils.h"

namespace tcpxb {

constexpr uint32_t kRxPageBytes = 4096;

struct PageRun {
  uint32_t first;  // page index
  uint32_t count;
};

// Hands out pool pages.  Not thread-safe by itself (RxBufMgr locks around it).
class PageAllocator {
 public:
  // `scatter`: groups of `run_pages` consecutive pages come out in a pseudo-random
  // order, like a NIC page pool after some churn (run_pages = 1 scatters single
  // pages); otherwise ascending, so allocations are mostly contiguous.
  PageAllocator(uint32_t n_pages, bool scatter, uint64_t seed = 0x9e3779b97f4a7c15ull, uint32_t run_pages = 1);
  // Appends runs covering exactly n pages; false (and nothing taken) when fewer are
  // free.  Pages promised to reservations are not free for anybody else;
  // `from_reservation` draws on such a promise (the caller tracks how much it holds).
  bool alloc(uint32_t n, std::vector<PageRun>* out, bool from_reservation = false);
  void release(uint32_t first, uint32_t count);
  // All-or-nothing promise of n pages.  A message that reserves everything it needs
  // before it takes its first page can never wait while holding pages, so messages of
  // several connections that share one pool cannot block one another for good.
  bool reserve(uint32_t n);
  void unreserve(uint32_t n);
  uint32_t freePages() const { return (uint32_t)stack_.size(); }
  uint32_t reservedPages() const { return reserved_; }
  uint32_t totalPages() const { return total_; }

 private:
  uint32_t total_;
  uint32_t reserved_ = 0;
  std::vector<uint32_t> stack_;     // free pages; back() is handed out next
  std::vector<uint8_t> in_use_;     // double-release guard
};

struct FlowRule {
  SocketAddress local, peer;
  std::string gpu_pci;
  int fd;
};

class RxBufMgr {
 public:
  virtual ~RxBufMgr() = default;
  // Pool addresses.  hostBase() is where recv() writes (the pool itself, or its
  // pinned mirror in device mode); devBase() is what kernels read.
  virtual uint8_t* hostBase() = 0;
  virtual uint8_t* devBase() = 0;
  virtual uint64_t bytes() const = 0;
  virtual bool deviceResident() const = 0;
  virtual bool allocPages(uint32_t n, std::vector<PageRun>* out, bool from_reservation = false) = 0;
  virtual void releasePages(const PageRun* runs, size_t n) = 0;
  virtual bool reservePages(uint32_t n) = 0;     // see PageAllocator::reserve
  virtual void unreservePages(uint32_t n) = 0;
  virtual uint32_t freePages() = 0;
  virtual uint32_t totalPages() = 0;
  // Service hooks with the reference's call points.
  virtual Result installFlowRule(int fd, const std::string& gpu_pci) = 0;
  virtual Result removeFlowRule(int fd) = 0;
  virtual Result registerApplication(int pid) = 0;
  virtual Result deregisterApplication(int pid) = 0;
  virtual std::vector<FlowRule> flowRules() = 0;
  // devmem transmit: the id under which the NIC knows the dma-buf `dmabuf_fd` (what the
  // privileged side's netlink bind returns).  The in-process managers own no NIC and
  // hand out consecutive ids, which is all the socket layer's bookkeeping needs.
  virtual Result bindTxDmabuf(int dmabuf_fd, uint32_t* id) {
    (void)dmabuf_fd;
    static std::atomic<uint32_t> next{1};
    *id = next.fetch_add(1);
    return kSuccess;
  }
  // The id of the rx pool's own dma-buf binding, as fragment records will name it (0 = unknown: accept any).
  virtual uint32_t rxDmabufId() { return 0; }
};

// The emulator for GPU `dev` (or `dev` = -1: a host-only pool for machines without
// a GPU), created on first use with the sizes and modes the flags give.
RxBufMgr* rxBufMgrFor(int dev);
// Test hook: a private emulator with explicit geometry (host memory only).
RxBufMgr* newHostRxBufMgr(uint64_t bytes, bool scatter, uint32_t run_pages = 1);

}  // namespace tcpxb
#endif  // TCPXB_RX_BUF_MGR_H_
