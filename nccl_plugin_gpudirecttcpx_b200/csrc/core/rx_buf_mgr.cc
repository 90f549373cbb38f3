#include "tcpxb/rx_buf_mgr.h"

#include <algorithm>
#include <map>
#include <memory>
#include <unistd.h>

#include <stdio.h>
#include <sys/mman.h>
#include <sys/stat.h>

#include "tcpxb/cu_driver.h"
#include "tcpxb/flags.h"
#include "tcpxb/gpu.h"
#include "tcpxb/rxdm.h"
#include "tcpxb/rxdm_proto.h"

namespace tcpxb {

PageAllocator::PageAllocator(uint32_t n_pages, bool scatter, uint64_t seed, uint32_t run_pages)
    : total_(n_pages), in_use_(n_pages, 0) {
  if (run_pages < 1) run_pages = 1;
  // order in which pages are handed out: groups of run_pages, ascending inside a group
  std::vector<uint32_t> groups((n_pages + run_pages - 1) / run_pages);
  for (uint32_t g = 0; g < groups.size(); ++g) groups[g] = g;
  if (scatter && groups.size() > 1) {
    // Fisher-Yates with a fixed xorshift stream: reproducible scatter
    uint64_t x = seed ? seed : 1;
    for (uint32_t i = (uint32_t)groups.size() - 1; i > 0; --i) {
      x ^= x << 13; x ^= x >> 7; x ^= x << 17;
      uint32_t j = (uint32_t)(x % (i + 1));
      std::swap(groups[i], groups[j]);
    }
  }
  stack_.reserve(n_pages);
  // back() is handed out first, so fill from the last page of the last group
  for (size_t gi = groups.size(); gi > 0; --gi) {
    const uint32_t first = groups[gi - 1] * run_pages;
    const uint32_t last = std::min(first + run_pages, n_pages);
    for (uint32_t p = last; p > first; --p) stack_.push_back(p - 1);
  }
}

bool PageAllocator::alloc(uint32_t n, std::vector<PageRun>* out, bool from_reservation) {
  if (n > stack_.size()) return false;
  if (from_reservation) reserved_ -= std::min(n, reserved_);
  else if (stack_.size() - n < reserved_) return false;  // would eat into somebody's promise
  for (uint32_t i = 0; i < n; ++i) {
    const uint32_t page = stack_.back();
    stack_.pop_back();
    in_use_[page] = 1;
    if (!out->empty() && i > 0 && out->back().first + out->back().count == page) ++out->back().count;
    else out->push_back({page, 1});
  }
  return true;
}

bool PageAllocator::reserve(uint32_t n) {
  if (stack_.size() < (size_t)reserved_ + n) return false;
  reserved_ += n;
  return true;
}

void PageAllocator::unreserve(uint32_t n) { reserved_ -= std::min(n, reserved_); }

void PageAllocator::release(uint32_t first, uint32_t count) {
  // pushed in descending order so the run comes out ascending (contiguous) again
  for (uint32_t i = count; i > 0; --i) {
    const uint32_t page = first + i - 1;
    if (page >= total_ || !in_use_[page]) {
      WARN("rx page %u released twice or out of range", page);
      continue;
    }
    in_use_[page] = 0;
    stack_.push_back(page);
  }
}

namespace {

class EmulatedRxBufMgr final : public RxBufMgr {
 public:
  EmulatedRxBufMgr(int dev, uint64_t bytes, bool scatter, bool device_resident, uint32_t run_pages)
      : dev_(dev), bytes_(bytes / kRxPageBytes * kRxPageBytes), device_resident_(device_resident),
        alloc_((uint32_t)(bytes / kRxPageBytes), scatter, 0x9e3779b97f4a7c15ull, run_pages) {}

  ~EmulatedRxBufMgr() override {
    if (device_resident_) gpu::deviceFree(dev_base_);
    gpu::hostFreeMapped(host_base_);
  }

  Result init() {
    void* h = nullptr;
    void* d = nullptr;
    TCPXB_CHECK(gpu::hostAllocMapped(bytes_, &h, &d));
    host_base_ = static_cast<uint8_t*>(h);
    dev_base_ = static_cast<uint8_t*>(d);
    if (device_resident_) {
      void* p = nullptr;
      TCPXB_CHECK(gpu::deviceAlloc(bytes_, &p));
      dev_base_ = static_cast<uint8_t*>(p);
    }
    INFO(kSubInit | kSubNet, "rx pool for GPU %d: %lu MiB, %s, host %p device %p", dev_,
         (unsigned long)(bytes_ >> 20), device_resident_ ? "device memory + pinned mirror" : "pinned, device-mapped",
         (void*)host_base_, (void*)dev_base_);
    return kSuccess;
  }

  uint8_t* hostBase() override { return host_base_; }
  uint8_t* devBase() override { return dev_base_; }
  uint64_t bytes() const override { return bytes_; }
  bool deviceResident() const override { return device_resident_; }

  bool allocPages(uint32_t n, std::vector<PageRun>* out, bool from_reservation) override {
    std::lock_guard<std::mutex> l(mu_);
    return alloc_.alloc(n, out, from_reservation);
  }
  bool reservePages(uint32_t n) override {
    std::lock_guard<std::mutex> l(mu_);
    return alloc_.reserve(n);
  }
  void unreservePages(uint32_t n) override {
    std::lock_guard<std::mutex> l(mu_);
    alloc_.unreserve(n);
  }
  uint32_t totalPages() override { return alloc_.totalPages(); }
  void releasePages(const PageRun* runs, size_t n) override {
    std::lock_guard<std::mutex> l(mu_);
    for (size_t i = 0; i < n; ++i) alloc_.release(runs[i].first, runs[i].count);
  }
  uint32_t freePages() override {
    std::lock_guard<std::mutex> l(mu_);
    return alloc_.freePages();
  }

  Result installFlowRule(int fd, const std::string& gpu_pci) override {
    FlowRule r;
    memset(&r.local, 0, sizeof r.local);
    memset(&r.peer, 0, sizeof r.peer);
    socklen_t ll = sizeof r.local, pl = sizeof r.peer;
    if (getsockname(fd, &r.local.sa, &ll) != 0 || getpeername(fd, &r.peer.sa, &pl) != 0) return kSystemError;
    r.gpu_pci = gpu_pci;
    r.fd = fd;
    std::lock_guard<std::mutex> l(mu_);
    rules_.push_back(r);
    TRACE(kSubNet, "flow rule %s -> %s steers to GPU %s", addressToString(r.peer).c_str(),
          addressToString(r.local).c_str(), gpu_pci.c_str());
    return kSuccess;
  }
  Result removeFlowRule(int fd) override {
    std::lock_guard<std::mutex> l(mu_);
    rules_.erase(std::remove_if(rules_.begin(), rules_.end(), [fd](const FlowRule& r) { return r.fd == fd; }),
                 rules_.end());
    return kSuccess;
  }
  Result registerApplication(int pid) override {
    std::lock_guard<std::mutex> l(mu_);
    apps_.push_back(pid);
    return kSuccess;
  }
  Result deregisterApplication(int pid) override {
    std::lock_guard<std::mutex> l(mu_);
    apps_.erase(std::remove(apps_.begin(), apps_.end(), pid), apps_.end());
    return kSuccess;
  }
  std::vector<FlowRule> flowRules() override {
    std::lock_guard<std::mutex> l(mu_);
    return rules_;
  }

 private:
  int dev_;
  uint64_t bytes_;
  bool device_resident_;
  std::mutex mu_;
  PageAllocator alloc_;
  uint8_t* host_base_ = nullptr;
  uint8_t* dev_base_ = nullptr;
  std::vector<FlowRule> rules_;
  std::vector<int> apps_;
};

// Pool, rules and registry live in the tcpxb_rxdm daemon; this process maps the pool
// it is handed (a descriptor over SCM_RIGHTS) and allocates pages from it locally, as
// the NIC + kernel would on a devmem-TCP host.  A host pool is a memfd: mapped and
// registered with CUDA.  A device pool is a shareable handle of GPU memory the daemon
// allocated: imported and mapped through the driver's virtual memory API (reference:
// src/gpu/common.cu:25-65); without a devmem NIC to write into it, payload lands in a
// pinned mirror of the same size and the copy engine places each page run.
class DaemonRxBufMgr final : public RxBufMgr {
 public:
  DaemonRxBufMgr(int dev, std::string prefix) : dev_(dev), prefix_(std::move(prefix)) {}
  ~DaemonRxBufMgr() override {
    if (device_pool_) {
      cu::sharedRelease(&imported_);
      cu::ipcRelease(&ipc_);
      gpu::hostFreeMapped(host_base_);
    } else if (host_base_ != nullptr) {
      gpu::hostUnregister(host_base_);
      munmap(host_base_, bytes_);
    }
    if (pool_fd_ >= 0) close(pool_fd_);
  }

  Result init() {
    pci_ = dev_ >= 0 ? gpu::pciBusId(dev_) : std::string("host");
    if (pci_.empty()) pci_ = "gpu" + std::to_string(dev_);
    proto_wire_ = flags().rxdm_wire_proto;
    if (!flags().rxmem_import_use_gpu_pci_client) {
      // The reference's older import (reference: src/gpu/rx_pool.cu:30-55, chosen by
      // NCCL_TCPX_RXMEM_IMPORT_USE_GPU_PCI_CLIENT=0): the pool's owner left a 64-byte memory handle
      // in <prefix>/nvdma-<pci>; open it and ask the driver how large the allocation is.
      if (dev_ < 0) { WARN("the memory-handle import needs a GPU"); return kInvalidUsage; }
      const std::string path = prefix_ + "/nvdma-" + pci_;
      unsigned char handle[cu::kIpcHandleBytes];
      FILE* f = fopen(path.c_str(), "rb");
      if (f == nullptr) { WARN("no memory handle at %s: %s", path.c_str(), strerror(errno)); return kSystemError; }
      const size_t got = fread(handle, 1, sizeof handle, f);
      fclose(f);
      if (got != sizeof handle) { WARN("%s holds %zu bytes, a memory handle has %zu", path.c_str(), got, sizeof handle); return kRemoteError; }
      TCPXB_CHECK(cu::deviceInit(dev_));
      if (cu::ipcOpen(dev_, handle, &ipc_) != kSuccess) { WARN("opening the memory handle of %s failed: %s", path.c_str(), cu::lastError()); return kUnhandledCudaError; }
      bytes_ = ipc_.bytes / kRxPageBytes * kRxPageBytes;
      device_pool_ = true;
      legacy_ipc_ = true;
    } else if (proto_wire_) {
      // the reference's exchange: one socket pair per GPU, the request carries the PCI
      // address as raw bytes, the descriptor comes first and {fd, size, align} second
      // (reference: src/gpu/rx_pool.cu:62-124)
      rxproto::Message q, rep;
      q.kind = rxproto::kRawBytes;
      q.raw_bytes = pci_;
      TCPXB_CHECK(rxproto::call(prefix_, "get_gpu_fd_" + pci_, q, nullptr, &pool_fd_));
      TCPXB_CHECK(rxproto::call(prefix_, "get_gpu_metadata_" + pci_, q, &rep, nullptr));
      rxproto::GpuMemMetadata md;
      if (rep.kind != rxproto::kRawBytes || !rxproto::decodeMetadata(rep.raw_bytes, &md)) {
        WARN("rx buffer manager sent no pool metadata for %s", pci_.c_str());
        return kRemoteError;
      }
      bytes_ = md.size / kRxPageBytes * kRxPageBytes;
      // That daemon only hands out device memory and says nothing about the kind.  This
      // repository's daemon can also serve a memfd of host memory, which is a regular
      // file of the pool's size; a shareable handle of device memory is not.
      struct stat sb;
      device_pool_ = !(pool_fd_ >= 0 && fstat(pool_fd_, &sb) == 0 && S_ISREG(sb.st_mode) && (uint64_t)sb.st_size >= md.size);
    } else {
      RxdmMessage q, rep;
      memset(&q, 0, sizeof q);
      q.magic = kRxdmMagic;
      q.type = kRxdmGetGpuMetadata;
      snprintf(q.gpu.gpu_pci, sizeof q.gpu.gpu_pci, "%s", pci_.c_str());
      TCPXB_CHECK(rxdmCall(prefix_, "get_gpu_metadata", q, &rep, nullptr));
      bytes_ = rep.reply.a / kRxPageBytes * kRxPageBytes;
      device_pool_ = rep.reply.c == (uint64_t)kRxdmPoolDevice;
      q.type = kRxdmGetGpuFd;
      TCPXB_CHECK(rxdmCall(prefix_, "get_gpu_fd", q, &rep, &pool_fd_));
    }
    if ((pool_fd_ < 0 && !legacy_ipc_) || bytes_ == 0) { WARN("rx buffer manager sent no pool for %s", pci_.c_str()); return kRemoteError; }
    if (bytes_ > (4ull << 30)) { WARN("rx pool of %lu bytes is larger than 4 GiB (record offsets are 32-bit)", (unsigned long)bytes_); return kInvalidUsage; }
    if (device_pool_) {
      if (dev_ < 0) { WARN("a device rx pool needs a GPU"); return kInvalidUsage; }
      if (legacy_ipc_) {
        dev_base_ = static_cast<uint8_t*>(ipc_.dptr);
      } else {
        TCPXB_CHECK(cu::deviceInit(dev_));
        TCPXB_CHECK(cu::sharedImport(dev_, pool_fd_, bytes_, &imported_));
        dev_base_ = static_cast<uint8_t*>(imported_.dptr);
      }
      void* h = nullptr;
      void* hd = nullptr;
      TCPXB_CHECK(gpu::hostAllocMapped(bytes_, &h, &hd));  // landing mirror
      host_base_ = static_cast<uint8_t*>(h);
    } else {
      void* p = mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, pool_fd_, 0);
      if (p == MAP_FAILED) { WARN("mapping the rx pool failed: %s", strerror(errno)); return kSystemError; }
      host_base_ = static_cast<uint8_t*>(p);
      void* d = nullptr;
      TCPXB_CHECK(gpu::hostRegisterMapped(host_base_, bytes_, &d));
      dev_base_ = static_cast<uint8_t*>(d);
    }
    const Flags& f = flags();
    // a device pool is filled by the copy engine one page run at a time: keep runs contiguous
    alloc_ = std::make_unique<PageAllocator>((uint32_t)(bytes_ / kRxPageBytes), f.rx_pool_scatter != 0 && !device_pool_,
                                             0x9e3779b97f4a7c15ull, (uint32_t)f.rx_pool_run_pages);
    INFO(kSubInit | kSubNet, "rx pool for %s imported from %s: %lu MiB of %s memory, host %p device %p", pci_.c_str(), prefix_.c_str(),
         (unsigned long)(bytes_ >> 20), device_pool_ ? "device" : "host", (void*)host_base_, (void*)dev_base_);
    return kSuccess;
  }

  uint8_t* hostBase() override { return host_base_; }
  uint8_t* devBase() override { return dev_base_; }
  uint64_t bytes() const override { return bytes_; }
  bool deviceResident() const override { return device_pool_; }
  bool allocPages(uint32_t n, std::vector<PageRun>* out, bool from_reservation) override {
    std::lock_guard<std::mutex> l(mu_);
    return alloc_->alloc(n, out, from_reservation);
  }
  bool reservePages(uint32_t n) override {
    std::lock_guard<std::mutex> l(mu_);
    return alloc_->reserve(n);
  }
  void unreservePages(uint32_t n) override {
    std::lock_guard<std::mutex> l(mu_);
    alloc_->unreserve(n);
  }
  uint32_t totalPages() override { return alloc_->totalPages(); }
  void releasePages(const PageRun* runs, size_t n) override {
    std::lock_guard<std::mutex> l(mu_);
    for (size_t i = 0; i < n; ++i) alloc_->release(runs[i].first, runs[i].count);
  }
  uint32_t freePages() override {
    std::lock_guard<std::mutex> l(mu_);
    return alloc_->freePages();
  }

  Result installFlowRule(int fd, const std::string& gpu_pci) override {
    FlowRule r;
    memset(&r.local, 0, sizeof r.local);
    memset(&r.peer, 0, sizeof r.peer);
    socklen_t ll = sizeof r.local, pl = sizeof r.peer;
    if (getsockname(fd, &r.local.sa, &ll) != 0 || getpeername(fd, &r.peer.sa, &pl) != 0) return kSystemError;
    r.gpu_pci = gpu_pci.empty() ? pci_ : gpu_pci;
    r.fd = fd;
    if (proto_wire_) {
      TCPXB_CHECK(protoRuleCall("rx_rule_manager", r));
    } else {
      RxdmMessage rep;
      TCPXB_CHECK(rxdmCall(prefix_, "rx_rule_manager", rxdmMakeRule(kRxdmFlowRule, r.local, r.peer, r.gpu_pci), &rep, nullptr));
    }
    std::lock_guard<std::mutex> l(mu_);
    rules_.push_back(r);
    return kSuccess;
  }
  Result removeFlowRule(int fd) override {
    FlowRule found;
    bool have = false;
    {
      std::lock_guard<std::mutex> l(mu_);
      for (size_t i = 0; i < rules_.size(); ++i)
        if (rules_[i].fd == fd) { found = rules_[i]; rules_.erase(rules_.begin() + (long)i); have = true; break; }
    }
    if (!have) return kSuccess;
    if (proto_wire_) return protoRuleCall("rx_rule_uninstall", found);
    RxdmMessage rep;
    return rxdmCall(prefix_, "rx_rule_uninstall", rxdmMakeRule(kRxdmFlowRuleUninstall, found.local, found.peer, found.gpu_pci),
                    &rep, nullptr);
  }
  Result registerApplication(int pid) override {
    if (proto_wire_) {
      // the registration is the open connection here too; the daemon learns the pid from the socket's credentials
      rxproto::Message m, rep;
      m.kind = rxproto::kAppRegister;
      m.register_client = true;
      int fd = -1;
      TCPXB_CHECK(proto_keepalive_.connectTo(prefix_ + "/rxdm_application_registry"));
      TCPXB_CHECK(proto_keepalive_.sendMessage(m));
      Result r = proto_keepalive_.recv(&rep, &fd);
      if (fd >= 0) close(fd);
      return r == kSuccess ? kSuccess : kRemoteError;
    }
    RxdmMessage m, rep;
    memset(&m, 0, sizeof m);
    m.magic = kRxdmMagic;
    m.type = kRxdmAppRegister;
    m.app.register_client = 1;
    m.app.pid = pid;
    // the registration is the connection: the daemon drops the entry when it closes
    TCPXB_CHECK(keepalive_.connectTo(prefix_ + "/rxdm_application_registry"));
    TCPXB_CHECK(keepalive_.send(m));
    Result r = keepalive_.recv(&rep, nullptr);
    return (r == kSuccess && rep.reply.status == 0) ? kSuccess : kRemoteError;
  }
  Result deregisterApplication(int /*pid*/) override {
    if (proto_wire_ && proto_keepalive_.fd() >= 0) {
      rxproto::Message m, rep;
      m.kind = rxproto::kAppRegister;
      m.register_client = false;
      (void)rxproto::call(prefix_, "rxdm_application_registry", m, &rep, nullptr);
      proto_keepalive_.closeNow();
      return kSuccess;
    }
    keepalive_.closeNow();
    return kSuccess;
  }
  std::vector<FlowRule> flowRules() override {
    std::lock_guard<std::mutex> l(mu_);
    return rules_;
  }

 private:
  Result protoRuleCall(const char* service, const FlowRule& r) {
    rxproto::Message rep;
    TCPXB_CHECK(rxproto::call(prefix_, service, rxproto::makeRule(r.local, r.peer, r.gpu_pci), &rep, nullptr));
    if (rep.kind != rxproto::kRawBytes || rep.raw_bytes != "Ok.") {
      WARN("rx buffer manager refused %s: %s", service, rep.kind == rxproto::kRawBytes ? rep.raw_bytes.c_str() : "(no text)");
      return kRemoteError;
    }
    return kSuccess;
  }

  int dev_;
  std::string prefix_, pci_;
  bool proto_wire_ = false;
  rxproto::Connection proto_keepalive_;
  std::mutex mu_;
  std::unique_ptr<PageAllocator> alloc_;
  uint8_t* host_base_ = nullptr;
  uint8_t* dev_base_ = nullptr;
  uint64_t bytes_ = 0;
  int pool_fd_ = -1;
  bool device_pool_ = false;
  cu::SharedAllocation imported_;
  cu::IpcAllocation ipc_;     // the pool when it came by memory handle
  bool legacy_ipc_ = false;
  std::vector<FlowRule> rules_;
  UnixSocketConnection keepalive_;
};

std::mutex g_mu;
std::map<int, std::unique_ptr<RxBufMgr>> g_mgrs;

}  // namespace

RxBufMgr* rxBufMgrFor(int dev) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_mgrs.find(dev);
  if (it != g_mgrs.end()) return it->second.get();
  const Flags& f = flags();
  if (f.rxmem_import_skip_odds && dev >= 0 && dev % 2 == 1) {
    // the reference's four-pool layout: only even GPUs own receive memory (reference:
    // src/gpu/cuda_wrapper.cu:179-196); a receive into an odd GPU's memory is then an error
    WARN("GPU %d has no rx pool: NCCL_TCPX_RXMEM_IMPORT_SKIP_ODDS leaves odd GPUs without one", dev);
    return nullptr;
  }
  if (f.rx_buf_mgr_daemon) {
    auto m = std::make_unique<DaemonRxBufMgr>(dev, f.unix_client_prefix);
    if (m->init() != kSuccess) return nullptr;
    RxBufMgr* raw = m.get();
    g_mgrs[dev] = std::move(m);
    return raw;
  }
  const bool device_resident = dev >= 0 && f.rx_pool_mode == kRxPoolDevice && gpu::available();
  // a device-resident pool is filled by the copy engine one page run at a time, so
  // its allocator keeps runs contiguous whatever the scatter flag says
  auto m = std::make_unique<EmulatedRxBufMgr>(dev, (uint64_t)f.rx_pool_bytes, f.rx_pool_scatter != 0 && !device_resident,
                                              device_resident, (uint32_t)f.rx_pool_run_pages);
  if (m->init() != kSuccess) return nullptr;
  RxBufMgr* raw = m.get();
  g_mgrs[dev] = std::move(m);
  return raw;
}

RxBufMgr* newHostRxBufMgr(uint64_t bytes, bool scatter, uint32_t run_pages) {
  auto* m = new EmulatedRxBufMgr(-1, bytes, scatter, false, run_pages);
  if (m->init() != kSuccess) { delete m; return nullptr; }
  return m;
}

}  // namespace tcpxb
