#include "tcpxb/devmem.h"

#include <errno.h>
#include <linux/errqueue.h>
#include <netinet/in.h>
#include <string.h>

#include <algorithm>
#include <atomic>

#include "tcpxb/rx_buf_mgr.h"

#ifndef SO_EE_ORIGIN_ZEROCOPY
#define SO_EE_ORIGIN_ZEROCOPY 5
#endif
#ifndef MSG_ZEROCOPY
#define MSG_ZEROCOPY 0x4000000
#endif

namespace tcpxb {
namespace devmem {

const SocketOps& systemOps() {
  static const SocketOps ops = {
      [](int fd, struct msghdr* msg, int flags) -> ssize_t { return ::recvmsg(fd, msg, flags); },
      [](int fd, const struct msghdr* msg, int flags) -> ssize_t { return ::sendmsg(fd, msg, flags); },
      [](int fd, int level, int optname, const void* val, socklen_t len) -> int { return ::setsockopt(fd, level, optname, val, len); },
  };
  return ops;
}

namespace {
std::atomic<const SocketOps*> g_test_ops{nullptr};
}
const SocketOps& activeOps() {
  const SocketOps* t = g_test_ops.load(std::memory_order_acquire);
  return t != nullptr ? *t : systemOps();
}
void setOpsForTests(const SocketOps* ops) { g_test_ops.store(ops, std::memory_order_release); }

size_t rxControlBytes(size_t fragments) { return fragments * CMSG_SPACE(sizeof(DmabufCmsg)); }

namespace {
void noteToken(std::vector<DmabufToken>* runs, uint32_t token) {
  if (runs == nullptr) return;
  if (!runs->empty() && runs->back().token_start + runs->back().token_count == token) {
    ++runs->back().token_count;  // the kernel numbers a flow's fragments consecutively: long runs are the rule
    return;
  }
  runs->push_back({token, 1});
}
}  // namespace

Result parseRecv(const struct msghdr* msg, ssize_t returned, uint64_t dst_offset, RxSink* sink) {
  if (msg == nullptr || sink == nullptr || sink->records == nullptr || returned < 0) return kInvalidArgument;
  if (msg->msg_flags & MSG_CTRUNC) {
    WARN("devmem receive: the control buffer (%zu bytes) was too small for the fragments of one recvmsg", (size_t)msg->msg_controllen);
    return kInternalError;
  }
  uint64_t total = 0;
  int fragments = 0;
  Result bad = kSuccess;
  // The walk goes on after the first unusable fragment, recording tokens only: every
  // fragment the kernel reported holds pool pages until its token goes back.
  for (struct cmsghdr* cm = CMSG_FIRSTHDR(const_cast<struct msghdr*>(msg)); cm != nullptr;
       cm = CMSG_NXTHDR(const_cast<struct msghdr*>(msg), cm)) {
    if (cm->cmsg_level != SOL_SOCKET || (cm->cmsg_type != kSoDevmemDmabuf && cm->cmsg_type != kSoDevmemLinear)) continue;
    if (cm->cmsg_len < CMSG_LEN(sizeof(DmabufCmsg))) {
      WARN("devmem receive: control message of %zu bytes is shorter than a fragment record", (size_t)cm->cmsg_len);
      bad = kInternalError;
      continue;
    }
    DmabufCmsg f;
    memcpy(&f, CMSG_DATA(cm), sizeof f);
    if (cm->cmsg_type == kSoDevmemLinear) {
      if (f.frag_size > 0 && bad == kSuccess) {
        // The bytes are in the iovec's host buffer, not in the pool.  The scatter list
        // cannot describe them; the flow is not (or no longer) steered to a devmem queue.
        WARN("devmem receive: %u bytes of payload arrived in host memory (flow not steered to a devmem queue?)", f.frag_size);
        bad = kInternalError;
      }
      continue;
    }
    ++fragments;
    noteToken(sink->tokens, f.frag_token);
    if (bad != kSuccess) continue;
    if (sink->dmabuf_id != 0 && f.dmabuf_id != sink->dmabuf_id) {
      WARN("devmem receive: fragment in dma-buf %u, expected %u", f.dmabuf_id, sink->dmabuf_id);
      bad = kInternalError;
      continue;
    }
    if (f.frag_offset + f.frag_size > sink->pool_bytes || f.frag_offset + f.frag_size > (1ull << 32)) {
      WARN("devmem receive: fragment [%llu, +%u) lies outside the %llu-byte pool", (unsigned long long)f.frag_offset, f.frag_size,
           (unsigned long long)sink->pool_bytes);
      bad = kInternalError;
      continue;
    }
    // one record per fragment; a fragment longer than a page becomes several records
    // so that consumers sized for page fragments can take it
    const uint32_t step = sink->max_fragment ? sink->max_fragment : f.frag_size;
    for (uint32_t off = 0; off < f.frag_size; off += step) {
      if (sink->filled >= sink->capacity) {
        WARN("devmem receive: more than %llu fragments for one message", (unsigned long long)sink->capacity);
        bad = kInternalError;
        break;
      }
      const uint32_t len = std::min(step, f.frag_size - off);
      LoadMeta& m = sink->records[sink->filled++];
      m.src_off = (uint32_t)(f.frag_offset + off);
      m.len = len;
      m.dst_off = dst_offset + total + off;
    }
    total += f.frag_size;
  }
  if (bad != kSuccess) return bad;
  if (fragments == 0 && returned > 0) {
    WARN("devmem receive: %zd bytes returned without any fragment record", returned);
    return kInternalError;
  }
  if (total != (uint64_t)returned) {
    WARN("devmem receive: fragments add up to %llu bytes, recvmsg returned %zd", (unsigned long long)total, returned);
    return kInternalError;
  }
  return kSuccess;
}

ssize_t recvInto(const SocketOps& ops, int fd, size_t want, void* control, size_t control_bytes, uint64_t dst_offset,
                 RxSink* sink) {
  // The iovec only bounds how many bytes this call may take; on a devmem queue
  // nothing is copied into it (linear fragments would be, and are refused).
  static char dummy[64];
  struct iovec iov = {dummy, want};
  struct msghdr msg;
  memset(&msg, 0, sizeof msg);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = control;
  msg.msg_controllen = control_bytes;
  const ssize_t n = ops.recvmsg(fd, &msg, kMsgSockDevmem | MSG_DONTWAIT);
  if (n < 0) return (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) ? -EAGAIN : -(ssize_t)(errno ? errno : EIO);
  if (n == 0) return 0;
  return parseRecv(&msg, n, dst_offset, sink) == kSuccess ? n : -EPROTO;
}

Result recycle(const SocketOps& ops, int fd, std::vector<DmabufToken>* runs, size_t* calls) {
  if (runs == nullptr) return kInvalidArgument;
  for (size_t i = 0; i < runs->size(); i += kMaxDontneedRuns) {
    const size_t n = std::min(kMaxDontneedRuns, runs->size() - i);
    if (calls != nullptr) ++*calls;
    if (ops.setsockopt(fd, SOL_SOCKET, kSoDevmemDontneed, runs->data() + i, (socklen_t)(n * sizeof(DmabufToken))) < 0) {
      WARN("SO_DEVMEM_DONTNEED of %zu token runs failed: %s", n, strerror(errno));
      runs->erase(runs->begin(), runs->begin() + (long)i);  // what was handed back stays handed back
      return kSystemError;
    }
  }
  runs->clear();
  return kSuccess;
}

void buildSend(TxMessage* m, uint32_t dmabuf_id, uint64_t offset, size_t len) {
  memset(m, 0, sizeof *m);
  // with a dma-buf control message the "address" of the iovec is the offset inside the dma-buf
  m->iov.iov_base = reinterpret_cast<void*>(static_cast<uintptr_t>(offset));
  m->iov.iov_len = len;
  m->msg.msg_iov = &m->iov;
  m->msg.msg_iovlen = 1;
  m->msg.msg_control = m->control;
  m->msg.msg_controllen = sizeof m->control;
  struct cmsghdr* cm = CMSG_FIRSTHDR(&m->msg);
  cm->cmsg_level = SOL_SOCKET;
  cm->cmsg_type = kSoDevmemDmabuf;
  cm->cmsg_len = CMSG_LEN(sizeof(uint32_t));
  memcpy(CMSG_DATA(cm), &dmabuf_id, sizeof dmabuf_id);
}

ssize_t sendFrom(const SocketOps& ops, int fd, TxMessage* m) {
  const ssize_t n = ops.sendmsg(fd, &m->msg, MSG_ZEROCOPY | MSG_DONTWAIT | MSG_NOSIGNAL);
  if (n < 0) return (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) ? -EAGAIN : -(ssize_t)(errno ? errno : EIO);
  return n;
}

bool parseZerocopyNotice(const struct msghdr* msg, uint32_t* lo, uint32_t* hi) {
  for (struct cmsghdr* cm = CMSG_FIRSTHDR(const_cast<struct msghdr*>(msg)); cm != nullptr;
       cm = CMSG_NXTHDR(const_cast<struct msghdr*>(msg), cm)) {
    if (!((cm->cmsg_level == SOL_IP && cm->cmsg_type == IP_RECVERR) || (cm->cmsg_level == SOL_IPV6 && cm->cmsg_type == IPV6_RECVERR)))
      continue;
    if (cm->cmsg_len < CMSG_LEN(sizeof(struct sock_extended_err))) continue;
    struct sock_extended_err ee;
    memcpy(&ee, CMSG_DATA(cm), sizeof ee);
    if (ee.ee_errno != 0 || ee.ee_origin != SO_EE_ORIGIN_ZEROCOPY) continue;
    *lo = ee.ee_info;
    *hi = ee.ee_data + 1;  // the kernel reports an inclusive range
    return true;
  }
  return false;
}

void TxCompletions::onNotice(uint32_t lo, uint32_t hi) {
  if (lo == hi) return;
  pending_.push_back({lo, hi});
  // advance over every range that starts at or before the frontier (wrap-safe compares)
  bool moved = true;
  while (moved) {
    moved = false;
    for (size_t i = 0; i < pending_.size(); ++i) {
      const uint32_t a = pending_[i].first, b = pending_[i].second;
      if ((int32_t)(a - done_) <= 0) {            // starts at or behind the frontier
        if ((int32_t)(b - done_) > 0) done_ = b;  // and reaches past it
        pending_.erase(pending_.begin() + (long)i);
        moved = true;
        break;
      }
    }
  }
}

}  // namespace devmem
}  // namespace tcpxb
