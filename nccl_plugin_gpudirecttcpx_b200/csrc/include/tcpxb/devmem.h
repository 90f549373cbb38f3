// devmem-TCP datapath on the upstream Linux API (receive since Linux 6.12, transmit
// since 6.16): the NIC writes payload straight into a dma-buf (the GPU rx pool) and
// reads transmit payload straight out of one, and the socket calls carry only
// descriptions of where the bytes are.
//
// Counterpart of the reference's socket datapath (reference: src/sock/tcpx.h:48-90
// zero-copy send with a dma-buf control message, :92-127 completion notices from the
// error queue, :130-228 walk over the fragment control messages of a receive,
// :299-326 hand-back of page tokens).  The reference is written against Google's
// pre-upstream kernel interface (SO_DEVMEM_* 97..99, a 12-byte fragment record); this
// file speaks the interface that was merged upstream:
//
//   receive   recvmsg(fd, msg, MSG_SOCK_DEVMEM); every fragment arrives as a control
//             message SOL_SOCKET / SCM_DEVMEM_DMABUF holding a `DmabufCmsg`; payload the
//             kernel had to put in host memory arrives as SCM_DEVMEM_LINEAR;
//   recycle   setsockopt(fd, SOL_SOCKET, SO_DEVMEM_DONTNEED, DmabufToken[], bytes);
//   transmit  sendmsg(fd, msg, MSG_ZEROCOPY) with a control message SCM_DEVMEM_DMABUF
//             holding the u32 id of a dma-buf bound for transmit; iov_base is the offset
//             inside that dma-buf; completion notices as for MSG_ZEROCOPY.
//
// What this file holds is the part that needs no NIC: the control-message walk that
// turns fragments into scatter-list records and token runs, the batched hand-back,
// the transmit message builder and the completion accounting.  The system calls go
// through a small table (`SocketOps`) so that tests can put a model of the kernel
// behind them; on a host with a devmem-capable NIC the default table is the real
// calls.  Binding the pool to NIC queues and steering flows to them is the buffer
// manager daemon's job (netlink, privileged) and is not done here.
#ifndef TCPXB_DEVMEM_H_
#define TCPXB_DEVMEM_H_

#include <stddef.h>
#include <stdint.h>
#include <sys/socket.h>
#include <sys/uio.h>

#include <vector>

#include "tcpxb/base.h"
#include "tcpxb/dev_queue.h"

namespace tcpxb {
namespace devmem {

// ---- kernel interface (include/uapi/linux/uio.h, asm-generic/socket.h) --------------
constexpr int kMsgSockDevmem = 0x2000000;  // MSG_SOCK_DEVMEM
constexpr int kSoDevmemLinear = 78;        // SO_DEVMEM_LINEAR  == SCM_DEVMEM_LINEAR
constexpr int kSoDevmemDmabuf = 79;        // SO_DEVMEM_DMABUF  == SCM_DEVMEM_DMABUF
constexpr int kSoDevmemDontneed = 80;      // SO_DEVMEM_DONTNEED
struct DmabufCmsg {
  uint64_t frag_offset;  // offset of the fragment inside the dma-buf
  uint32_t frag_size;
  uint32_t frag_token;   // to be given back with SO_DEVMEM_DONTNEED
  uint32_t dmabuf_id;
  uint32_t flags;
};
struct DmabufToken {
  uint32_t token_start;
  uint32_t token_count;
};
static_assert(sizeof(DmabufCmsg) == 24 && sizeof(DmabufToken) == 8, "kernel ABI");
// The kernel frees at most this many token runs per SO_DEVMEM_DONTNEED call.
constexpr size_t kMaxDontneedRuns = 128;

// ---- system-call seam -----------------------------------------------------------------
struct SocketOps {
  ssize_t (*recvmsg)(int fd, struct msghdr* msg, int flags);
  ssize_t (*sendmsg)(int fd, const struct msghdr* msg, int flags);
  int (*setsockopt)(int fd, int level, int optname, const void* val, socklen_t len);
};
// The real calls.
const SocketOps& systemOps();
// The table the transport's devmem datapath uses: the real calls unless a test put a
// model of the kernel in their place (null restores the real calls).
const SocketOps& activeOps();
void setOpsForTests(const SocketOps* ops);

// ---- receive ----------------------------------------------------------------------------
// Where the fragments of a message go.
struct RxSink {
  LoadMeta* records = nullptr;   // scatter-list slot (or a task's private list)
  uint64_t capacity = 0;         // records the list can hold
  uint64_t filled = 0;           // records written so far (updated)
  std::vector<DmabufToken>* tokens = nullptr;  // runs to hand back once the consumer is done (appended, coalesced)
  uint64_t pool_bytes = 0;       // size of the bound dma-buf; record offsets are 32-bit, so <= 4 GiB
  uint32_t dmabuf_id = 0;        // expected dma-buf; 0 = accept any
  uint32_t max_fragment = kUnpackPageBytes;  // longer fragments are cut into records of this size
};
// Control-buffer bytes needed for a receive of up to `fragments` fragments.
size_t rxControlBytes(size_t fragments);
// Walks the control messages of one recvmsg(MSG_SOCK_DEVMEM) that returned `returned`
// bytes and appends one record per fragment (dst_off counting up from `dst_offset`).
// Fails, consuming nothing further, when: the control buffer was truncated; payload
// arrived in host memory (a linear fragment: the flow is not steered to a devmem
// queue); a fragment lies outside the pool or in another dma-buf; the list is full;
// or the fragments do not add up to `returned`.  Tokens seen before a failure are
// still recorded, so that they can be handed back.
Result parseRecv(const struct msghdr* msg, ssize_t returned, uint64_t dst_offset, RxSink* sink);
// recvmsg + parse.  Returns bytes received (> 0), 0 when the peer closed, -EAGAIN when
// the socket would block, another negative errno on socket errors, and -EPROTO when
// the control messages were unusable (details logged).
ssize_t recvInto(const SocketOps& ops, int fd, size_t want, void* control, size_t control_bytes,
                 uint64_t dst_offset, RxSink* sink);
// Hands token runs back to the kernel in batches of kMaxDontneedRuns.  *calls (optional)
// counts system calls.  The list is cleared on success.
Result recycle(const SocketOps& ops, int fd, std::vector<DmabufToken>* runs, size_t* calls = nullptr);

// ---- transmit ---------------------------------------------------------------------------
struct TxMessage {
  struct msghdr msg;
  struct iovec iov;
  alignas(struct cmsghdr) char control[CMSG_SPACE(sizeof(uint32_t))];
};
// One zero-copy send of [offset, offset + len) of the transmit-bound dma-buf `dmabuf_id`.
void buildSend(TxMessage* m, uint32_t dmabuf_id, uint64_t offset, size_t len);
// sendmsg(MSG_ZEROCOPY | MSG_DONTWAIT | MSG_NOSIGNAL); same return convention as recvInto.
ssize_t sendFrom(const SocketOps& ops, int fd, TxMessage* m);

// One notice from the socket's error queue: the sendmsg calls [lo, hi) completed
// (sequence numbers count zero-copy sendmsg calls per socket and wrap at 2^32).
// Returns false when `msg` holds no zero-copy notice.
bool parseZerocopyNotice(const struct msghdr* msg, uint32_t* lo, uint32_t* hi);

// Which zero-copy sends of a socket have completed.  Notices may arrive out of order
// and may overlap; a send is complete when every send before it is.
class TxCompletions {
 public:
  explicit TxCompletions(uint32_t first_id = 0) : next_(first_id), done_(first_id) {}
  uint32_t onSend() { return next_++; }            // id of the sendmsg call just made
  void onNotice(uint32_t lo, uint32_t hi);         // ids [lo, hi) completed
  uint32_t outstanding() const { return next_ - done_; }
  // True when ids [first, first + count) have all completed (wrap-safe).
  bool completed(uint32_t first, uint32_t count) const { return (int32_t)(done_ - (first + count)) >= 0; }
  uint32_t done() const { return done_; }
 private:
  uint32_t next_, done_;
  std::vector<std::pair<uint32_t, uint32_t>> pending_;  // completed ranges ahead of done_
};

}  // namespace devmem
}  // namespace tcpxb
#endif  // TCPXB_DEVMEM_H_
