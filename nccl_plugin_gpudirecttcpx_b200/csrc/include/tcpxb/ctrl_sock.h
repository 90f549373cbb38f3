// Buffered ends of the control socket.
//
// The sender coalesces up to eight 16-byte control records into one send()
// (flushed explicitly), the receiver refills a buffer of the same size and hands
// out whole records; bytes already buffered can be drained raw, which is how an
// inline payload that follows a record is read (reference: src/ctrl_sock.h:20-76,
// buffer size src/common.h:195).
#ifndef TCPXB_CTRL_SOCK_H_
#define TCPXB_CTRL_SOCK_H_

#include <stdint.h>
#include <string.h>

#include "tcpxb/socket_utils.h"

namespace tcpxb {

// Control record, sender -> receiver (reference: src/common.h:127-133).
struct __attribute__((__packed__)) CtrlMsg {
  uint16_t type;    // CtrlType
  uint16_t index;   // data socket that carries the chunk
  uint32_t size;    // chunk bytes (inline: payload bytes)
  uint32_t offset;  // chunk offset in the message
  uint32_t total;   // message bytes
};
static_assert(sizeof(CtrlMsg) == 16, "wire format");
enum CtrlType : uint16_t { kCtrlNormal = 0, kCtrlInline = 1, kCtrlMaxType = 2 };
constexpr int kCtrlBufferBytes = 8 * sizeof(CtrlMsg);

class CtrlSendBuffer {
 public:
  void attach(int fd) { fd_ = fd; len_ = 0; sent_ = 0; }
  int fd() const { return fd_; }
  bool full() const { return len_ + (int)sizeof(CtrlMsg) > kCtrlBufferBytes; }
  bool pending() const { return sent_ < len_; }
  // Queues one record; flushes first when the buffer is full.  kInProgress means
  // the socket would block and the record was NOT queued.
  Result push(const CtrlMsg& m) {
    if (full()) {
      Result r = flush();
      if (r != kSuccess) return r;
    }
    memcpy(buf_ + len_, &m, sizeof m);
    len_ += sizeof m;
    return kSuccess;
  }
  // Tries to write everything queued.  kInProgress when bytes remain.
  Result flush() {
    if (sent_ < len_) {
      Result r = socketProgress(kSockSend, fd_, buf_, len_, &sent_);
      if (r != kSuccess) return r;
      if (sent_ < len_) return kInProgress;
    }
    len_ = sent_ = 0;
    return kSuccess;
  }

 private:
  int fd_ = -1;
  int len_ = 0, sent_ = 0;
  char buf_[kCtrlBufferBytes];
};

class CtrlRecvBuffer {
 public:
  void attach(int fd) { fd_ = fd; head_ = tail_ = 0; }
  int fd() const { return fd_; }
  int buffered() const { return tail_ - head_; }
  // One whole record if available (non-blocking).  kInProgress when not yet.
  Result pop(CtrlMsg* m) {
    if (buffered() < (int)sizeof(CtrlMsg)) {
      if (head_ > 0) {  // compact so a whole record always fits behind the data
        memmove(buf_, buf_ + head_, (size_t)buffered());
        tail_ -= head_;
        head_ = 0;
      }
      ssize_t n = recv(fd_, buf_ + tail_, (size_t)(kCtrlBufferBytes - tail_), MSG_DONTWAIT);
      if (n == 0) return kRemoteError;
      if (n < 0) {
        if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return kInProgress;
        return (errno == ECONNRESET) ? kRemoteError : kSystemError;
      }
      tail_ += (int)n;
      if (buffered() < (int)sizeof(CtrlMsg)) return kInProgress;
    }
    memcpy(m, buf_ + head_, sizeof *m);
    head_ += sizeof *m;
    return kSuccess;
  }
  // Copies out up to `size` already-buffered bytes; returns how many.
  int drain(void* dst, int size) {
    int n = buffered() < size ? buffered() : size;
    if (n > 0) { memcpy(dst, buf_ + head_, (size_t)n); head_ += n; }
    return n;
  }

 private:
  int fd_ = -1;
  int head_ = 0, tail_ = 0;
  char buf_[kCtrlBufferBytes];
};

}  // namespace tcpxb
#endif  // TCPXB_CTRL_SOCK_H_
