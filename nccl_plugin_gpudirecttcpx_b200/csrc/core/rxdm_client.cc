#include "tcpxb/rxdm.h"

#include <arpa/inet.h>
#include <poll.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace tcpxb {

UnixSocketConnection::~UnixSocketConnection() { closeNow(); }

void UnixSocketConnection::closeNow() {
  if (fd_ >= 0) close(fd_);
  fd_ = -1;
}

Result UnixSocketConnection::connectTo(const std::string& path, int timeout_ms) {
  closeNow();
  struct sockaddr_un addr;
  memset(&addr, 0, sizeof addr);
  addr.sun_family = AF_UNIX;
  if (path.size() >= sizeof addr.sun_path) return kInvalidArgument;
  memcpy(addr.sun_path, path.c_str(), path.size());
  const uint64_t tries = timeout_ms > 0 ? (uint64_t)timeout_ms / 10 + 1 : 1;
  for (uint64_t i = 0; i < tries; ++i) {
    int fd = socket(AF_UNIX, SOCK_STREAM, 0);
    if (fd < 0) return kSystemError;
    if (connect(fd, (struct sockaddr*)&addr, sizeof addr) == 0) {
      fd_ = fd;
      return kSuccess;
    }
    close(fd);
    if (errno != ENOENT && errno != ECONNREFUSED) break;
    usleep(10000);  // the daemon may still be starting
  }
  return kSystemError;
}

Result UnixSocketConnection::send(const RxdmMessage& m, int fd_to_pass) {
  if (fd_ < 0) return kInvalidUsage;
  const uint16_t len = htons((uint16_t)sizeof m);
  char frame[2 + sizeof m];
  memcpy(frame, &len, 2);
  memcpy(frame + 2, &m, sizeof m);
  struct iovec iov = {frame, sizeof frame};
  struct msghdr msg;
  memset(&msg, 0, sizeof msg);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  char control[CMSG_SPACE(sizeof(int))];
  if (fd_to_pass >= 0) {
    memset(control, 0, sizeof control);
    msg.msg_control = control;
    msg.msg_controllen = sizeof control;
    struct cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = SCM_RIGHTS;
    cm->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(cm), &fd_to_pass, sizeof(int));
  }
  ssize_t n = sendmsg(fd_, &msg, MSG_NOSIGNAL);
  return n == (ssize_t)sizeof frame ? kSuccess : kSystemError;
}

Result UnixSocketConnection::recv(RxdmMessage* m, int* fd_out, int timeout_ms) {
  if (fd_out != nullptr) *fd_out = -1;
  if (fd_ < 0) return kInvalidUsage;
  char frame[2 + sizeof *m];
  size_t got = 0;
  while (got < sizeof frame) {
    struct pollfd pfd = {fd_, POLLIN, 0};
    int pr = poll(&pfd, 1, timeout_ms);
    if (pr == 0) return kInProgress;
    if (pr < 0) { if (errno == EINTR) continue; return kSystemError; }
    struct iovec iov = {frame + got, sizeof frame - got};
    struct msghdr msg;
    memset(&msg, 0, sizeof msg);
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char control[CMSG_SPACE(sizeof(int))];
    msg.msg_control = control;
    msg.msg_controllen = sizeof control;
    ssize_t n = recvmsg(fd_, &msg, 0);
    if (n == 0) return kRemoteError;
    if (n < 0) { if (errno == EINTR) continue; return kSystemError; }
    got += (size_t)n;
    for (struct cmsghdr* cm = CMSG_FIRSTHDR(&msg); cm != nullptr; cm = CMSG_NXTHDR(&msg, cm)) {
      if (cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS && fd_out != nullptr)
        memcpy(fd_out, CMSG_DATA(cm), sizeof(int));
    }
  }
  uint16_t len;
  memcpy(&len, frame, 2);
  if (ntohs(len) != sizeof *m) return kRemoteError;
  memcpy(m, frame + 2, sizeof *m);
  return m->magic == kRxdmMagic ? kSuccess : kRemoteError;
}

Result rxdmCall(const std::string& prefix, const std::string& name, const RxdmMessage& request,
                RxdmMessage* reply, int* fd_out) {
  UnixSocketConnection c;
  Result r = c.connectTo(prefix + "/" + name);
  if (r != kSuccess) {
    WARN("rx buffer manager service %s/%s is not reachable", prefix.c_str(), name.c_str());
    return r;
  }
  TCPXB_CHECK(c.send(request));
  r = c.recv(reply, fd_out);
  if (r != kSuccess) return r == kInProgress ? kRemoteError : r;
  if (reply->reply.status != 0) {
    WARN("rx buffer manager refused %s: %s", name.c_str(), reply->reply.text);
    return kRemoteError;
  }
  return kSuccess;
}

RxdmMessage rxdmMakeRule(uint16_t type, const SocketAddress& local, const SocketAddress& peer,
                         const std::string& gpu_pci) {
  RxdmMessage m;
  memset(&m, 0, sizeof m);
  m.magic = kRxdmMagic;
  m.type = type;
  // the rule steers what the peer sends us: source = peer, destination = local
  snprintf(m.rule.src_ip, sizeof m.rule.src_ip, "%s", addressToString(peer, false).c_str());
  m.rule.src_port = (uint16_t)addressPort(peer);
  snprintf(m.rule.dst_ip, sizeof m.rule.dst_ip, "%s", addressToString(local, false).c_str());
  m.rule.dst_port = (uint16_t)addressPort(local);
  m.rule.flow_type = local.sa.sa_family == AF_INET6 ? 2 : 1;
  m.rule.queue_id = -1;
  snprintf(m.rule.gpu_pci, sizeof m.rule.gpu_pci, "%s", gpu_pci.c_str());
  return m;
}

}  // namespace tcpxb
