#include "tcpxb/rxdm_proto.h"

#include <arpa/inet.h>
#include <errno.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace tcpxb {
namespace rxproto {

namespace {

// ---- protobuf wire primitives: varints, and fields of wire type 0 (varint) and 2 (bytes)
void putVarint(std::string* out, uint64_t v) {
  while (v >= 0x80) { out->push_back((char)(v | 0x80)); v >>= 7; }
  out->push_back((char)v);
}
void putTag(std::string* out, int field, int wire) { putVarint(out, (uint64_t)field << 3 | (uint64_t)wire); }
void putInt32(std::string* out, int field, int32_t v) {
  putTag(out, field, 0);
  putVarint(out, (uint64_t)(int64_t)v);  // negative int32 travels sign-extended to 64 bits
}
void putBytes(std::string* out, int field, const std::string& b) {
  putTag(out, field, 2);
  putVarint(out, b.size());
  out->append(b);
}

struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool varint(uint64_t* v) {
    uint64_t r = 0;
    for (int shift = 0; shift < 64 && p < end; shift += 7) {
      const uint8_t b = *p++;
      r |= (uint64_t)(b & 0x7f) << shift;
      if (!(b & 0x80)) { *v = r; return true; }
    }
    return false;
  }
  bool bytes(std::string* s) {
    uint64_t n;
    if (!varint(&n) || n > (uint64_t)(end - p)) return false;
    s->assign(reinterpret_cast<const char*>(p), (size_t)n);
    p += n;
    return true;
  }
  bool skip(int wire) {
    uint64_t v;
    std::string s;
    switch (wire) {
      case 0: return varint(&v);
      case 1: if (end - p < 8) return false; p += 8; return true;
      case 2: return bytes(&s);
      case 5: if (end - p < 4) return false; p += 4; return true;
      default: return false;
    }
  }
};

std::string encodeAddr(const SocketAddr& a) {
  std::string s;
  putBytes(&s, 1, a.ip);
  putInt32(&s, 2, a.port);
  return s;
}
bool decodeAddr(const std::string& raw, SocketAddr* a) {
  Reader r{reinterpret_cast<const uint8_t*>(raw.data()), reinterpret_cast<const uint8_t*>(raw.data()) + raw.size()};
  a->present = true;
  while (r.p < r.end) {
    uint64_t tag, v;
    if (!r.varint(&tag)) return false;
    const int field = (int)(tag >> 3), wire = (int)(tag & 7);
    if (field == 1 && wire == 2) { if (!r.bytes(&a->ip)) return false; }
    else if (field == 2 && wire == 0) { if (!r.varint(&v)) return false; a->port = (int32_t)v; }
    else if (!r.skip(wire)) return false;
  }
  return true;
}

bool decodeNtuple(const std::string& raw, Message* m) {
  Reader r{reinterpret_cast<const uint8_t*>(raw.data()), reinterpret_cast<const uint8_t*>(raw.data()) + raw.size()};
  m->has_ntuple = true;
  while (r.p < r.end) {
    uint64_t tag, v;
    std::string sub;
    if (!r.varint(&tag)) return false;
    const int field = (int)(tag >> 3), wire = (int)(tag & 7);
    if (field == 1 && wire == 0) { if (!r.varint(&v)) return false; m->flow_type = (int32_t)v; }
    else if (field == 2 && wire == 2) { if (!r.bytes(&sub) || !decodeAddr(sub, &m->src)) return false; }
    else if (field == 3 && wire == 2) { if (!r.bytes(&sub) || !decodeAddr(sub, &m->dst)) return false; }
    else if (!r.skip(wire)) return false;
  }
  return true;
}

bool decodeRule(const std::string& raw, Message* m) {
  Reader r{reinterpret_cast<const uint8_t*>(raw.data()), reinterpret_cast<const uint8_t*>(raw.data()) + raw.size()};
  while (r.p < r.end) {
    uint64_t tag, v;
    std::string sub;
    if (!r.varint(&tag)) return false;
    const int field = (int)(tag >> 3), wire = (int)(tag & 7);
    if (field == 1 && wire == 2) { if (!r.bytes(&sub) || !decodeNtuple(sub, m)) return false; }
    else if (field == 2 && wire == 0) { if (!r.varint(&v)) return false; m->queue_id = (int32_t)v; m->has_queue_id = true; }
    else if (field == 3 && wire == 2) { if (!r.bytes(&m->gpu_pci_addr)) return false; }
    else if (!r.skip(wire)) return false;
  }
  return true;
}

}  // namespace

std::string encode(const Message& m) {
  std::string out, sub;
  switch (m.kind) {
    case kRawBytes:
      putBytes(&out, 1, m.raw_bytes);
      break;
    case kFlowSteerRule: {
      if (m.has_ntuple) {
        std::string nt;
        putInt32(&nt, 1, m.flow_type);
        if (m.src.present) putBytes(&nt, 2, encodeAddr(m.src));
        if (m.dst.present) putBytes(&nt, 3, encodeAddr(m.dst));
        putBytes(&sub, 1, nt);
      }
      if (m.has_queue_id) putInt32(&sub, 2, m.queue_id);
      if (!m.gpu_pci_addr.empty()) putBytes(&sub, 3, m.gpu_pci_addr);
      putBytes(&out, 2, sub);
      break;
    }
    case kQueueIdQuery:
      putBytes(&sub, 1, m.gpu_pci_addr);
      putBytes(&out, 3, sub);
      break;
    case kQueueIdResponse:
      for (int32_t q : m.queue_ids) putInt32(&sub, 1, q);
      putBytes(&out, 4, sub);
      break;
    case kAppRegister:
      putTag(&sub, 1, 0);
      putVarint(&sub, m.register_client ? 1 : 0);
      putBytes(&out, 6, sub);
      break;
    case kNone:
      break;
  }
  return out;
}

bool decode(const void* data, size_t len, Message* out) {
  *out = Message();
  Reader r{static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + len};
  while (r.p < r.end) {
    uint64_t tag;
    if (!r.varint(&tag)) return false;
    const int field = (int)(tag >> 3), wire = (int)(tag & 7);
    std::string sub;
    if (wire != 2 || (field != 1 && field != 2 && field != 3 && field != 4 && field != 6)) {
      if (!r.skip(wire)) return false;
      continue;
    }
    if (!r.bytes(&sub)) return false;
    Reader s{reinterpret_cast<const uint8_t*>(sub.data()), reinterpret_cast<const uint8_t*>(sub.data()) + sub.size()};
    out->kind = (Kind)field;  // the last member of the oneof on the wire wins, as in protobuf
    switch (field) {
      case 1: out->raw_bytes = sub; break;
      case 2: if (!decodeRule(sub, out)) return false; break;
      case 3:
        while (s.p < s.end) {
          uint64_t t;
          if (!s.varint(&t)) return false;
          if ((t >> 3) == 1 && (t & 7) == 2) { if (!s.bytes(&out->gpu_pci_addr)) return false; }
          else if (!s.skip((int)(t & 7))) return false;
        }
        break;
      case 4:
        while (s.p < s.end) {
          uint64_t t, v;
          if (!s.varint(&t)) return false;
          if ((t >> 3) == 1 && (t & 7) == 0) { if (!s.varint(&v)) return false; out->queue_ids.push_back((int32_t)v); }
          else if ((t >> 3) == 1 && (t & 7) == 2) {  // packed encoding of the repeated field
            std::string packed;
            if (!s.bytes(&packed)) return false;
            Reader pr{reinterpret_cast<const uint8_t*>(packed.data()), reinterpret_cast<const uint8_t*>(packed.data()) + packed.size()};
            while (pr.p < pr.end) { if (!pr.varint(&v)) return false; out->queue_ids.push_back((int32_t)v); }
          } else if (!s.skip((int)(t & 7))) return false;
        }
        break;
      case 6:
        while (s.p < s.end) {
          uint64_t t, v;
          if (!s.varint(&t)) return false;
          if ((t >> 3) == 1 && (t & 7) == 0) { if (!s.varint(&v)) return false; out->register_client = v != 0; }
          else if (!s.skip((int)(t & 7))) return false;
        }
        break;
    }
  }
  return true;
}

// struct IpcGpuMemFdMetadata { int fd; size_t size; size_t align; } as laid out on x86-64
std::string encodeMetadata(const GpuMemMetadata& md) {
  char buf[24];
  memset(buf, 0, sizeof buf);
  memcpy(buf, &md.fd, 4);
  memcpy(buf + 8, &md.size, 8);
  memcpy(buf + 16, &md.align, 8);
  return std::string(buf, sizeof buf);
}
bool decodeMetadata(const std::string& raw, GpuMemMetadata* out) {
  if (raw.size() < 24) return false;
  memcpy(&out->fd, raw.data(), 4);
  memcpy(&out->size, raw.data() + 8, 8);
  memcpy(&out->align, raw.data() + 16, 8);
  return true;
}

// ---------------------------------------------------------------------- Connection
Connection::~Connection() { closeNow(); }
void Connection::closeNow() {
  if (fd_ >= 0) close(fd_);
  fd_ = -1;
}

Result Connection::connectTo(const std::string& path, int timeout_ms) {
  closeNow();
  struct sockaddr_un addr;
  memset(&addr, 0, sizeof addr);
  addr.sun_family = AF_UNIX;
  if (path.size() >= sizeof addr.sun_path) return kInvalidArgument;
  memcpy(addr.sun_path, path.c_str(), path.size());
  for (int waited = 0;; waited += 10) {
    int fd = socket(AF_UNIX, SOCK_STREAM, 0);
    if (fd < 0) return kSystemError;
    if (connect(fd, (struct sockaddr*)&addr, sizeof addr) == 0) { fd_ = fd; return kSuccess; }
    close(fd);
    if ((errno != ENOENT && errno != ECONNREFUSED) || waited >= timeout_ms) return kSystemError;
    usleep(10000);
  }
}

Result Connection::sendMessage(const Message& m) {
  if (fd_ < 0) return kInvalidUsage;
  const std::string body = encode(m);
  if (body.size() > 0xffff) return kInvalidArgument;
  std::string frame(2, '\0');
  const uint16_t len = htons((uint16_t)body.size());
  memcpy(&frame[0], &len, 2);
  frame += body;
  size_t off = 0;
  while (off < frame.size()) {
    ssize_t n = ::send(fd_, frame.data() + off, frame.size() - off, MSG_NOSIGNAL);
    if (n < 0) { if (errno == EINTR) continue; return kSystemError; }
    off += (size_t)n;
  }
  return kSuccess;
}

Result Connection::sendFd(int fd) {
  if (fd_ < 0 || fd < 0) return kInvalidUsage;
  char dummy = 0;
  struct iovec iov = {&dummy, 1};
  struct msghdr msg;
  memset(&msg, 0, sizeof msg);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  char control[CMSG_SPACE(sizeof(int))];
  memset(control, 0, sizeof control);
  msg.msg_control = control;
  msg.msg_controllen = sizeof control;
  struct cmsghdr* cm = CMSG_FIRSTHDR(&msg);
  cm->cmsg_level = SOL_SOCKET;
  cm->cmsg_type = SCM_RIGHTS;
  cm->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(cm), &fd, sizeof(int));
  return sendmsg(fd_, &msg, MSG_NOSIGNAL) == 1 ? kSuccess : kSystemError;
}

// Reads exactly `len` bytes unless a descriptor arrives first (then *fd_out is set and the
// dummy byte that carried it is dropped).
Result Connection::readExact(void* buf, size_t len, int timeout_ms, int* fd_out) {
  size_t got = 0;
  while (got < len) {
    struct pollfd pfd = {fd_, POLLIN, 0};
    int pr = poll(&pfd, 1, timeout_ms);
    if (pr == 0) return kInProgress;
    if (pr < 0) { if (errno == EINTR) continue; return kSystemError; }
    struct iovec iov = {static_cast<char*>(buf) + got, len - got};
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
    for (struct cmsghdr* cm = CMSG_FIRSTHDR(&msg); cm != nullptr; cm = CMSG_NXTHDR(&msg, cm)) {
      if (cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS && cm->cmsg_len == CMSG_LEN(sizeof(int))) {
        memcpy(fd_out, CMSG_DATA(cm), sizeof(int));
        return kSuccess;
      }
    }
    got += (size_t)n;
  }
  return kSuccess;
}

Result Connection::recv(Message* m, int* fd_out, int timeout_ms) {
  if (fd_ < 0 || fd_out == nullptr) return kInvalidUsage;
  *fd_out = -1;
  uint16_t len_be = 0;
  // a descriptor arrives with one dummy byte and no length prefix: read the first byte alone
  uint8_t first = 0;
  Result r = readExact(&first, 1, timeout_ms, fd_out);  // kInProgress = nothing arrived in time
  if (r != kSuccess || *fd_out >= 0) return r;
  uint8_t second = 0;
  int unexpected = -1;
  r = readExact(&second, 1, timeout_ms, &unexpected);
  if (r != kSuccess) return r == kInProgress ? kRemoteError : r;  // half a frame and then silence
  if (unexpected >= 0) { close(unexpected); return kRemoteError; }
  len_be = (uint16_t)(first | (uint16_t)second << 8);
  const size_t len = ntohs(len_be);
  std::string body(len, '\0');
  if (len > 0) {
    r = readExact(&body[0], len, timeout_ms, &unexpected);
    if (r != kSuccess) return r == kInProgress ? kRemoteError : r;
    if (unexpected >= 0) { close(unexpected); return kRemoteError; }
  }
  return decode(body.data(), body.size(), m) ? kSuccess : kRemoteError;
}

Result call(const std::string& prefix, const std::string& name, const Message& request, Message* reply, int* fd_out) {
  Connection c;
  Result r = c.connectTo(prefix + "/" + name);
  if (r != kSuccess) {
    WARN("rx buffer manager service %s/%s is not reachable", prefix.c_str(), name.c_str());
    return r;
  }
  TCPXB_CHECK(c.sendMessage(request));
  if (fd_out != nullptr) *fd_out = -1;
  Message scratch;
  int fd = -1;
  r = c.recv(reply != nullptr ? reply : &scratch, &fd);
  if (r != kSuccess) return r == kInProgress ? kRemoteError : r;
  if (fd >= 0) {
    if (fd_out != nullptr) *fd_out = fd;
    else close(fd);
  }
  return kSuccess;
}

Message makeRule(const SocketAddress& local, const SocketAddress& peer, const std::string& gpu_pci) {
  Message m;
  m.kind = kFlowSteerRule;
  m.has_ntuple = true;
  m.flow_type = local.sa.sa_family == AF_INET6 ? kFlowTcpV6 : kFlowTcpV4;
  m.src.present = m.dst.present = true;
  m.src.ip = addressToString(peer, false);
  m.src.port = addressPort(peer);
  m.dst.ip = addressToString(local, false);
  m.dst.port = addressPort(local);
  m.gpu_pci_addr = gpu_pci;
  return m;
}

}  // namespace rxproto
}  // namespace tcpxb
