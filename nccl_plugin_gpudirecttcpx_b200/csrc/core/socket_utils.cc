#include "tcpxb/socket_utils.h"

#include "tcpxb/flags.h"

#include <algorithm>
#include <arpa/inet.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netdb.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdio.h>
#include <stdlib.h>
#include <unistd.h>

namespace tcpxb {

socklen_t addressLength(const SocketAddress& a) {
  return a.sa.sa_family == AF_INET6 ? sizeof(struct sockaddr_in6) : sizeof(struct sockaddr_in);
}

int addressPort(const SocketAddress& a) {
  return ntohs(a.sa.sa_family == AF_INET6 ? a.sin6.sin6_port : a.sin.sin_port);
}

void setAddressPort(SocketAddress* a, int port) {
  if (a->sa.sa_family == AF_INET6) a->sin6.sin6_port = htons((uint16_t)port);
  else a->sin.sin_port = htons((uint16_t)port);
}

std::string addressToString(const SocketAddress& a, bool with_port) {
  char host[NI_MAXHOST] = "?";
  if (a.sa.sa_family == AF_INET) inet_ntop(AF_INET, &a.sin.sin_addr, host, sizeof host);
  else if (a.sa.sa_family == AF_INET6) inet_ntop(AF_INET6, &a.sin6.sin6_addr, host, sizeof host);
  std::string s(host);
  if (with_port) s += "<" + std::to_string(addressPort(a)) + ">";
  return s;
}

Result socketProgress(SockOp op, int fd, void* ptr, int size, int* offset, int extra_flags) {
  if (*offset >= size) return kSuccess;
  char* p = static_cast<char*>(ptr) + *offset;
  const int want = size - *offset;
  ssize_t n;
  if (op == kSockRecv) n = recv(fd, p, want, MSG_DONTWAIT | extra_flags);
  else n = send(fd, p, want, MSG_DONTWAIT | MSG_NOSIGNAL | extra_flags);
  if (n > 0) { *offset += (int)n; return kSuccess; }
  if (n == 0 && op == kSockRecv) return kRemoteError;  // orderly shutdown by the peer
  if (n == 0) return kSuccess;
  if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) return kSuccess;
  if (errno == ECONNRESET || errno == EPIPE) return kRemoteError;
  WARN("socket %s on fd %d failed: %s", op == kSockRecv ? "recv" : "send", fd, strerror(errno));
  return kSystemError;
}

Result socketSpin(SockOp op, int fd, void* ptr, int size, int* offset) {
  while (*offset < size) {
    Result r = socketProgress(op, fd, ptr, size, offset);
    if (r != kSuccess) return r;
  }
  return kSuccess;
}

namespace {
Result socketWait(SockOp op, int fd, void* ptr, int size, int timeout_ms) {
  int off = 0;
  while (off < size) {
    Result r = socketProgress(op, fd, ptr, size, &off);
    if (r != kSuccess) return r;
    if (off >= size) break;
    struct pollfd pfd = {fd, (short)(op == kSockRecv ? POLLIN : POLLOUT), 0};
    int pr = poll(&pfd, 1, timeout_ms < 0 ? 1000 : timeout_ms);
    if (pr == 0 && timeout_ms >= 0) return kInProgress;  // caller's deadline passed
    if (pr < 0 && errno != EINTR) return kSystemError;
  }
  return kSuccess;
}
}  // namespace

Result socketSend(int fd, const void* ptr, int size, int timeout_ms) {
  return socketWait(kSockSend, fd, const_cast<void*>(ptr), size, timeout_ms);
}
Result socketRecv(int fd, void* ptr, int size, int timeout_ms) {
  return socketWait(kSockRecv, fd, ptr, size, timeout_ms);
}

IfList parseIfList(const char* s) {
  IfList l;
  if (s == nullptr) return l;
  if (*s == '^') { l.exclude = true; ++s; }
  if (*s == '=') { l.exact = true; ++s; }
  std::string str(s);
  size_t pos = 0;
  while (pos <= str.size()) {
    size_t end = str.find(',', pos);
    if (end == std::string::npos) end = str.size();
    std::string tok = str.substr(pos, end - pos);
    pos = end + 1;
    if (tok.empty()) continue;
    IfSpec spec{tok, -1};
    size_t colon = tok.find(':');
    if (colon != std::string::npos) {
      spec.prefix = tok.substr(0, colon);
      spec.port = atoi(tok.c_str() + colon + 1);
    }
    if (!spec.prefix.empty()) l.specs.push_back(spec);
  }
  return l;
}

bool matchIfList(const IfList& l, const char* name, int port) {
  if (l.specs.empty()) return true;
  bool hit = false;
  for (const IfSpec& sp : l.specs) {
    bool name_ok = l.exact ? (sp.prefix == name) : (strncmp(name, sp.prefix.c_str(), sp.prefix.size()) == 0);
    bool port_ok = (sp.port == -1 || port == -1 || sp.port == port);
    if (name_ok && port_ok) { hit = true; break; }
  }
  return l.exclude ? !hit : hit;
}

int envSocketFamily(const std::string& v) {
  if (v == "AF_INET") return AF_INET;
  if (v == "AF_INET6") return AF_INET6;
  return AF_UNSPEC;
}

namespace {

bool sameSubnet(const struct ifaddrs* ifa, const SocketAddress& hint) {
  if (ifa->ifa_addr->sa_family != hint.sa.sa_family || ifa->ifa_netmask == nullptr) return false;
  if (hint.sa.sa_family == AF_INET) {
    uint32_t a = ((struct sockaddr_in*)ifa->ifa_addr)->sin_addr.s_addr;
    uint32_t m = ((struct sockaddr_in*)ifa->ifa_netmask)->sin_addr.s_addr;
    return ((a ^ hint.sin.sin_addr.s_addr) & m) == 0;
  }
  const uint8_t* a = ((struct sockaddr_in6*)ifa->ifa_addr)->sin6_addr.s6_addr;
  const uint8_t* m = ((struct sockaddr_in6*)ifa->ifa_netmask)->sin6_addr.s6_addr;
  const uint8_t* h = hint.sin6.sin6_addr.s6_addr;
  for (int i = 0; i < 16; ++i) if ((a[i] ^ h[i]) & m[i]) return false;
  return true;
}

bool parseHostPort(const char* s, SocketAddress* out) {
  // "a.b.c.d:port", "[v6]:port" or a bare address
  std::string str(s);
  std::string host = str;
  if (!str.empty() && str[0] == '[') {
    size_t rb = str.find(']');
    if (rb == std::string::npos) return false;
    host = str.substr(1, rb - 1);
  } else {
    size_t colon = str.rfind(':');
    if (colon != std::string::npos && str.find(':') == colon) host = str.substr(0, colon);
  }
  memset(out, 0, sizeof *out);
  if (inet_pton(AF_INET, host.c_str(), &out->sin.sin_addr) == 1) { out->sa.sa_family = AF_INET; return true; }
  if (inet_pton(AF_INET6, host.c_str(), &out->sin6.sin6_addr) == 1) { out->sa.sa_family = AF_INET6; return true; }
  return false;
}

enum class Pick { kList, kSubnet };

std::vector<NetIf> scan(const IfList& list, int family, const SocketAddress* subnet_hint, int max_ifs) {
  std::vector<NetIf> out;
  struct ifaddrs* all = nullptr;
  if (getifaddrs(&all) != 0) return out;
  for (struct ifaddrs* ifa = all; ifa != nullptr && (int)out.size() < max_ifs; ifa = ifa->ifa_next) {
    if (ifa->ifa_addr == nullptr) continue;
    const int fam = ifa->ifa_addr->sa_family;
    if (fam != AF_INET && fam != AF_INET6) continue;
    if (family != AF_UNSPEC && fam != family) continue;
    if (!(ifa->ifa_flags & IFF_UP)) continue;
    if (fam == AF_INET6) {
      // link-local v6 needs a scope id per socket; ::1 duplicates 127.0.0.1 unless v6 was asked for
      const struct sockaddr_in6* s6 = (const struct sockaddr_in6*)ifa->ifa_addr;
      if (IN6_IS_ADDR_LINKLOCAL(&s6->sin6_addr)) continue;
      if (IN6_IS_ADDR_LOOPBACK(&s6->sin6_addr) && family != AF_INET6) continue;
    }
    if (subnet_hint ? !sameSubnet(ifa, *subnet_hint) : !matchIfList(list, ifa->ifa_name)) continue;
    bool dup = false;
    for (const NetIf& n : out) if (!strcmp(n.name, ifa->ifa_name)) dup = true;
    if (dup) continue;
    NetIf n;
    memset(&n, 0, sizeof n);
    snprintf(n.name, sizeof n.name, "%.*s", kMaxIfNameSize - 1, ifa->ifa_name);
    memcpy(&n.addr, ifa->ifa_addr, fam == AF_INET ? sizeof(struct sockaddr_in) : sizeof(struct sockaddr_in6));
    n.loopback = (ifa->ifa_flags & IFF_LOOPBACK) != 0;
    out.push_back(n);
  }
  freeifaddrs(all);
  std::sort(out.begin(), out.end(), [](const NetIf& a, const NetIf& b) { return strcmp(a.name, b.name) < 0; });
  return out;
}

}  // namespace

std::vector<NetIf> findInterfaces(const char* prefix_list, int family, const char* comm_id_hint, int max_ifs) {
  if (prefix_list != nullptr && *prefix_list != 0) return scan(parseIfList(prefix_list), family, nullptr, max_ifs);
  std::vector<NetIf> r = scan(parseIfList("ib"), family, nullptr, max_ifs);
  if (!r.empty()) return r;
  if (comm_id_hint != nullptr && *comm_id_hint != 0) {
    SocketAddress hint;
    if (parseHostPort(comm_id_hint, &hint)) {
      r = scan(IfList(), family, &hint, max_ifs);
      if (!r.empty()) return r;
    }
  }
  r = scan(parseIfList("^docker,lo"), family, nullptr, max_ifs);
  if (!r.empty()) return r;
  r = scan(parseIfList("docker"), family, nullptr, max_ifs);
  if (!r.empty()) return r;
  return scan(parseIfList("lo"), family, nullptr, max_ifs);
}

std::vector<NetIf> expandVirtual(const NetIf& base, int n) {
  std::vector<NetIf> out;
  for (int k = 0; k < n; ++k) {
    NetIf v = base;
    snprintf(v.name, sizeof v.name, "%.*s#%d", kMaxIfNameSize - 1, base.name, k % 100);
    if (base.loopback && base.addr.sa.sa_family == AF_INET) {
      // every 127/8 address is local on lo, so each virtual NIC gets its own
      v.addr.sin.sin_addr.s_addr = htonl(0x7f000001u + (uint32_t)k);
    }
    out.push_back(v);
  }
  return out;
}

Result setNonBlocking(int fd, bool on) {
  int fl = fcntl(fd, F_GETFL, 0);
  if (fl < 0) return kSystemError;
  fl = on ? (fl | O_NONBLOCK) : (fl & ~O_NONBLOCK);
  return fcntl(fd, F_SETFL, fl) < 0 ? kSystemError : kSuccess;
}

void setNoDelay(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
}

void setQuickAck(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_QUICKACK, &one, sizeof one);
}

Result createListenSocket(int* fd_out, SocketAddress* local) {
  int fd = socket(local->sa.sa_family, SOCK_STREAM, 0);
  if (fd < 0) { WARN("socket() failed: %s", strerror(errno)); return kSystemError; }
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  if (bind(fd, &local->sa, addressLength(*local)) != 0) {
    WARN("bind(%s) failed: %s", addressToString(*local).c_str(), strerror(errno));
    close(fd);
    return kSystemError;
  }
  socklen_t len = addressLength(*local);
  if (getsockname(fd, &local->sa, &len) != 0 || listen(fd, kListenBacklog) != 0) {
    WARN("listen on %s failed: %s", addressToString(*local).c_str(), strerror(errno));
    close(fd);
    return kSystemError;
  }
  *fd_out = fd;
  return kSuccess;
}

Result connectAddress(int* fd_out, const SocketAddress& remote, const SocketAddress* local) {
  int refused = 0, timedout = 0;
  for (;;) {
    int fd = socket(remote.sa.sa_family, SOCK_STREAM, 0);
    if (fd < 0) { WARN("socket() failed: %s", strerror(errno)); return kSystemError; }
    if (local != nullptr && local->sa.sa_family == remote.sa.sa_family) {
      SocketAddress l = *local;
      setAddressPort(&l, 0);
      if (bind(fd, &l.sa, addressLength(l)) != 0)
        INFO(kSubNet, "bind(%s) before connect failed: %s", addressToString(l).c_str(), strerror(errno));
    }
    setNoDelay(fd);
    if (connect(fd, &remote.sa, addressLength(remote)) == 0) {
      setNonBlocking(fd, true);
      *fd_out = fd;
      return kSuccess;
    }
    const int err = errno;
    close(fd);
    if (err == ECONNREFUSED && ++refused < (int)flags().connect_refused_retries) { usleep(1000); continue; }
    if (err == ETIMEDOUT && ++timedout < kRetryTimedOut) continue;
    if (err == EINTR) continue;
    WARN("connect to %s failed: %s", addressToString(remote).c_str(), strerror(err));
    return kSystemError;
  }
}

Result acceptSocket(int listen_fd, int* fd_out, int timeout_ms) {
  for (;;) {
    struct pollfd pfd = {listen_fd, POLLIN, 0};
    int pr = poll(&pfd, 1, timeout_ms);
    if (pr == 0) return kInProgress;
    if (pr < 0) { if (errno == EINTR) continue; return kSystemError; }
    SocketAddress peer;
    socklen_t len = sizeof peer;
    int fd = accept(listen_fd, &peer.sa, &len);
    if (fd < 0) {
      if (errno == EINTR || errno == EAGAIN || errno == ECONNABORTED) continue;
      WARN("accept failed: %s", strerror(errno));
      return kSystemError;
    }
    setNonBlocking(fd, true);
    *fd_out = fd;
    return kSuccess;
  }
}

std::string flowString(int fd, bool passive) {
  SocketAddress l, p;
  socklen_t ll = sizeof l, pl = sizeof p;
  memset(&l, 0, sizeof l);
  memset(&p, 0, sizeof p);
  if (getsockname(fd, &l.sa, &ll) != 0 || getpeername(fd, &p.sa, &pl) != 0) return "unconnected";
  return addressToString(l) + "->" + addressToString(p) + (passive ? " rx" : " tx");
}

int interfaceSpeedMbps(const char* ifname) {
  std::string name(ifname);
  size_t hash = name.find('#');
  if (hash != std::string::npos) name.resize(hash);
  std::string path = "/sys/class/net/" + name + "/speed";
  FILE* f = fopen(path.c_str(), "r");
  if (f == nullptr) return 0;
  int v = 0;
  if (fscanf(f, "%d", &v) != 1) v = 0;
  fclose(f);
  return v > 0 ? v : 0;
}

}  // namespace tcpxb
