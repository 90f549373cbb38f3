// TCP socket helpers and interface discovery.
//
// Covers what the reference keeps in src/misc/socket_utils.{h,cc}: progress / spin /
// blocking send-recv loops (socket_utils.cc:34-67), interface enumeration with
// NCCL's prefix-list syntax ("eth", "^docker,lo", "=eth0", "name:port";
// socket_utils.cc:250-314, 528-576), listen / connect with bounded retries
// (:578-702) and the "local->peer" flow string (:222-241).  New here: one physical
// interface can be presented as several devices ("virtual NICs"), which is how a
// single box with only `lo` gets the multi-NIC layout the transport stripes over.
#ifndef TCPXB_SOCKET_UTILS_H_
#define TCPXB_SOCKET_UTILS_H_

#include <netinet/in.h>
#include <stddef.h>
#include <sys/socket.h>

#include <string>
#include <vector>

#include "tcpxb/base.h"

namespace tcpxb {

constexpr int kMaxIfs = 16;
constexpr int kMaxIfNameSize = 16;
constexpr int kListenBacklog = 16384;
constexpr int kRetryRefused = 20000;   // x 1 ms
constexpr int kRetryTimedOut = 3;

union SocketAddress {
  struct sockaddr sa;
  struct sockaddr_in sin;
  struct sockaddr_in6 sin6;
};
socklen_t addressLength(const SocketAddress& a);
std::string addressToString(const SocketAddress& a, bool with_port = true);
int addressPort(const SocketAddress& a);
void setAddressPort(SocketAddress* a, int port);

enum SockOp { kSockSend = 0, kSockRecv = 1 };

// One non-blocking attempt.  Advances *offset.  kSuccess also when nothing moved;
// kRemoteError when the peer closed; kSystemError on any other errno.
Result socketProgress(SockOp op, int fd, void* ptr, int size, int* offset, int extra_flags = 0);
// Repeats until all `size` bytes moved (busy loop on EAGAIN).
Result socketSpin(SockOp op, int fd, void* ptr, int size, int* offset);
// Blocking-style helpers over a possibly non-blocking fd (poll between attempts);
// `timeout_ms` < 0 waits forever.
Result socketSend(int fd, const void* ptr, int size, int timeout_ms = -1);
Result socketRecv(int fd, void* ptr, int size, int timeout_ms = -1);

struct NetIf {
  char name[kMaxIfNameSize + 8];
  SocketAddress addr;
  bool loopback;
};

// One entry of a prefix list: "eth" (prefix), "=eth0" (exact), optional ":port".
struct IfSpec { std::string prefix; int port; };
struct IfList { bool exclude = false; bool exact = false; std::vector<IfSpec> specs; };
IfList parseIfList(const char* s);
bool matchIfList(const IfList& l, const char* name, int port = -1);

// Enumerates usable interfaces.  `prefix_list` empty selects automatically: "ib*",
// then the subnet of `comm_id_hint`, then anything but docker/lo, then docker, then lo.
// `family` is AF_UNSPEC, AF_INET or AF_INET6.  Result is sorted by name.
std::vector<NetIf> findInterfaces(const char* prefix_list, int family, const char* comm_id_hint,
                                  int max_ifs = kMaxIfs);
// Presents `n` devices on interface `base`: on an IPv4 loopback they get addresses
// 127.0.0.(k+1), elsewhere they share the address.  Names become "<if>#k".
std::vector<NetIf> expandVirtual(const NetIf& base, int n);

int envSocketFamily(const std::string& value);  // "AF_INET" / "AF_INET6" / other -> AF_UNSPEC

Result createListenSocket(int* fd, SocketAddress* local /* in: address, out: bound port */);
// Binds to `local` (port 0) when given, sets TCP_NODELAY, connects with the retry
// policy above, leaves the socket non-blocking.
Result connectAddress(int* fd, const SocketAddress& remote, const SocketAddress* local);
Result acceptSocket(int listen_fd, int* fd, int timeout_ms);
Result setNonBlocking(int fd, bool on);
void setNoDelay(int fd);
void setQuickAck(int fd);
// "127.0.0.1<4242>->127.0.0.2<5151> tx"
std::string flowString(int fd, bool passive);
// Mb/s from /sys/class/net/<if>/speed, or 0 when unreadable / non-positive.
int interfaceSpeedMbps(const char* ifname);

}  // namespace tcpxb
#endif  // TCPXB_SOCKET_UTILS_H_
