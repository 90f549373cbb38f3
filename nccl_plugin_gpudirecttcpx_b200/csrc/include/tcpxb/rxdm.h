// Client side of the receive-datapath manager ("RxDM") protocol and the framing
// both ends share.
//
// The reference talks to an external daemon over AF_UNIX stream sockets, one
// socket per service under a prefix directory, with u16 length-prefixed messages
// and file descriptors passed as SCM_RIGHTS (reference:
// src/rx_buf_mgr_client/unix_socket_connection.cc:47-177 framing and fd passing,
// rx_rule_client.cc:38-110 flow-steering rules, application_registry_client.cc:28-73
// lifecycle registration, src/gpu/rx_pool.cu:62-124 pool fd + {size, align}).
// The same services exist here, served by the small daemon in tools/rxdm.cc; the
// message bodies are fixed binary structs instead of protobuf.  Service sockets:
//   <prefix>/rx_rule_manager, <prefix>/rx_rule_uninstall,
//   <prefix>/get_gpu_fd, <prefix>/get_gpu_metadata (the request names the GPU; the
//   reference has one socket per PCI address), <prefix>/rxdm_application_registry,
//   <prefix>/rxdm_status
// Without a daemon the in-process emulator (rx_buf_mgr.h) provides the same calls.
#ifndef TCPXB_RXDM_H_
#define TCPXB_RXDM_H_

#include <stdint.h>

#include <string>

#include "tcpxb/base.h"
#include "tcpxb/socket_utils.h"

namespace tcpxb {

constexpr uint32_t kRxdmMagic = 0x4d445852;  // "RXDM"
enum RxdmType : uint16_t {
  kRxdmFlowRule = 1,
  kRxdmFlowRuleUninstall = 2,
  kRxdmGetGpuFd = 3,
  kRxdmGetGpuMetadata = 4,
  kRxdmAppRegister = 5,
  kRxdmStatus = 6,
  kRxdmReply = 0x8000,
};

// What a pool descriptor stands for: a memfd of host memory (map it, register it with
// CUDA) or a shareable handle of device memory (import and map it through the driver).
enum RxdmPoolKind : int { kRxdmPoolHost = 0, kRxdmPoolDevice = 1 };

struct RxdmFlowRule {
  char src_ip[46];
  uint16_t src_port;
  char dst_ip[46];
  uint16_t dst_port;
  int32_t flow_type;   // 1 = TCP over IPv4, 2 = TCP over IPv6
  int32_t queue_id;    // -1: the daemon picks the queue
  char gpu_pci[32];
};
struct RxdmGpuQuery { char gpu_pci[32]; };
struct RxdmAppRegister { int32_t register_client; int32_t pid; };

struct RxdmMessage {
  uint32_t magic;
  uint16_t type;
  uint16_t reserved;
  union {
    RxdmFlowRule rule;
    RxdmGpuQuery gpu;
    RxdmAppRegister app;
    struct {
      int32_t status;     // 0 = ok
      char text[64];      // "Ok." on success, like the reference's raw reply
      uint64_t a, b;      // metadata: size, alignment; status: rules, apps
      uint64_t c;         // metadata: RxdmPoolKind; status: pools
    } reply;
  };
};

// One connected AF_UNIX stream socket with the framing above.
class UnixSocketConnection {
 public:
  UnixSocketConnection() = default;
  explicit UnixSocketConnection(int fd) : fd_(fd) {}
  ~UnixSocketConnection();
  UnixSocketConnection(const UnixSocketConnection&) = delete;
  UnixSocketConnection& operator=(const UnixSocketConnection&) = delete;
  Result connectTo(const std::string& path, int timeout_ms = 2000);
  Result send(const RxdmMessage& m, int fd_to_pass = -1);
  // Receives one message; *fd_out gets a passed descriptor or -1.
  Result recv(RxdmMessage* m, int* fd_out, int timeout_ms = 2000);
  int fd() const { return fd_; }
  int release() { int f = fd_; fd_ = -1; return f; }
  void closeNow();

 private:
  int fd_ = -1;
};

// One request/reply exchange with service `name` under `prefix`.
Result rxdmCall(const std::string& prefix, const std::string& name, const RxdmMessage& request,
                RxdmMessage* reply, int* fd_out);

RxdmMessage rxdmMakeRule(uint16_t type, const SocketAddress& local, const SocketAddress& peer,
                         const std::string& gpu_pci);

}  // namespace tcpxb
#endif  // TCPXB_RXDM_H_
