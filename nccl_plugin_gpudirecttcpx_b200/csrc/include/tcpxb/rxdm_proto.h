// The receive-datapath manager's protobuf wire format, written out by hand.
//
// Google's daemon and the reference's client exchange `UnixSocketProto` messages
// (proto2) framed by a 16-bit big-endian length, one request per connection, with file
// descriptors travelling as SCM_RIGHTS beside one dummy byte (reference:
// src/rx_buf_mgr_client/proto/unix_socket_proto.proto:17-70,
// unix_socket_connection.cc:47-177 framing, rx_rule_client.cc:38-75 rule request and
// the "Ok." reply, application_registry_client.cc:28-73, src/gpu/rx_pool.cu:62-124 pool
// descriptor and `{fd, size, align}` metadata from per-GPU sockets).  The handful of
// messages involved is small enough to encode and decode directly, which keeps the
// plugin free of a protobuf dependency and still lets it talk to that daemon:
//
//   UnixSocketProto.oneof { 1: bytes raw_bytes, 2: FlowSteerRuleRequest,
//                           3: QueueIdQuery, 4: QueueIdResponse, 6: ApplicationRegisterRequest }
//   FlowSteerRuleRequest  { 1: FlowSteerNtupleProto, 2: int32 queue_id, 3: string gpu_pci_addr }
//   FlowSteerNtupleProto  { 1: int32 flow_type, 2: SocketAddress src, 3: SocketAddress dst }
//   SocketAddress         { 1: string ip_address, 2: int32 port }
//   QueueIdQuery          { 1: string gpu_pci_addr }      QueueIdResponse { 1: repeated int32 queue_ids }
//   ApplicationRegisterRequest { 1: bool register_client }
//
// Selected with NCCL_GPUDIRECTTCPX_RXDM_WIRE=proto (client) and `tcpxb_rxdm --wire proto`
// (this repository's daemon, which then serves the per-GPU socket names too).
#ifndef TCPXB_RXDM_PROTO_H_
#define TCPXB_RXDM_PROTO_H_

#include <stddef.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "tcpxb/base.h"
#include "tcpxb/socket_utils.h"

namespace tcpxb {
namespace rxproto {

enum Kind { kNone = 0, kRawBytes = 1, kFlowSteerRule = 2, kQueueIdQuery = 3, kQueueIdResponse = 4, kAppRegister = 6 };

struct SocketAddr {
  std::string ip;  // presentation format
  int32_t port = 0;
  bool present = false;
};
struct Message {
  Kind kind = kNone;
  std::string raw_bytes;            // kRawBytes
  // kFlowSteerRule
  bool has_ntuple = false;
  int32_t flow_type = 0;            // ethtool's numbering: 1 = TCP_V4_FLOW, 5 = TCP_V6_FLOW
  SocketAddr src, dst;
  bool has_queue_id = false;
  int32_t queue_id = 0;
  std::string gpu_pci_addr;         // also kQueueIdQuery
  std::vector<int32_t> queue_ids;   // kQueueIdResponse
  bool register_client = false;     // kAppRegister
};

// Serialises `m` as a UnixSocketProto.
std::string encode(const Message& m);
// Parses a UnixSocketProto; unknown fields are skipped.  False on malformed input.
bool decode(const void* data, size_t len, Message* out);

// The pool metadata the daemon sends as raw bytes on get_gpu_metadata_<pci>.
struct GpuMemMetadata {
  int32_t fd = -1;
  uint64_t size = 0, align = 0;
};
std::string encodeMetadata(const GpuMemMetadata& md);   // the daemon's in-memory struct: int, padding, two size_t
bool decodeMetadata(const std::string& raw, GpuMemMetadata* out);

// One AF_UNIX stream connection with the framing above.
class Connection {
 public:
  Connection() = default;
  explicit Connection(int fd) : fd_(fd) {}
  ~Connection();
  Connection(const Connection&) = delete;
  Connection& operator=(const Connection&) = delete;
  Result connectTo(const std::string& path, int timeout_ms = 2000);
  Result sendMessage(const Message& m);
  Result sendFd(int fd);
  // Receives the next item: a message (*fd_out = -1) or a descriptor (*fd_out >= 0, *m untouched).
  Result recv(Message* m, int* fd_out, int timeout_ms = 2000);
  int fd() const { return fd_; }
  int release() { int f = fd_; fd_ = -1; return f; }
  void closeNow();

 private:
  Result readExact(void* buf, size_t len, int timeout_ms, int* fd_out);
  int fd_ = -1;
};

constexpr int32_t kFlowTcpV4 = 1, kFlowTcpV6 = 5;

// One request on a fresh connection to <prefix>/<name>, and the reply: a message, a
// descriptor (*fd_out, when the caller expects one) or both in either order.
Result call(const std::string& prefix, const std::string& name, const Message& request, Message* reply, int* fd_out);
// The rule that steers what `peer` sends to `local` (source = peer, destination = local).
Message makeRule(const SocketAddress& local, const SocketAddress& peer, const std::string& gpu_pci);

}  // namespace rxproto
}  // namespace tcpxb
#endif  // TCPXB_RXDM_PROTO_H_
