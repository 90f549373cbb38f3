// Core transport: communicators striped over several TCP sockets, the progress
// engine behind isend / irecv / test, helper threads, and the public C++ API the
// plugin table and the collective engine call.
//
// Functional counterpart of the reference's core (reference: src/net_tcpx.cc:454-1543,
// structures in src/common.h:42-219, connection layer src/connect.cc).  What is
// kept: the connect handle layout, the control-record wire format, the
// ctrl-first handshake, one request ring (16) per comm and one task ring (6) per
// socket, chunk striping by a flow mapper, in-order completion.  What differs:
// errors propagate to test() instead of exiting or hanging, helper threads block
// in poll() when every socket would block, test() writes the received size, CUDA
// buffers are served by staging plus the emulated rx page pool, and nothing
// sleeps during connection setup unless asked to.
//
// CUDA buffers and the caller's thread.  Under NCCL the data path runs on NCCL's
// proxy thread while a collective kernel waits for it.  A CUDA call made there
// (copy, launch, event) can block behind a synchronous call of the application,
// e.g. a pageable device-to-host copy waiting for that very collective: both then
// wait for each other.  So, as with the reference, the mode meant for NCCL is
// "unpack": payload lands in the mapped page pool, NCCL's kernel copies it out,
// and this library makes no CUDA call after set-up.  Host receive mode takes CUDA
// pointers only when NCCL_GPUDIRECTTCPX_CUDA_BUFFERS=1 (the collective engine
// uses it: there the caller's own thread drives everything).
#ifndef TCPXB_TRANSPORT_H_
#define TCPXB_TRANSPORT_H_

#include <sys/uio.h>

#include <atomic>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "tcpxb/base.h"
#include "tcpxb/ctrl_sock.h"
#include "tcpxb/dev_queue.h"
#include "tcpxb/devmem.h"
#include "tcpxb/flags.h"
#include "tcpxb/flow_mapper.h"
#include "tcpxb/gpu.h"
#include "tcpxb/rx_buf_mgr.h"
#include "tcpxb/socket_utils.h"
#include "tcpxb/stage_ring.h"
#include "tcpxb/telemetry.h"
#include "tcpxb/timeout.h"

namespace tcpxb {

constexpr int kPtrHost = 1, kPtrCuda = 2;
constexpr int kHandleMaxSize = 128;  // NCCL_NET_HANDLE_MAXSIZE
constexpr int kMaxInlineThreshold = 2048;
constexpr int kMaxTxSegments = 8;

// ---- devices ------------------------------------------------------------------
struct NetDevice {
  NetIf nif;
  std::string pci_path;  // realpath of /sys/class/net/<if>/device, "" for virtual ones
  int speed_mbps = 10000;
};

// Core ranges per NIC, "eth1:8-21,112-125;eth2:..." (reference: src/common.cc:65-123).
constexpr int kMaxRanges = 8;
struct CpuBindings {
  int n_ranges[kMaxIfs] = {};
  int lo[kMaxIfs][kMaxRanges] = {};
  int hi[kMaxIfs][kMaxRanges] = {};
};
// `if_names[i]` is the name of device i; entries naming unknown NICs are skipped.
bool parseCoreRanges(const char* text, const std::vector<std::string>& if_names, CpuBindings* out);

// ---- wire: connect handle (reference: src/common.h:101-110) ----------------------
struct Handle {
  SocketAddress connect_addr;
  int port_start, port_count;
  int num_socks;
  int num_threads;
  bool redirect_ctrl;
  SocketAddress ctrl_addr;
  void* connect_args;  // scratch of the connecting side, zero on the wire
};
static_assert(sizeof(Handle) <= kHandleMaxSize, "handle must fit NCCL's handle buffer");

std::string handleToString(const Handle& h);

enum ConnState : int { kConnOk = 0, kConnPending = 1, kConnFailed = 2 };

struct Comm;
struct Request;

struct MemHandle {
  void* ptr;
  size_t size;
  int type;     // kPtrHost / kPtrCuda
  int gpu_dev;  // owning GPU for CUDA memory, else -1
  // devmem datapath: the buffer exported as a dma-buf for zero-copy transmit
  // (reference: src/gpu/tx_pool.cu:104-181); -1 when not exported
  int dmabuf_fd = -1;
  uint64_t dmabuf_offset = 0;  // of `ptr` inside the exported range
  uint32_t dmabuf_id = 0;      // id the NIC binding gave the dma-buf (0 = not bound)
};

// ---- tasks: one chunk on one data socket ------------------------------------------
enum TaskStage { kTaskActive = 1, kTaskCompleting = 2, kTaskInactive = 3 };
struct Task {
  Request* r = nullptr;
  int op = 0;                 // SockOp
  uint8_t* host_ptr = nullptr;  // contiguous source / destination, or null when scattered
  int size = 0;
  int offset = 0;             // bytes moved so far
  int msg_offset = 0;         // chunk offset in the message
  // receive into pool pages
  std::vector<PageRun> pages;
  std::vector<struct iovec> iov;
  size_t iov_pos = 0;
  // zero-copy accounting: notification ids [zc_first, zc_first + zc_count)
  uint32_t zc_first = 0, zc_count = 0;
  bool zerocopy = false;
  // a send from the staging ring may be queued before the copy engine has filled it:
  // the helper starts once the counter has reached the mark (null = nothing to wait for)
  const gpu::StreamCounter* wait_counter = nullptr;
  uint32_t wait_mark = 0;
  // devmem datapath.  Receive: the kernel reports fragments, collected here until the
  // progress engine moves them into the request's scatter list.  Send: the payload is
  // read by the NIC from the dma-buf `dmabuf_id` at `dmabuf_off`.
  bool devmem = false;
  std::vector<LoadMeta> records;
  uint64_t records_filled = 0;
  std::vector<devmem::DmabufToken> tokens;
  uint32_t dmabuf_id = 0;
  uint64_t dmabuf_off = 0;
};

enum ReqStage { kReqPosted = 1, kReqActive = 2, kReqTransmitting = 3, kReqFinished = 4 };
struct Request {
  Comm* comm = nullptr;
  int op = 0;
  uint8_t* data = nullptr;
  int size = 0;             // send: message bytes; recv: buffer bytes, then message bytes
  int capacity = 0;         // recv: posted buffer bytes
  int tag = 0;
  int mem_type = kPtrHost;
  int gpu_dev = -1;
  int offset = 0;           // bytes scheduled into tasks
  int size_pending = 0;     // bytes not yet moved (-1: size still unknown)
  bool size_known = false;
  bool reported = false;    // test() returned done
  bool consumed = false;    // unpack mode: irecvConsumed arrived
  // CUDA send: staging
  uint8_t* stage = nullptr;
  uint64_t stage_bytes = 0;
  int seg_bytes = 0, n_segs = 0, segs_done = 0;
  uint32_t seg_mark[kMaxTxSegments] = {};  // value the comm's staging counter reaches when segment i is in host memory
  // CUDA receive
  UnpackSlot slot;
  std::vector<PageRun> pages;
  bool pages_promised = false;    // the pool promised every page this message needs
  uint32_t pages_reserved = 0;    // what is left of that promise
  // devmem datapath: page tokens to hand back per data socket once the consumer is done,
  // and the registration of a send buffer (its dma-buf)
  std::vector<devmem::DmabufToken> tokens[kMaxSockets];
  const MemHandle* mh = nullptr;
  bool unpack_launched = false;
  uint32_t unpack_mark = 0;       // value the comm's unpack counter reaches when this request's kernel (or placement) is done
  uint64_t posted_ns = 0, last_stall_report_ns = 0;
  // inline transfer progress
  int inline_off = 0;
  bool inline_queued = false;  // send: the inline record is in the control buffer
  // receive-sync word read from the control socket
  uint32_t sync_word = 0;
  int sync_got = 0;
};

using TaskRing = StageRing<Task, kMaxTasks, 3, true>;
using RequestRing = StageRing<Request, kMaxRequests, 4, false>;

struct SocketCtx {
  int fd = -1;
  TaskRing tasks;
  FlowStats stats;
  std::string flow;
  StallDetector stall;
  // zero-copy notification ids: [zc_done, zc_next) are outstanding
  uint32_t zc_next = 0, zc_done = 0;
  bool zerocopy_enabled = false;
  std::vector<char> devmem_control;  // control buffer of this socket's devmem receives
};

struct HelperThread {
  int id = 0;
  std::thread thread;
  std::mutex mu;
  std::condition_variable cv;
  std::atomic<uint32_t> kicks{0};
  std::atomic<bool> sleeping{false};  // blocked (or about to block) on `cv`: a kick must notify
  // where the thread waits: asleep with no task at all, and inside poll() because
  // every socket with a task would block (the peer or the kernel is the slower side)
  std::atomic<uint64_t> idle_ns{0}, blocked_ns{0};
  uint32_t seen = 0;
};

// Lets the thread that polls test() sleep between polls.  That thread arms the
// notifier, looks once more for work, and blocks on `event_fd` (an eventfd, usually
// inside ppoll together with the control sockets); a helper thread that finishes a
// task, or fails, disarms it and writes the eventfd.  Shared by any number of comms.
struct Notifier {
  int event_fd = -1;
  std::atomic<uint32_t> armed{0};
};

struct Comm {
  bool passive = false;  // receiving side
  std::atomic<int> conn_state{kConnPending};
  std::atomic<int> error{kSuccess};  // first fatal Result seen by any thread
  int dev = 0;
  int num_socks = 0, num_threads = 0;
  SocketCtx sock[kMaxSockets];
  int ctrl_fd = -1;
  std::string ctrl_flow;
  CtrlSendBuffer ctrl_send;
  CtrlRecvBuffer ctrl_recv;
  StallDetector ctrl_stall;
  FlowStats ctrl_stats;
  RequestRing rq;
  std::unique_ptr<FlowMapper> mapper;
  HelperThread helpers[kMaxThreads];
  std::atomic<bool> stop{false};
  bool threads_started = false;
  int rotate = 0;  // socket the reaping pass starts from
  // idle helper threads nap this long, this many times, before they sleep until woken (0 = sleep at once)
  std::atomic<int> helper_nap_us{0}, helper_nap_rounds{0};
  uint32_t kick_mask = 0;        // helpers that got new tasks in the current progress round
  Notifier* notifier = nullptr;  // owned by the caller of netSetNotifier
  // pending control record on the receive side
  bool have_ctrl = false;
  CtrlMsg ctrl;
  uint64_t ctrl_quiet_until_ns = 0;  // no control-socket read before this time (after an empty read)
  bool ctrl_hinted = false;          // the caller polls the control socket itself and calls netHintCtrlReadable
  bool ctrl_readable_hint = false;   // ... and said so since the last empty read
  // CUDA resources (lazy)
  int gpu_dev = -1;
  int recv_mode = kRecvModeHost;
  bool devmem = false;  // CUDA buffers travel by devmem-TCP sockets (no staging, no page allocator)
  gpu::Stream stream = nullptr;
  RxBufMgr* rxmgr = nullptr;
  std::unique_ptr<DevQueue> devq;
  uint8_t* tx_stage = nullptr;
  uint64_t tx_stage_bytes = 0, tx_head = 0, tx_tail = 0;  // ring offsets (monotonic)
  uint32_t* unpack_status_host = nullptr;
  uint32_t* unpack_status_dev = nullptr;
  gpu::Event send_dependency = nullptr;
  // stream-ordered completion counters in mapped host memory: staging copies (send
  // side) and unpack kernels / page placements (receive side) on `stream`
  gpu::StreamCounter stage_marks, unpack_marks;
  bool cuda_prepared = false;
  uint32_t api_calls = 0, done_calls = 0;  // for the first-calls INFO lines
  std::atomic<const char*> where{"idle"};  // last checkpoint the API thread passed (watchdog)
  std::atomic<uint64_t> where_ns{0};
  bool want_device_handle = false;
  uint32_t polls_not_driving = 0;  // test() calls since the progress engine last ran
  // telemetry
  std::unique_ptr<EventLog> events;
  std::unique_ptr<Exporter> exporter;
  uint64_t id = 0;
  uint32_t stride = 0;
  SocketAddress peer_addr;
};

struct ListenComm {
  int dev = 0;
  int data_fd = -1;
  int ctrl_fd = -1;
  int num_socks = 0, num_threads = 0;
  void* accept_state = nullptr;
};

// ---- public API --------------------------------------------------------------------
Result netInit(LoggerFn logger);
Result netDevices(int* ndev);
const NetDevice* netDevice(int dev);
struct NetProperties {
  const char* name;
  const char* pci_path;  // nullptr for virtual interfaces
  uint64_t guid;
  int ptr_support;
  int speed_mbps;
  int port;
  float latency;
  int max_comms;
  int max_recvs;
  int device_type;     // 0 host, 1 unpack
  int device_version;
};
Result netGetProperties(int dev, NetProperties* props);
Result netListen(int dev, void* handle, ListenComm** lcomm);
// Non-blocking: *comm stays null until the connection is up.
Result netConnect(int dev, void* handle, Comm** comm);
Result netAccept(ListenComm* lcomm, Comm** comm);
Result netRegMr(Comm* comm, void* data, size_t size, int type, MemHandle** mh);
Result netDeregMr(Comm* comm, MemHandle* mh);
// Creates every CUDA resource of the comm's data path ahead of time (see transport.cc).
Result netPrepareCuda(Comm* comm, int gpu_dev);
Result netIsend(Comm* comm, void* data, int size, int tag, MemHandle* mh, Request** req);
Result netIrecv(Comm* comm, int n, void** data, int* sizes, int* tags, MemHandle** mhs, Request** req);
Result netIflush(Comm* comm, int n, void** data, int* sizes, MemHandle** mhs, Request** req);
Result netTest(Request* req, int* done, int* size);
Result netClose(Comm* comm);
Result netCloseListen(ListenComm* lcomm);
// Unpack mode.  The device handle NCCL's kernels read; the memory handle they get.
Result netGetDeviceHandle(Comm* comm, void** dev_handle, size_t* size);
Result netGetDeviceMr(Comm* comm, MemHandle* mh, void** dptr_mhandle);
Result netIrecvConsumed(Comm* comm, int n, Request* req);
// Selects the receive mode of comms accepted from now on by this thread's next
// netAccept (used by the collective engine, which unpacks with its own kernels).
void netSetAcceptRecvMode(ListenComm* lcomm, int recv_mode);

// How the comm's idle helper threads wait for their next task, instead of what the
// HELPER_NAP_* flags say: nap `nap_us` at a time for `rounds` rounds, then sleep on their
// condition variable.  Naps spare the queueing thread a futex call per task, at the price of
// periodic wake-ups; right for a process with a handful of busy comms (the collective engine),
// wrong for one with dozens (NCCL with many channels), hence off by default.
void netSetHelperNap(Comm* comm, int nap_us, int rounds);
// Size of a send comm's pinned staging ring for CUDA buffers, instead of the
// TX_STAGING_BYTES flag.  A ring just large enough for the requests in flight is walked
// over and over and stays in the CPU's caches; a large one is always cold.  Call before
// the comm's first CUDA send (before netPrepareCuda).
Result netSetTxStagingBytes(Comm* comm, uint64_t bytes);
// Completion wake-ups for a driving thread that sleeps (see Notifier); null detaches.
// Set it while no request is in flight.
void netSetNotifier(Comm* comm, Notifier* notifier);
// The descriptor whose readability means "the peer sent control records this comm
// has not read yet" (receive side), or -1 when waiting on it would return at once
// (a record is already buffered) or never (send side).
int netCtrlPollFd(Comm* comm);
// For callers that poll() the descriptors of netCtrlPollFd themselves: "this comm's
// control socket is readable".  From the first call on, the comm reads its control
// socket only after such a hint (plus a rare blind retry), instead of trying, and
// paying a system call, on every progress round.
void netHintCtrlReadable(Comm* comm);
// Bytes per chunk for a message of `message_bytes` on a comm with `num_socks` data sockets.
int chunkBytesFor(int message_bytes, int num_socks);
constexpr int kMaxAdaptiveChunk = 4 << 20;

// The next netIsend of a CUDA buffer on `comm` first makes the comm's copy stream
// wait for `event` (the kernel that produces the data), then stages the data.
void netSetSendDependency(Comm* comm, gpu::Event event);

// Scatter list of a finished unpack-mode receive.
struct ScatterList {
  const LoadMeta* host;
  const LoadMeta* dev;
  uint64_t count;
  void* pool_dev;
  uint64_t pool_bytes;
};
Result netRequestScatterList(Request* req, ScatterList* out);

// Test and statistics accessors.
struct FlowCounters {
  uint64_t flow_id, bytes_posted, bytes_done, tx_cnt, tx_completion_cnt, rx_cnt;
};
int netCommFlowCounters(Comm* comm, FlowCounters* out, int max);
// Sums over the comm's helper threads: time asleep for want of a task, and time in
// poll() waiting for a socket to become ready.  Tells which side of a slow transfer waits.
void netCommHelperWaits(Comm* comm, uint64_t* idle_ns, uint64_t* blocked_ns);
std::vector<std::string> netCommStatsLines(Comm* comm);
void netResetForTests();

// Connection layer internals shared by transport.cc and connect.cc.
Result connectionInit();
Result startHelpers(Comm* comm);
Comm* newComm(int dev, bool passive);
void freeComm(Comm* comm);
// threads x sockets-per-thread for device `dev` (reference: src/connect.cc:165-220).
void chooseSocksThreads(int dev, int* nsocks, int* nthreads);

}  // namespace tcpxb
#endif  // TCPXB_TRANSPORT_H_
