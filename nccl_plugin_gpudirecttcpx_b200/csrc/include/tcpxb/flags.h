// Environment flag registry.
//
// Keeps the reference's whole environment surface (reference: src/net_tcpx.cc:69-122
// declares the parameters, :475-565 range-checks them into globals, src/flags.cc:19-74
// holds the compiled defaults) behind one declarative table instead of a macro per
// flag.  Two differences, both deliberate:
//   * an unset variable always means the documented default.  In the reference a
//     parameter whose own "unset" value is in range overrides the compiled default,
//     which turns the 128 KiB striping quantum into 0; that cannot happen here.
//   * out-of-range values are reported and ignored, never fatal.
// Names: "NCCL_<X>" for the generic ones shared with NCCL's socket transport,
// "NCCL_GPUDIRECTTCPX_<X>" for the plugin's own.
#ifndef TCPXB_FLAGS_H_
#define TCPXB_FLAGS_H_

#include <stdint.h>
#include <string>
#include <vector>

#include "tcpxb/base.h"

namespace tcpxb {

enum SlownessKind { kSlowTxComp = 0, kSlowSendRecv = 1, kSlowRxCtrl = 2, kSlowKinds = 3 };
enum SchedAlg { kSchedRR = 0, kSchedKaty = 1 };
enum RxPoolMode { kRxPoolHostMapped = 0, kRxPoolDevice = 1 };
enum RecvMode { kRecvModeHost = 0, kRecvModeUnpack = 1 };

struct Flags {
  // --- generic names (NCCL_*)
  int64_t min_zcopy_size = 0;          // NCCL_MIN_ZCOPY_SIZE; 0 disables MSG_ZEROCOPY
  int64_t nsocks_per_thread = -2;      // NCCL_NSOCKS_PERTHREAD; -2 = auto
  int64_t nthreads = -2;               // NCCL_SOCKET_NTHREADS; -2 = auto
  int64_t inline_threshold = 0;        // NCCL_INLINE_THRESHOLD, <= 2048
  int64_t dynamic_chunk_size = 128 * 1024;  // NCCL_DYNAMIC_CHUNK_SIZE
  int64_t thread_spin = 0;             // NCCL_THREAD_SPIN_ENABLE
  int64_t scatter_copy_min = 8192;     // NCCL_SCATTER_COPY_MIN_MESSAGE_SIZE (accepted, unused)
  int64_t staging_buffer_size = 8192;  // NCCL_STAGING_BUFFER_SIZE (accepted, unused)
  int64_t use_dma_buf = 1;             // NCCL_USE_DMA_BUF
  // --- plugin names (NCCL_GPUDIRECTTCPX_*)
  int64_t enable = 1;                  // SOCKET_ENABLE
  int64_t port_begin = -2, port_end = -2;  // PORT_BEGIN / PORT_END (accepted, unused)
  int64_t connection_retry = 3;        // CONNECTION_RETRY
  int64_t recv_sync = 0;               // RECV_SYNC
  int64_t force_ack = 0;               // FORCE_ACK
  int64_t tx_completion_nanosleep = 0; // TX_COMPLETION_NANOSLEEP
  int64_t timeout_threshold_ns = 10000000000ll;   // TIMEOUT_THRESHOLD_NS
  int64_t timeout_frequency_ns = 30000000000ll;   // TIMEOUT_FREQUENCY_NS
  int64_t spinwait_connect = 1;        // SPINWAIT_CONNECT
  int64_t log_stats_to_stdout = 0;     // LOG_STATS_TO_STDOUT
  int64_t task_level_stats = 0;        // TELEMETRY_ENABLE_TASK_LEVEL_STATS
  int64_t request_level_stats = 0;     // TELEMETRY_ENABLE_REQUEST_LEVEL_STATS
  int64_t export_stats_to_file = 0;    // TELEMETRY_EXPORT_STATS_TO_FILE
  int64_t sampling_factor = 1;         // TELEMETRY_SAMPLING_FACTOR
  int64_t log_line_limit = 256;        // TELEMETRY_LOG_LINE_LIMIT
  int64_t exporter_core_index = 171;   // TELEMETRY_EXPORTER_CORE_INDEX
  int64_t gc_core_index = 172;         // TELEMETRY_GARBAGE_COLLECTOR_INDEX
  int64_t file_life_min = 0;           // TELEMETRY_FILE_LIFE (minutes, 0 = keep)
  int64_t file_remove_frequency_s = 600;  // TELEMETRY_FILE_REMOVE_FREQUENCY
  int64_t report_lifecycle = 0;        // REPORT_LIFECYCLE
  int64_t cuda_use_primary_ctx = 1;    // CUDA_USE_PRIMARY_CTX
  int64_t nic_n_rxqs = 32;             // NIC_N_RXQS
  int64_t flow_steering_strategy = 3;  // FLOW_STEERING_STRATEGY (3 = unix client)
  int64_t flow_steering_wait_us = 0;   // PROGRAM_FLOW_STEERING_WAIT_MICROS
  int64_t rxmem_import_use_gpu_pci_client = 1;  // NCCL_TCPX_RXMEM_IMPORT_USE_GPU_PCI_CLIENT
  int64_t rxmem_import_skip_odds = 0;           // NCCL_TCPX_RXMEM_IMPORT_SKIP_ODDS
  int64_t reg_dmabuf_use_internal_api = 0;      // REG_DMABUF_USE_INTERNAL_API
  int64_t worker_pin_threads = 0;      // WORKER_PIN_THREADS
  int64_t worker_spray_count = 1;      // WORKER_SPRAY_COUNT
  int64_t worker_spray_stride = 0;     // WORKER_SPRAY_STRIDE
  std::string exporter_path = "/tmp";  // TELEMETRY_EXPORTER_PATH
  std::string socket_ifname;           // SOCKET_IFNAME
  std::string socket_family;           // SOCKET_FAMILY
  std::string ctrl_dev;                // CTRL_DEV
  std::string ctrl_sockcond;           // CTRL_SOCKCOND
  std::string port_mapping;            // PORT_MAPPING
  std::string tx_bindings, rx_bindings, tx_irq_bindings, rx_irq_bindings;
  std::string sched_alg_name;          // SCHED_ALG: RR | KATY
  std::string slowness_switch, slowness_report;
  std::string unix_client_prefix = "/tmp";  // UNIX_CLIENT_PREFIX
  std::string net_comm_id;             // NET_COMM_ID
  // --- additions of this implementation (NCCL_GPUDIRECTTCPX_*)
  int64_t virtual_nics = 0;            // VIRTUAL_NICS: present N devices on one interface (127.0.0.k on lo)
  int64_t rx_pool_bytes = 1ll << 30;   // RX_POOL_BYTES per GPU (<= 4 GiB: src_off is 32-bit)
  int64_t socket_sndbuf = 0;           // SOCKET_SNDBUF: bytes, 0 = auto-tuning
  int64_t socket_rcvbuf = 0;           // SOCKET_RCVBUF
  int64_t rx_pool_scatter = 1;         // RX_POOL_SCATTER: hand out pages in a scattered order
  int64_t rx_pool_run_pages = 8;       // RX_POOL_RUN_PAGES: consecutive pages per scattered group
  int64_t tx_staging_bytes = 32ll << 20;  // TX_STAGING_BYTES per send comm with CUDA buffers
  int64_t connect_refused_retries = 20000;  // CONNECT_REFUSED_RETRIES x 1 ms before a refused connect fails
  int64_t connect_pacing_us = 0;       // CONNECT_PACING_US per socket (the reference sleeps 100 ms)
  int64_t nic_speed_mbps = 0;          // NIC_SPEED_MBPS override for getProperties (0 = sysfs, else 10000)
  int64_t cuda_buffers = 0;            // CUDA_BUFFERS: accept CUDA pointers in host receive mode (see transport.h)
  int64_t adaptive_chunk = 1;          // ADAPTIVE_CHUNK: about one chunk per socket and message (see chunkBytesFor)
  int64_t helper_nap_us = 0;           // HELPER_NAP_US: idle helper threads nap this long at a time (0 = off; the engine turns it on for its comms) ...
  int64_t helper_nap_rounds = 50;      // HELPER_NAP_ROUNDS: ... this many times before they sleep until woken
  int64_t poll_block_us = 200;         // helper threads block in poll() this long when every socket would block
  std::string rx_pool_mode_name;       // RX_POOL_MODE: host | device
  std::string recv_mode_name;          // RECV_MODE: host | unpack
  std::string rx_buf_mgr_name;         // RX_BUF_MGR: emulated (in process) | daemon (tcpxb_rxdm over UNIX sockets) | devmem (kernel devmem-TCP)
  std::string rxdm_wire_name;          // RXDM_WIRE: native | proto
  // --- derived
  int sched_alg = kSchedRR;
  int rx_pool_mode = kRxPoolHostMapped;
  int recv_mode = kRecvModeHost;
  bool recv_mode_fell_back = false;  // unpack was asked for without NCCL_PROTO=Simple + NCCL_ALGO=Ring
  bool rx_buf_mgr_daemon = false;
  bool rxdm_wire_proto = false;       // talk to the daemon in the reference's protobuf wire format
  bool rx_buf_mgr_devmem = false;    // devmem-TCP datapath: pool from the daemon, fragments from the kernel
  bool slow_switch[kSlowKinds] = {false, false, false};
  bool slow_report[kSlowKinds] = {false, false, false};
};

// Parses the environment into `out`, logging every value (INFO, ENV subsystem) and
// every rejected one (WARN).  Never fails.
void loadFlags(Flags* out);
// The process-wide instance, loaded on first use and re-loadable for tests.
const Flags& flags();
void reloadFlags();

// "TX_COMP,SENDRECV,RX_CTRL,ALL" list -> per-kind booleans; unknown tokens are
// reported and skipped (reference: src/flags.cc:119-151).
bool parseSlownessList(const char* value, bool out[kSlowKinds]);

struct FlagDoc { const char* env; const char* kind; const char* dflt; const char* doc; };
// One line per known variable, for documentation and tests.
const std::vector<FlagDoc>& flagDocs();

}  // namespace tcpxb
#endif  // TCPXB_FLAGS_H_
