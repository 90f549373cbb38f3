#include "tcpxb/flags.h"

#include <limits.h>

#include <atomic>
#include <mutex>
#include <stdlib.h>
#include <strings.h>

namespace tcpxb {
namespace {

constexpr const char* kGen = "NCCL_";
constexpr const char* kOwn = "NCCL_GPUDIRECTTCPX_";

struct IntSpec {
  const char* prefix;
  const char* name;
  int64_t Flags::*field;
  int64_t lo, hi;  // accepted when lo <= v < hi
  const char* doc;
};
struct StrSpec {
  const char* prefix;
  const char* name;
  std::string Flags::*field;
  const char* doc;
};

constexpr int64_t kMax = INT64_MAX;

const IntSpec kInts[] = {
    {kGen, "MIN_ZCOPY_SIZE", &Flags::min_zcopy_size, 0, INT_MAX, "minimum bytes for MSG_ZEROCOPY on host sends (0 = off)"},
    {kGen, "NSOCKS_PERTHREAD", &Flags::nsocks_per_thread, -2, 9, "data sockets per helper thread (-2 = auto)"},
    {kGen, "SOCKET_NTHREADS", &Flags::nthreads, -2, 17, "helper threads per comm (-2 = auto)"},
    {kGen, "INLINE_THRESHOLD", &Flags::inline_threshold, 0, 2049, "payloads up to this size ride the ctrl socket"},
    {kGen, "DYNAMIC_CHUNK_SIZE", &Flags::dynamic_chunk_size, 1, INT_MAX, "striping quantum in bytes"},
    {kGen, "THREAD_SPIN_ENABLE", &Flags::thread_spin, 0, 2, "helper threads never sleep"},
    {kGen, "SCATTER_COPY_MIN_MESSAGE_SIZE", &Flags::scatter_copy_min, 0, kMax, "accepted for compatibility, unused"},
    {kGen, "STAGING_BUFFER_SIZE", &Flags::staging_buffer_size, 0, kMax, "accepted for compatibility, unused"},
    {kGen, "USE_DMA_BUF", &Flags::use_dma_buf, 0, 2, "devmem datapath: export registered CUDA buffers as dma-bufs for zero-copy transmit"},
    {kOwn, "SOCKET_ENABLE", &Flags::enable, 0, 2, "0 makes init fail so NCCL falls back"},
    {kOwn, "PORT_BEGIN", &Flags::port_begin, -2, 65536, "accepted for compatibility, unused"},
    {kOwn, "PORT_END", &Flags::port_end, -2, 65536, "accepted for compatibility, unused"},
    {kOwn, "CONNECTION_RETRY", &Flags::connection_retry, 0, 1000, "handshake retries per socket"},
    {kOwn, "RECV_SYNC", &Flags::recv_sync, 0, 2, "sender waits for the receiver's posted index per request"},
    {kOwn, "FORCE_ACK", &Flags::force_ack, 0, 2, "TCP_QUICKACK when a socket's receive queue drains"},
    {kOwn, "TX_COMPLETION_NANOSLEEP", &Flags::tx_completion_nanosleep, 0, 1000000000, "sleep while waiting for zero-copy completions"},
    {kOwn, "TIMEOUT_THRESHOLD_NS", &Flags::timeout_threshold_ns, 100000, kMax, "first slowness warning after this long"},
    {kOwn, "TIMEOUT_FREQUENCY_NS", &Flags::timeout_frequency_ns, 100000, kMax, "repeat slowness warnings this often"},
    {kOwn, "SPINWAIT_CONNECT", &Flags::spinwait_connect, 0, 2, "isend/irecv wait for the connection instead of returning no request"},
    {kOwn, "LOG_STATS_TO_STDOUT", &Flags::log_stats_to_stdout, 0, 2, "per-flow statistics at close"},
    {kOwn, "TELEMETRY_ENABLE_TASK_LEVEL_STATS", &Flags::task_level_stats, 0, 2, "task tracepoints into the event log"},
    {kOwn, "TELEMETRY_ENABLE_REQUEST_LEVEL_STATS", &Flags::request_level_stats, 0, 2, "request tracepoints into the event log"},
    {kOwn, "TELEMETRY_EXPORT_STATS_TO_FILE", &Flags::export_stats_to_file, 0, 2, "run the exporter thread"},
    {kOwn, "TELEMETRY_SAMPLING_FACTOR", &Flags::sampling_factor, 1, 1000001, "log one object in N"},
    {kOwn, "TELEMETRY_LOG_LINE_LIMIT", &Flags::log_line_limit, 1, 257, "bytes per event-log line"},
    {kOwn, "TELEMETRY_EXPORTER_CORE_INDEX", &Flags::exporter_core_index, 0, 4096, "core of the exporter thread"},
    {kOwn, "TELEMETRY_GARBAGE_COLLECTOR_INDEX", &Flags::gc_core_index, 0, 4096, "core of the log garbage collector"},
    {kOwn, "TELEMETRY_FILE_LIFE", &Flags::file_life_min, 0, kMax, "remove event logs older than this many minutes (0 = keep)"},
    {kOwn, "TELEMETRY_FILE_REMOVE_FREQUENCY", &Flags::file_remove_frequency_s, 1, kMax, "seconds between garbage-collector passes"},
    {kOwn, "REPORT_LIFECYCLE", &Flags::report_lifecycle, 0, 2, "register the process with the rx buffer manager"},
    {kOwn, "CUDA_USE_PRIMARY_CTX", &Flags::cuda_use_primary_ctx, 0, 2, "driver-API services use the device's primary context (0: a context of the library's own, for the buffer manager daemon)"},
    {kOwn, "NIC_N_RXQS", &Flags::nic_n_rxqs, 1, 4096, "receive queues per NIC assumed by the queue-balance bookkeeping"},
    {kOwn, "FLOW_STEERING_STRATEGY", &Flags::flow_steering_strategy, 0, 4, "3 = rules through the rx buffer manager"},
    {kOwn, "PROGRAM_FLOW_STEERING_WAIT_MICROS", &Flags::flow_steering_wait_us, 0, kMax, "receiver pause after accept"},
    {"NCCL_TCPX_", "RXMEM_IMPORT_USE_GPU_PCI_CLIENT", &Flags::rxmem_import_use_gpu_pci_client, 0, 2, "with RX_BUF_MGR=daemon: 1 = pool descriptor from the daemon's sockets, 0 = 64-byte memory handle from <UNIX_CLIENT_PREFIX>/nvdma-<pci>"},
    {"NCCL_TCPX_", "RXMEM_IMPORT_SKIP_ODDS", &Flags::rxmem_import_skip_odds, 0, 2, "1 = odd-numbered GPUs get no rx pool (receives into their memory fail)"},
    {kOwn, "REG_DMABUF_USE_INTERNAL_API", &Flags::reg_dmabuf_use_internal_api, 0, 2, "1 asks for the driver's procfs dma-buf interface, which is not offered: the CUDA export call is used"},
    {kOwn, "WORKER_PIN_THREADS", &Flags::worker_pin_threads, 0, 2, "pin every helper thread to one core"},
    {kOwn, "WORKER_SPRAY_COUNT", &Flags::worker_spray_count, 1, 4096, "helper placement: candidates per thread"},
    {kOwn, "WORKER_SPRAY_STRIDE", &Flags::worker_spray_stride, 0, 4096, "helper placement: stride between comms"},
    {kOwn, "VIRTUAL_NICS", &Flags::virtual_nics, 0, 17, "present N devices on one interface (127.0.0.k on lo)"},
    {kOwn, "RX_POOL_BYTES", &Flags::rx_pool_bytes, 1 << 20, (4ll << 30) + 1, "rx page pool per GPU"},
    {kOwn, "SOCKET_SNDBUF", &Flags::socket_sndbuf, 0, kMax, "SO_SNDBUF of every data socket in bytes (0 = the kernel's auto-tuning; values below 65536 are raised to it)"},
    {kOwn, "SOCKET_RCVBUF", &Flags::socket_rcvbuf, 0, kMax, "SO_RCVBUF of every data socket in bytes (0 = the kernel's auto-tuning; values below 65536 are raised to it)"},
    {kOwn, "RX_POOL_SCATTER", &Flags::rx_pool_scatter, 0, 2, "hand out rx pages in a scattered order"},
    {kOwn, "RX_POOL_RUN_PAGES", &Flags::rx_pool_run_pages, 1, 1025, "consecutive pages per scattered group of the rx pool"},
    {kOwn, "TX_STAGING_BYTES", &Flags::tx_staging_bytes, 1 << 16, kMax, "pinned staging per send comm for CUDA buffers"},
    {kOwn, "CONNECT_REFUSED_RETRIES", &Flags::connect_refused_retries, 0, 10000000, "retries, 1 ms apart, while the peer refuses the connection"},
    {kOwn, "CONNECT_PACING_US", &Flags::connect_pacing_us, 0, kMax, "pause per socket during connection setup"},
    {kOwn, "NIC_SPEED_MBPS", &Flags::nic_speed_mbps, 0, 100000000, "speed reported to NCCL (0 = sysfs, else 10000)"},
    {kOwn, "CUDA_BUFFERS", &Flags::cuda_buffers, 0, 2, "host receive mode also takes CUDA pointers (plugin-side copies and kernels)"},
    {kOwn, "ADAPTIVE_CHUNK", &Flags::adaptive_chunk, 0, 2, "cut a message into about one chunk per socket (0 = always NCCL_DYNAMIC_CHUNK_SIZE)"},
    {kOwn, "HELPER_NAP_US", &Flags::helper_nap_us, 0, 100000, "idle helper threads nap this long at a time before sleeping until woken (0 = sleep at once; the collective engine uses 20 for its own comms)"},
    {kOwn, "HELPER_NAP_ROUNDS", &Flags::helper_nap_rounds, 0, 1000000, "naps an idle helper thread takes before it sleeps until woken"},
    {kOwn, "POLL_BLOCK_US", &Flags::poll_block_us, 0, 1000000, "helper threads block in poll() this long when idle on EAGAIN"},
};

const StrSpec kStrs[] = {
    {kOwn, "TELEMETRY_EXPORTER_PATH", &Flags::exporter_path, "directory of the event logs"},
    {kOwn, "SOCKET_IFNAME", &Flags::socket_ifname, "data interfaces, NCCL prefix-list syntax"},
    {kOwn, "SOCKET_FAMILY", &Flags::socket_family, "AF_INET or AF_INET6"},
    {kOwn, "CTRL_DEV", &Flags::ctrl_dev, "interface that carries the ctrl sockets"},
    {kOwn, "CTRL_SOCKCOND", &Flags::ctrl_sockcond, "ctrl socket CPU-locality check (diagnostic)"},
    {kOwn, "PORT_MAPPING", &Flags::port_mapping, "parsed and logged; the fixed-port strategy is not offered"},
    {kOwn, "TX_BINDINGS", &Flags::tx_bindings, "core ranges per NIC for sending helpers"},
    {kOwn, "RX_BINDINGS", &Flags::rx_bindings, "core ranges per NIC for receiving helpers"},
    {kOwn, "TX_IRQ_BINDINGS", &Flags::tx_irq_bindings, "core ranges per NIC, tx interrupts (recorded)"},
    {kOwn, "RX_IRQ_BINDINGS", &Flags::rx_irq_bindings, "core ranges per NIC, rx interrupts (recorded)"},
    {kOwn, "SCHED_ALG", &Flags::sched_alg_name, "RR or KATY"},
    {kOwn, "SLOWNESS_SWITCH", &Flags::slowness_switch, "detectors to run: TX_COMP,SENDRECV,RX_CTRL,ALL"},
    {kOwn, "SLOWNESS_REPORT", &Flags::slowness_report, "detectors that print: TX_COMP,SENDRECV,RX_CTRL,ALL"},
    {kOwn, "UNIX_CLIENT_PREFIX", &Flags::unix_client_prefix, "directory of the rx buffer manager's sockets"},
    {"", "NET_COMM_ID", &Flags::net_comm_id, "subnet hint for interface auto-selection"},
    {kOwn, "RX_POOL_MODE", &Flags::rx_pool_mode_name, "host (pinned, device-mapped) or device (copy-engine placement)"},
    {kOwn, "RECV_MODE", &Flags::recv_mode_name, "host (plugin unpacks) or unpack (NCCL's kernels unpack)"},
    {kOwn, "RX_BUF_MGR", &Flags::rx_buf_mgr_name, "emulated (in process), daemon (tcpxb_rxdm under UNIX_CLIENT_PREFIX), devmem (kernel devmem-TCP sockets, pool from the daemon) or devmem-local (the same with a pool of the process's own)"},
    {kOwn, "RXDM_WIRE", &Flags::rxdm_wire_name, "native (fixed structs, tcpxb_rxdm) or proto (the protobuf messages and per-GPU socket names of Google's daemon)"},
};

std::string envName(const char* prefix, const char* name) { return std::string(prefix) + name; }

// Variables of the plugin's own family are also read under the stand-alone prefix
// NET_TCPX_ (reference: src/adapter/native/param.h:35), for programs that use the
// transport without NCCL; the NCCL-style name wins when both are set.
const char* lookup(const char* prefix, const char* name, std::string* used) {
  *used = envName(prefix, name);
  const char* v = getenv(used->c_str());
  if ((v == nullptr || *v == 0) && strcmp(prefix, kOwn) == 0) {
    const std::string alt = envName("NET_TCPX_", name);
    const char* a = getenv(alt.c_str());
    if (a != nullptr && *a != 0) { *used = alt; return a; }
  }
  return v;
}

}  // namespace

bool parseSlownessList(const char* value, bool out[kSlowKinds]) {
  for (int i = 0; i < kSlowKinds; ++i) out[i] = false;
  if (value == nullptr || *value == 0) return true;
  bool ok = true;
  std::string s(value);
  size_t pos = 0;
  while (pos <= s.size()) {
    size_t end = s.find(',', pos);
    if (end == std::string::npos) end = s.size();
    std::string tok = s.substr(pos, end - pos);
    pos = end + 1;
    if (tok.empty()) continue;
    if (!strcasecmp(tok.c_str(), "TX_COMP")) out[kSlowTxComp] = true;
    else if (!strcasecmp(tok.c_str(), "SENDRECV")) out[kSlowSendRecv] = true;
    else if (!strcasecmp(tok.c_str(), "RX_CTRL")) out[kSlowRxCtrl] = true;
    else if (!strcasecmp(tok.c_str(), "ALL")) { for (int i = 0; i < kSlowKinds; ++i) out[i] = true; }
    else { WARN("unknown slowness detector '%s' ignored", tok.c_str()); ok = false; }
  }
  return ok;
}

void loadFlags(Flags* out) {
  *out = Flags();
  for (const IntSpec& s : kInts) {
    std::string env;
    const char* v = lookup(s.prefix, s.name, &env);
    if (v != nullptr && *v != 0) {
      char* end = nullptr;
      errno = 0;
      long long parsed = strtoll(v, &end, 0);
      if (errno != 0 || end == v || *end != 0) {
        WARN("%s='%s' is not an integer; keeping %lld", env.c_str(), v, (long long)(out->*s.field));
      } else if (parsed < s.lo || parsed >= s.hi) {
        WARN("%s=%lld outside [%lld, %lld); keeping %lld", env.c_str(), parsed, (long long)s.lo,
             (long long)s.hi, (long long)(out->*s.field));
      } else {
        out->*s.field = parsed;
      }
    }
    INFO(kSubEnv, "%s = %lld", env.c_str(), (long long)(out->*s.field));
  }
  for (const StrSpec& s : kStrs) {
    std::string env;
    const char* v = lookup(s.prefix, s.name, &env);
    if (v != nullptr && *v != 0) out->*s.field = v;
    if (!(out->*s.field).empty()) INFO(kSubEnv, "%s = %s", env.c_str(), (out->*s.field).c_str());
  }
  out->sched_alg = kSchedRR;
  if (!out->sched_alg_name.empty()) {
    if (!strcasecmp(out->sched_alg_name.c_str(), "KATY")) out->sched_alg = kSchedKaty;
    else if (strcasecmp(out->sched_alg_name.c_str(), "RR"))
      WARN("unknown scheduling algorithm '%s'; using RR", out->sched_alg_name.c_str());
  }
  out->rx_pool_mode = kRxPoolHostMapped;
  if (!strcasecmp(out->rx_pool_mode_name.c_str(), "device")) out->rx_pool_mode = kRxPoolDevice;
  else if (!out->rx_pool_mode_name.empty() && strcasecmp(out->rx_pool_mode_name.c_str(), "host"))
    WARN("unknown rx pool mode '%s'; using host", out->rx_pool_mode_name.c_str());
  out->recv_mode = kRecvModeHost;
  if (!strcasecmp(out->recv_mode_name.c_str(), "unpack")) out->recv_mode = kRecvModeUnpack;
  else if (!out->recv_mode_name.empty() && strcasecmp(out->recv_mode_name.c_str(), "host"))
    WARN("unknown receive mode '%s'; using host", out->recv_mode_name.c_str());
  if (out->recv_mode == kRecvModeUnpack) {
    // Only the ring primitives of NCCL's Simple protocol copy the payload out of the rx
    // pool; with any other algorithm or protocol the consumer would never run and the
    // user's buffers would keep stale data.  Without both settings the plugin does not
    // offer the unpack device type: it receives into host buffers like any net plugin.
    const char* proto = getenv("NCCL_PROTO");
    const char* algo = getenv("NCCL_ALGO");
    const bool ok = proto != nullptr && !strcasecmp(proto, "Simple") && algo != nullptr && !strcasecmp(algo, "Ring");
    if (!ok) {
      WARN("NCCL_GPUDIRECTTCPX_RECV_MODE=unpack needs NCCL_PROTO=Simple and NCCL_ALGO=Ring (found NCCL_PROTO=%s, NCCL_ALGO=%s): "
           "using host receive mode instead", proto ? proto : "(unset)", algo ? algo : "(unset)");
      out->recv_mode = kRecvModeHost;
      out->recv_mode_fell_back = true;
    }
  }
  const bool devmem_local = !strcasecmp(out->rx_buf_mgr_name.c_str(), "devmem-local");
  out->rx_buf_mgr_devmem = devmem_local || !strcasecmp(out->rx_buf_mgr_name.c_str(), "devmem");
  // the devmem datapath takes its pool (bound to the NIC's queues) from the daemon as well,
  // unless the process owns the binding itself ("devmem-local")
  out->rx_buf_mgr_daemon = (out->rx_buf_mgr_devmem && !devmem_local) || !strcasecmp(out->rx_buf_mgr_name.c_str(), "daemon");
  if (!out->rx_buf_mgr_daemon && !out->rx_buf_mgr_devmem && !out->rx_buf_mgr_name.empty() &&
      strcasecmp(out->rx_buf_mgr_name.c_str(), "emulated"))
    WARN("unknown rx buffer manager '%s'; using the in-process one", out->rx_buf_mgr_name.c_str());
  out->rxdm_wire_proto = !strcasecmp(out->rxdm_wire_name.c_str(), "proto") || !strcasecmp(out->rxdm_wire_name.c_str(), "protobuf");
  if (!out->rxdm_wire_proto && !out->rxdm_wire_name.empty() && strcasecmp(out->rxdm_wire_name.c_str(), "native"))
    WARN("unknown rx buffer manager wire format '%s'; using the native one", out->rxdm_wire_name.c_str());
  // A send buffer below two loopback segments (64 KiB MTU) lets the stream send one segment per
  // delayed ACK: measured 44 s for a step that takes 40 ms.  Small values are raised, not obeyed.
  for (int64_t* v : {&out->socket_sndbuf, &out->socket_rcvbuf}) {
    if (*v > 0 && *v < 65536) {
      WARN("socket buffer of %ld bytes is too small to keep a stream moving; using 65536", (long)*v);
      *v = 65536;
    }
  }
  parseSlownessList(out->slowness_switch.c_str(), out->slow_switch);
  parseSlownessList(out->slowness_report.c_str(), out->slow_report);
  if (out->inline_threshold > out->dynamic_chunk_size) out->inline_threshold = out->dynamic_chunk_size;
}

namespace {
// Readers are on every hot path (helper threads, progress engine), so they take no
// lock: the current set is published through one atomic pointer.  A reload builds
// a fresh set and swaps it in; the old one is left alive for readers still using it.
std::mutex g_mu;
std::atomic<Flags*> g_flags{nullptr};
}  // namespace

const Flags& flags() {
  Flags* f = g_flags.load(std::memory_order_acquire);
  if (f != nullptr) return *f;
  std::lock_guard<std::mutex> l(g_mu);
  f = g_flags.load(std::memory_order_acquire);
  if (f == nullptr) {
    f = new Flags();
    loadFlags(f);
    g_flags.store(f, std::memory_order_release);
  }
  return *f;
}

void reloadFlags() {
  // Readers hold plain references with no count, so a replaced table is never freed:
  // it is parked here, reachable until the process ends.  Reloads happen at init only.
  static std::vector<Flags*>* retired = new std::vector<Flags*>();
  std::lock_guard<std::mutex> l(g_mu);
  Flags* f = new Flags();
  loadFlags(f);
  Flags* old = g_flags.exchange(f, std::memory_order_acq_rel);
  if (old != nullptr) retired->push_back(old);
}

const std::vector<FlagDoc>& flagDocs() {
  static const std::vector<FlagDoc>* docs = [] {
    auto* v = new std::vector<FlagDoc>();
    static std::vector<std::string> names, dflts;
    Flags d;
    names.reserve(256);
    dflts.reserve(256);
    for (const IntSpec& s : kInts) {
      names.push_back(envName(s.prefix, s.name));
      dflts.push_back(std::to_string(d.*s.field));
      v->push_back({names.back().c_str(), "int", dflts.back().c_str(), s.doc});
    }
    for (const StrSpec& s : kStrs) {
      names.push_back(envName(s.prefix, s.name));
      dflts.push_back(d.*s.field);
      v->push_back({names.back().c_str(), "string", dflts.back().c_str(), s.doc});
    }
    return v;
  }();
  return *docs;
}

}  // namespace tcpxb
