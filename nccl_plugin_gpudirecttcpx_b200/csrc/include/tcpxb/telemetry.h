// Telemetry: per-flow counters, tracepoints, a bounded event log with an exporter
// thread, and a garbage collector for old log files.
//
// Mirrors the reference's stats directory in function (reference:
// src/stats/monitoring.h:25-41 counters, src/stats/tracepoint.cc:112-235
// tracepoints, src/stats/stats_buffer.h:33-137 bounded ring, src/stats/exporter.h:31-89
// file writer, src/net_tcpx.cc:394-430 log GC).  The event line format is kept:
//   "T <object> <passive> <state> <ns-since-epoch>"   task transition
//   "R <object> <passive> <state> <ns-since-epoch>"   request transition
// and the per-flow summary line:
//   per_flow_stats[<id>:<flow>] = tx [<completed>/<total>] tx_slow <n> tx_comp_slow <n>
//   per_flow_stats[<id>:<flow>] = rx <n> rx_slow <n>
#ifndef TCPXB_TELEMETRY_H_
#define TCPXB_TELEMETRY_H_

#include <atomic>
#include <condition_variable>
#include <mutex>
#include <stdint.h>
#include <string>
#include <thread>
#include <vector>

namespace tcpxb {

struct FlowStats {
  uint64_t flow_id = 0;
  std::atomic<uint64_t> tx_cnt{0};             // sendmsg calls that moved bytes
  std::atomic<uint64_t> tx_completion_cnt{0};  // zero-copy completions (or, without zero-copy, finished sends)
  std::atomic<uint64_t> tx_slow_cnt{0};
  std::atomic<uint64_t> tx_completion_slow_cnt{0};
  std::atomic<uint64_t> rx_cnt{0};             // recvmsg calls that moved bytes
  std::atomic<uint64_t> rx_slow_cnt{0};
  std::atomic<uint64_t> bytes_posted{0};       // handed to / taken from the kernel
  std::atomic<uint64_t> bytes_done{0};         // completed
};
uint64_t flowIdOf(const std::string& flow_string);
std::string flowStatsLine(const FlowStats& s, const std::string& flow, bool passive);

// Bounded multi-producer single-consumer log of short text lines.  Producers never
// block: a full log drops the line and counts it.
class EventLog {
 public:
  explicit EventLog(size_t capacity = 10000, size_t line_limit = 256);
  // printf-style; returns false when dropped.
  bool push(const char* fmt, ...) __attribute__((format(printf, 2, 3)));
  // Consumer: waits up to timeout_ms for a line.
  bool pop(std::string* out, int timeout_ms);
  size_t size();
  uint64_t dropped() const { return dropped_.load(); }
  void wake();

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<std::string> ring_;
  size_t head_ = 0, count_ = 0, line_limit_;
  std::atomic<uint64_t> dropped_{0};
};

// Drains an EventLog to "<dir>/exporter_<pid>_<tag>.log" on its own thread.
class Exporter {
 public:
  Exporter(EventLog* log, std::string dir, std::string tag, int core_index);
  ~Exporter();
  void stop();
  const std::string& path() const { return path_; }
  // "<dir>/exporter_stats_<pid>_<tag>.log"
  static std::string statsPath(const std::string& dir, const std::string& tag);
  static bool writeStatsFile(const std::string& path, const std::vector<std::string>& lines);

 private:
  void run(int core_index);
  EventLog* log_;
  std::string path_;
  std::atomic<bool> stop_{false};
  std::thread thread_;
};

// Removes "<dir>/exporter_*.log" files older than life_minutes, every period_s
// seconds, on a detached-style thread owned by this object.
class LogGarbageCollector {
 public:
  LogGarbageCollector(std::string dir, int64_t life_minutes, int64_t period_s, int core_index);
  ~LogGarbageCollector();
  static int sweepOnce(const std::string& dir, int64_t life_minutes);

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  bool stop_ = false;
  std::thread thread_;
};

// Tracepoint switches, copied from the flags at init.
struct TraceConfig {
  bool task_level = false, request_level = false, to_file = false;
  uint64_t sampling = 1;
};
void setTraceConfig(const TraceConfig& c);
const TraceConfig& traceConfig();
uint64_t epochNanos();

// Emits one transition line when the switches and the sampling of `object` allow.
void traceTransition(EventLog* log, char kind /* 'T' or 'R' */, const void* object, bool passive,
                     const char* state);

}  // namespace tcpxb
#endif  // TCPXB_TELEMETRY_H_
