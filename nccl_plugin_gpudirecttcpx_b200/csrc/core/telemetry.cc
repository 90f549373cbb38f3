#include "tcpxb/telemetry.h"

#include <dirent.h>
#include <functional>
#include <pthread.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include "tcpxb/base.h"

namespace tcpxb {

uint64_t flowIdOf(const std::string& flow_string) { return std::hash<std::string>{}(flow_string); }

std::string flowStatsLine(const FlowStats& s, const std::string& flow, bool passive) {
  char buf[512];
  if (!passive) {
    snprintf(buf, sizeof buf, "per_flow_stats[%lu:%s] = tx [%lu/%lu] tx_slow %lu tx_comp_slow %lu",
             (unsigned long)s.flow_id, flow.c_str(), (unsigned long)s.tx_completion_cnt.load(),
             (unsigned long)s.tx_cnt.load(), (unsigned long)s.tx_slow_cnt.load(),
             (unsigned long)s.tx_completion_slow_cnt.load());
  } else {
    snprintf(buf, sizeof buf, "per_flow_stats[%lu:%s] = rx %lu rx_slow %lu", (unsigned long)s.flow_id,
             flow.c_str(), (unsigned long)s.rx_cnt.load(), (unsigned long)s.rx_slow_cnt.load());
  }
  return buf;
}

uint64_t epochNanos() {
  struct timespec ts;
  clock_gettime(CLOCK_REALTIME, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

EventLog::EventLog(size_t capacity, size_t line_limit) : ring_(capacity), line_limit_(line_limit) {
  for (auto& s : ring_) s.reserve(line_limit_);
}

bool EventLog::push(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  int n = vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (n < 0) return false;
  size_t len = (size_t)n < sizeof buf ? (size_t)n : sizeof buf - 1;
  if (len > line_limit_) len = line_limit_;
  {
    std::lock_guard<std::mutex> l(mu_);
    if (count_ == ring_.size()) {
      dropped_.fetch_add(1, std::memory_order_relaxed);
      return false;
    }
    ring_[(head_ + count_) % ring_.size()].assign(buf, len);
    ++count_;
  }
  cv_.notify_one();
  return true;
}

bool EventLog::pop(std::string* out, int timeout_ms) {
  std::unique_lock<std::mutex> l(mu_);
  if (count_ == 0) {
    cv_.wait_for(l, std::chrono::milliseconds(timeout_ms), [&] { return count_ > 0; });
    if (count_ == 0) return false;
  }
  out->swap(ring_[head_]);
  ring_[head_].clear();
  head_ = (head_ + 1) % ring_.size();
  --count_;
  return true;
}

size_t EventLog::size() {
  std::lock_guard<std::mutex> l(mu_);
  return count_;
}

void EventLog::wake() { cv_.notify_all(); }

namespace {
void pinToCore(int core) {
  if (core < 0) return;
  long ncpu = sysconf(_SC_NPROCESSORS_ONLN);
  if (ncpu <= 0 || core >= ncpu) return;  // the default indices assume a large host
  cpu_set_t set;
  CPU_ZERO(&set);
  CPU_SET(core, &set);
  pthread_setaffinity_np(pthread_self(), sizeof set, &set);
}
}  // namespace

Exporter::Exporter(EventLog* log, std::string dir, std::string tag, int core_index) : log_(log) {
  path_ = dir + "/exporter_" + std::to_string((long)getpid()) + "_" + tag + ".log";
  thread_ = std::thread([this, core_index] { run(core_index); });
}

Exporter::~Exporter() { stop(); }

void Exporter::stop() {
  if (!thread_.joinable()) return;
  stop_.store(true);
  log_->wake();
  thread_.join();
}

void Exporter::run(int core_index) {
  pinToCore(core_index);
  FILE* f = fopen(path_.c_str(), "a");
  if (f == nullptr) {
    WARN("event log %s cannot be opened: %s", path_.c_str(), strerror(errno));
    return;
  }
  std::string line;
  for (;;) {
    bool got = log_->pop(&line, 100);
    if (got) {
      fputs(line.c_str(), f);
      fputc('\n', f);
    } else if (stop_.load()) {
      break;
    } else {
      fflush(f);
    }
  }
  fclose(f);
}

std::string Exporter::statsPath(const std::string& dir, const std::string& tag) {
  return dir + "/exporter_stats_" + std::to_string((long)getpid()) + "_" + tag + ".log";
}

bool Exporter::writeStatsFile(const std::string& path, const std::vector<std::string>& lines) {
  FILE* f = fopen(path.c_str(), "w");
  if (f == nullptr) return false;
  for (const auto& l : lines) fprintf(f, "%s\n", l.c_str());
  fclose(f);
  return true;
}

int LogGarbageCollector::sweepOnce(const std::string& dir, int64_t life_minutes) {
  if (life_minutes <= 0) return 0;
  DIR* d = opendir(dir.c_str());
  if (d == nullptr) return 0;
  int removed = 0;
  const time_t now = time(nullptr);
  while (struct dirent* e = readdir(d)) {
    const char* n = e->d_name;
    size_t len = strlen(n);
    if (strncmp(n, "exporter_", 9) != 0 || len < 4 || strcmp(n + len - 4, ".log") != 0) continue;
    std::string p = dir + "/" + n;
    struct stat st;
    if (stat(p.c_str(), &st) != 0) continue;
    if ((now - st.st_mtime) > life_minutes * 60 && unlink(p.c_str()) == 0) ++removed;
  }
  closedir(d);
  return removed;
}

LogGarbageCollector::LogGarbageCollector(std::string dir, int64_t life_minutes, int64_t period_s, int core_index) {
  thread_ = std::thread([this, dir, life_minutes, period_s, core_index] {
    pinToCore(core_index);
    std::unique_lock<std::mutex> l(mu_);
    while (!stop_) {
      l.unlock();
      sweepOnce(dir, life_minutes);
      l.lock();
      cv_.wait_for(l, std::chrono::seconds(period_s), [&] { return stop_; });
    }
  });
}

LogGarbageCollector::~LogGarbageCollector() {
  {
    std::lock_guard<std::mutex> l(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
}

namespace {
TraceConfig g_trace;
}
void setTraceConfig(const TraceConfig& c) { g_trace = c; }
const TraceConfig& traceConfig() { return g_trace; }

void traceTransition(EventLog* log, char kind, const void* object, bool passive, const char* state) {
  if (log == nullptr || !g_trace.to_file) return;
  if (kind == 'T' ? !g_trace.task_level : !g_trace.request_level) return;
  if (g_trace.sampling > 1 && (reinterpret_cast<uintptr_t>(object) / 64) % g_trace.sampling != 0) return;
  log->push("%c %p %d %s %lu", kind, object, passive ? 1 : 0, state, (unsigned long)epochNanos());
}

}  // namespace tcpxb
