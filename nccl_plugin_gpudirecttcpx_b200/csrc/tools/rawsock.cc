// Raw TCP ceiling of this machine: S parallel streams over loopback, one sender and
// one receiver thread per stream in two processes, plain send()/recv() of large
// blocks and nothing else.  The transport cannot beat this number; benchmarks
// report their socket stage as a fraction of it.
//   tcpxb_rawsock [--streams 8] [--mb-per-stream 2048] [--block-kb 512] [--nics 4]
//                 [--span-mb 0] [--sndbuf-kb 0] [--nonblocking 0] [--scatter-kb 0]
// Prints one JSON line.  Stream i uses address 127.0.0.(1 + i % nics).
// The defaults give the friendliest case (one block per thread, reused, so it stays
// in the core's cache; blocking calls).  The other options take that apart:
//   --span-mb M      every thread walks through a buffer of M MiB block by block, so that
//                    with a large M the copies miss the caches, as a transport's do when
//                    its staging and landing buffers are as large as the data in flight;
//   --sndbuf-kb K    SO_SNDBUF of K KiB on every sending socket instead of the kernel's auto-tuning
//                    (which lets megabytes per stream sit in the kernel, out of the caches);
//   --nonblocking 1  MSG_DONTWAIT calls with poll() when the socket would block;
//   --scatter-kb K   the receiver lands every block with one recvmsg over pieces of K KiB
//                    at shuffled places of its span (page-pool landing).
#include <arpa/inet.h>
#include <errno.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <sys/wait.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <string>
#include <thread>
#include <vector>

namespace {

double nowSec() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}

struct Options {
  int streams = 8;
  long mb = 2048;
  int block_kb = 512;
  int nics = 4;
  long span_mb = 0;
  long sndbuf_kb = 0;
  int nonblocking = 0;
  int scatter_kb = 0;
};

void waitFor(int fd, short events) {
  struct pollfd p = {fd, events, 0};
  poll(&p, 1, 100);
}

int receiver(const Options& o, int port_pipe, int go_pipe) {
  std::vector<int> lfd(o.streams), ports(o.streams);
  for (int i = 0; i < o.streams; ++i) {
    lfd[i] = socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_addr.s_addr = htonl(0x7f000001u + (uint32_t)(i % o.nics));
    if (bind(lfd[i], (sockaddr*)&a, sizeof a) != 0 || listen(lfd[i], 4) != 0) return 1;
    socklen_t len = sizeof a;
    getsockname(lfd[i], (sockaddr*)&a, &len);
    ports[i] = ntohs(a.sin_port);
  }
  if (write(port_pipe, ports.data(), ports.size() * sizeof(int)) < 0) return 1;
  std::vector<int> fd(o.streams);
  for (int i = 0; i < o.streams; ++i) fd[i] = accept(lfd[i], nullptr, nullptr);
  const size_t block = (size_t)o.block_kb << 10;
  const size_t total = (size_t)o.mb << 20;
  char go = 'g';
  if (write(go_pipe, &go, 1) != 1) return 1;
  const double t0 = nowSec();
  std::vector<std::thread> th;
  for (int i = 0; i < o.streams; ++i)
    th.emplace_back([&, i] {
      const size_t span = std::max(block, (size_t)o.span_mb << 20) / block * block;
      std::vector<char> buf(span);
      const int fl = o.nonblocking ? MSG_DONTWAIT : 0;
      // scattered landing: the pieces of the span in a fixed shuffled order
      const size_t piece = (size_t)o.scatter_kb << 10;
      std::vector<uint32_t> order;
      if (piece > 0) {
        order.resize(span / piece);
        for (uint32_t k = 0; k < order.size(); ++k) order[k] = k;
        uint64_t x = 0x9e3779b97f4a7c15ull + (uint64_t)i;
        for (size_t k = order.size(); k > 1; --k) {
          x ^= x << 13; x ^= x >> 7; x ^= x << 17;
          std::swap(order[k - 1], order[x % k]);
        }
      }
      std::vector<struct iovec> iov;
      size_t got = 0, pos = 0, next_piece = 0;
      while (got < total) {
        ssize_t n;
        if (piece > 0) {
          if (iov.empty()) {
            for (size_t b = 0; b < block; b += piece) {
              iov.push_back({buf.data() + (size_t)order[next_piece] * piece, piece});
              next_piece = (next_piece + 1) % order.size();
            }
          }
          struct msghdr msg;
          memset(&msg, 0, sizeof msg);
          msg.msg_iov = iov.data();
          msg.msg_iovlen = iov.size();
          n = recvmsg(fd[i], &msg, fl);
          if (n > 0) {
            size_t left = (size_t)n, k = 0;
            while (left > 0 && k < iov.size()) {
              if (left >= iov[k].iov_len) { left -= iov[k].iov_len; ++k; }
              else { iov[k].iov_base = (char*)iov[k].iov_base + left; iov[k].iov_len -= left; left = 0; }
            }
            iov.erase(iov.begin(), iov.begin() + (long)k);
          }
        } else {
          n = recv(fd[i], buf.data() + pos, block, fl);
          if (n > 0) pos = (pos + block) % span;
        }
        if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) { waitFor(fd[i], POLLIN); continue; }
        if (n <= 0) break;
        got += (size_t)n;
      }
    });
  for (auto& t : th) t.join();
  const double dt = nowSec() - t0;
  printf("{\"tool\": \"rawsock\", \"streams\": %d, \"block_kb\": %d, \"mb_per_stream\": %ld, \"span_mb\": %ld, \"sndbuf_kb\": %ld, \"nonblocking\": %d, "
         "\"scatter_kb\": %d, \"seconds\": %.4f, \"GBps\": %.3f}\n",
         o.streams, o.block_kb, o.mb, o.span_mb, o.sndbuf_kb, o.nonblocking, o.scatter_kb, dt, (double)total * o.streams / dt / 1e9);
  return 0;
}

int sender(const Options& o, int port_pipe, int go_pipe) {
  std::vector<int> ports(o.streams);
  size_t need = ports.size() * sizeof(int), got = 0;
  while (got < need) {
    ssize_t n = read(port_pipe, (char*)ports.data() + got, need - got);
    if (n <= 0) return 1;
    got += (size_t)n;
  }
  std::vector<int> fd(o.streams);
  for (int i = 0; i < o.streams; ++i) {
    fd[i] = socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_addr.s_addr = htonl(0x7f000001u + (uint32_t)(i % o.nics));
    a.sin_port = htons((uint16_t)ports[i]);
    int one = 1;
    setsockopt(fd[i], IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
    if (o.sndbuf_kb > 0) {
      const int bytes = (int)(o.sndbuf_kb << 10);
      setsockopt(fd[i], SOL_SOCKET, SO_SNDBUF, &bytes, sizeof bytes);
    }
    if (connect(fd[i], (sockaddr*)&a, sizeof a) != 0) return 1;
  }
  char go;
  if (read(go_pipe, &go, 1) != 1) return 1;
  const size_t block = (size_t)o.block_kb << 10;
  const size_t total = (size_t)o.mb << 20;
  std::vector<std::thread> th;
  for (int i = 0; i < o.streams; ++i)
    th.emplace_back([&, i] {
      const size_t span = std::max(block, (size_t)o.span_mb << 20) / block * block;
      std::vector<char> buf(span, (char)i);
      const int fl = MSG_NOSIGNAL | (o.nonblocking ? MSG_DONTWAIT : 0);
      size_t sent = 0, pos = 0, in_block = 0;
      while (sent < total) {
        const size_t want = std::min(block - in_block, total - sent);
        ssize_t n = send(fd[i], buf.data() + pos + in_block, want, fl);
        if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) { waitFor(fd[i], POLLOUT); continue; }
        if (n <= 0) break;
        sent += (size_t)n;
        in_block += (size_t)n;
        if (in_block == block) { in_block = 0; pos = (pos + block) % span; }
      }
    });
  for (auto& t : th) t.join();
  for (int f : fd) close(f);
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  Options o;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    if (a == "--help" || a == "-h") {
      printf("usage: tcpxb_rawsock [--streams 8] [--mb-per-stream 2048] [--block-kb 512] [--nics 4] [--span-mb 0] [--sndbuf-kb 0] "
             "[--nonblocking 0] [--scatter-kb 0]\n");
      return 0;
    }
    if (i + 1 >= argc) { fprintf(stderr, "%s needs a value (see --help)\n", a.c_str()); return 2; }
    const char* v = argv[++i];
    if (a == "--streams") o.streams = atoi(v);
    else if (a == "--mb-per-stream") o.mb = atol(v);
    else if (a == "--block-kb") o.block_kb = atoi(v);
    else if (a == "--nics") o.nics = atoi(v);
    else if (a == "--span-mb") o.span_mb = atol(v);
    else if (a == "--sndbuf-kb") o.sndbuf_kb = atol(v);
    else if (a == "--nonblocking") o.nonblocking = atoi(v);
    else if (a == "--scatter-kb") o.scatter_kb = atoi(v);
    else { fprintf(stderr, "unknown argument %s (see --help)\n", a.c_str()); return 2; }
  }
  if (o.streams < 1 || o.streams > 256 || o.nics < 1 || o.span_mb < 0 || o.scatter_kb < 0) return 2;
  if (o.scatter_kb > 0 && (o.block_kb % o.scatter_kb) != 0) { fprintf(stderr, "--block-kb must be a multiple of --scatter-kb\n"); return 2; }
  int ports[2], go[2];
  if (pipe(ports) != 0 || pipe(go) != 0) return 1;
  fflush(stdout);
  pid_t pid = fork();
  if (pid == 0) _exit(sender(o, ports[0], go[0]));
  int rc = receiver(o, ports[1], go[1]);
  int status = 0;
  waitpid(pid, &status, 0);
  return rc;
}
