// Raw TCP ceiling of this machine: S parallel streams over loopback, one sender and
// one receiver thread per stream in two processes, plain send()/recv() of large
// blocks and nothing else.  The transport cannot beat this number; benchmarks
// report their socket stage as a fraction of it.
//   tcpxb_rawsock [--streams 8] [--mb-per-stream 2048] [--block-kb 512] [--nics 4]
// Prints one JSON line.  Stream i uses address 127.0.0.(1 + i % nics).
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <time.h>
#include <unistd.h>

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
};

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
      std::vector<char> buf(block);
      size_t got = 0;
      while (got < total) {
        ssize_t n = recv(fd[i], buf.data(), block, 0);
        if (n <= 0) break;
        got += (size_t)n;
      }
    });
  for (auto& t : th) t.join();
  const double dt = nowSec() - t0;
  printf("{\"tool\": \"rawsock\", \"streams\": %d, \"block_kb\": %d, \"mb_per_stream\": %ld, \"seconds\": %.4f, \"GBps\": %.3f}\n",
         o.streams, o.block_kb, o.mb, dt, (double)total * o.streams / dt / 1e9);
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
    if (connect(fd[i], (sockaddr*)&a, sizeof a) != 0) return 1;
  }
  char go;
  if (read(go_pipe, &go, 1) != 1) return 1;
  const size_t block = (size_t)o.block_kb << 10;
  const size_t total = (size_t)o.mb << 20;
  std::vector<std::thread> th;
  for (int i = 0; i < o.streams; ++i)
    th.emplace_back([&, i] {
      std::vector<char> buf(block, (char)i);
      size_t sent = 0;
      while (sent < total) {
        ssize_t n = send(fd[i], buf.data(), block < total - sent ? block : total - sent, MSG_NOSIGNAL);
        if (n <= 0) break;
        sent += (size_t)n;
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
      printf("usage: tcpxb_rawsock [--streams 8] [--mb-per-stream 2048] [--block-kb 512] [--nics 4]\n");
      return 0;
    }
    if (i + 1 >= argc) { fprintf(stderr, "%s needs a value (see --help)\n", a.c_str()); return 2; }
    const char* v = argv[++i];
    if (a == "--streams") o.streams = atoi(v);
    else if (a == "--mb-per-stream") o.mb = atol(v);
    else if (a == "--block-kb") o.block_kb = atoi(v);
    else if (a == "--nics") o.nics = atoi(v);
    else { fprintf(stderr, "unknown argument %s (see --help)\n", a.c_str()); return 2; }
  }
  if (o.streams < 1 || o.streams > 256 || o.nics < 1) return 2;
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
