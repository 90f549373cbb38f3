// The kernel ABI of tcpxb/kernels.h, done on the CPU, for the host-only library.
//
// The host-only build (TCPXB_NO_CUDA) has a stand-in device whose memory is host
// memory (see tcpxb/gpu.h).  This file gives that device its "kernels": each entry
// point does, at once and on the calling thread, what the sm_100a kernel of the
// same name does on a stream: the same bounds and alignment checks with the same
// status words, the same arithmetic (bf16 sums formed in fp32 and rounded once to
// nearest-even), release stores for the peer flags and bounded acquire waits.
// "Peers" are plain pointers; tests that run several ranks map one another's
// buffers through shared memory.  The multicast variants store to the local buffer
// and to every peer, which is what a multimem store amounts to.
//
// This is a test double, not a product path: it lets the collective engine and the
// transport's device-memory paths run under the sanitizers on machines without a
// GPU, and it is a second, independent statement of what the kernels compute.
// The reference has no device code and nothing comparable (its receive side ends
// at the scatter list, reference: src/devcomm/nccl/unpack1.cu:52-63).
#ifndef TCPXB_NO_CUDA
#error "kernels_host.cc belongs to the host-only library; CUDA builds use unpack_kernels.cu"
#endif

#include <stdio.h>
#include <string.h>
#include <time.h>

#include "tcpxb/gpu.h"
#include "tcpxb/kernels.h"

namespace {

thread_local char g_err[256] = "";
int fail(int code, const char* what) {
  snprintf(g_err, sizeof g_err, "%s", what);
  return code;
}

uint64_t nowNs() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

constexpr uint64_t kDefaultWaitNs = 2000000000ull;

// First error wins word 0 and 1; word 2 counts every skipped record.
void report(uint32_t* status, uint32_t code, uint32_t index) {
  if (status == nullptr) return;
  uint32_t expected = 0;
  if (__atomic_compare_exchange_n(&status[0], &expected, code, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) status[1] = index;
  __atomic_fetch_add(&status[2], 1u, __ATOMIC_RELAXED);
}

float bf16ToFloat(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t floatToBf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);                      // round to nearest, ties to even
  return (uint16_t)(u >> 16);
}

// out[i] = a[i] + b[i] over n bytes of `dtype` elements; out may alias a or b.
void addInto(uint8_t* out, const uint8_t* a, const uint8_t* b, uint64_t n, int dtype) {
  if (dtype == TCPXB_BF16) {
    for (uint64_t i = 0; i + 2 <= n; i += 2) {
      uint16_t x, y;
      memcpy(&x, a + i, 2);
      memcpy(&y, b + i, 2);
      const uint16_t r = floatToBf16(bf16ToFloat(x) + bf16ToFloat(y));
      memcpy(out + i, &r, 2);
    }
  } else {
    for (uint64_t i = 0; i + 4 <= n; i += 4) {
      float x, y;
      memcpy(&x, a + i, 4);
      memcpy(&y, b + i, 4);
      const float r = x + y;
      memcpy(out + i, &r, 4);
    }
  }
}

struct Job {
  const uint8_t* pool;
  uint64_t pool_bytes;
  const uint8_t* acc;  // null = copy
  uint8_t* dst;
  uint64_t dst_bytes;
  void* const* peers;
  int npeers;
  const tcpxbLoadMeta* descs;
  uint32_t count;
  int dtype;
  bool add_into_peers;  // the L2 form of the fused reduce: every buffer keeps its own sum
  uint32_t* status;
  const tcpxbUnpackOpts* opts;
};

int validate(const Job& j) {
  if (j.count == 0) return TCPXB_K_OK;
  if (j.pool == nullptr || j.dst == nullptr || j.descs == nullptr) return fail(TCPXB_K_INVALID, "null pool, destination or descriptor array");
  if (j.npeers < 0 || j.npeers > TCPXB_MAX_PEERS) return fail(TCPXB_K_INVALID, "too many peers");
  if (j.npeers > 0 && j.peers == nullptr) return fail(TCPXB_K_INVALID, "null peer array");
  for (int i = 0; i < j.npeers; ++i)
    if (j.peers[i] == nullptr) return fail(TCPXB_K_INVALID, "null peer pointer");
  if (j.acc != nullptr && j.dtype != TCPXB_BF16 && j.dtype != TCPXB_F32) return fail(TCPXB_K_INVALID, "reduce needs bf16 or f32");
  return TCPXB_K_OK;
}

int run(const Job& j) {
  const int v = validate(j);
  if (v != TCPXB_K_OK) return v;
  const uint32_t* ready = j.opts ? j.opts->ready_count : nullptr;
  const uint64_t wait_ns = j.opts && j.opts->wait_ns ? j.opts->wait_ns : kDefaultWaitNs;
  bool errors = false;
  const uint32_t count = tcpxb::gpu::standinMovesData() ? j.count : 0;  // timing mode: no data is moved
  for (uint32_t i = 0; i < count; ++i) {
    if (ready != nullptr) {
      // streaming: record i exists once the producer's counter has passed it; the limit
      // bounds how long the producer may stay silent, and after a time-out nothing further is attempted
      uint64_t t0 = nowNs();
      uint32_t seen = __atomic_load_n(ready, __ATOMIC_ACQUIRE);
      bool timed_out = false;
      while (seen <= i) {
        const uint32_t now_seen = __atomic_load_n(ready, __ATOMIC_ACQUIRE);
        if (now_seen != seen) { seen = now_seen; t0 = nowNs(); continue; }
        if (nowNs() - t0 > wait_ns) { timed_out = true; break; }
      }
      if (timed_out) { report(j.status, TCPXB_ST_TIMEOUT, i); errors = true; break; }
    }
    const tcpxbLoadMeta m = j.descs[i];
    if ((uint64_t)m.src_off + m.len > j.pool_bytes || m.dst_off + m.len > j.dst_bytes || m.dst_off + m.len < m.dst_off) {
      report(j.status, TCPXB_ST_BOUNDS, i);
      errors = true;
      continue;
    }
    const uint8_t* src = j.pool + m.src_off;
    uint8_t* d = j.dst + m.dst_off;
    if (j.acc == nullptr) {
      memcpy(d, src, m.len);
      for (int p = 0; p < j.npeers; ++p) memcpy(static_cast<uint8_t*>(j.peers[p]) + m.dst_off, src, m.len);
      continue;
    }
    const uint32_t es = j.dtype == TCPXB_BF16 ? 2 : 4;
    const uint8_t* a = j.acc + m.dst_off;
    if ((((uintptr_t)src | (uintptr_t)d | (uintptr_t)a | m.len) & (es - 1)) != 0) {
      report(j.status, TCPXB_ST_ALIGN, i);
      errors = true;
      continue;
    }
    if (j.add_into_peers) {
      for (int p = 0; p < j.npeers; ++p) {
        uint8_t* q = static_cast<uint8_t*>(j.peers[p]) + m.dst_off;
        addInto(q, q, src, m.len, j.dtype);
      }
      addInto(d, a, src, m.len, j.dtype);
    } else {
      addInto(d, a, src, m.len, j.dtype);
      for (int p = 0; p < j.npeers; ++p) memcpy(static_cast<uint8_t*>(j.peers[p]) + m.dst_off, d, m.len);
    }
  }
  if (j.opts != nullptr && j.opts->flag_value != 0 && !errors) {
    // "every store of this launch has completed": trivially true here.  A launch that
    // recorded an error publishes nothing; the peers' bounded waits then run out.
    for (int p = 0; p < TCPXB_MAX_PEERS; ++p)
      if (j.opts->peer_flags[p] != nullptr) __atomic_store_n(j.opts->peer_flags[p], j.opts->flag_value, __ATOMIC_RELEASE);
  }
  return TCPXB_K_OK;
}

}  // namespace

extern "C" {

const char* tcpxb_kernel_last_error(void) { return g_err; }
int tcpxb_kernels_preload(void) { return TCPXB_K_OK; }

int tcpxb_unpack_copy(const void* pool, uint64_t pool_bytes, void* dst, uint64_t dst_bytes, const tcpxbLoadMeta* descs,
                      uint32_t count, uint32_t* status, const tcpxbUnpackOpts* opts, void*) {
  return run({static_cast<const uint8_t*>(pool), pool_bytes, nullptr, static_cast<uint8_t*>(dst), dst_bytes, nullptr, 0, descs, count,
              TCPXB_U8, false, status, opts});
}

int tcpxb_unpack_reduce(const void* pool, uint64_t pool_bytes, const void* acc, void* dst, uint64_t dst_bytes,
                        const tcpxbLoadMeta* descs, uint32_t count, int dtype, int impl, uint32_t* status,
                        const tcpxbUnpackOpts* opts, void*) {
  if (impl == TCPXB_REDUCE_L2 && acc != nullptr && acc != dst) return fail(TCPXB_K_INVALID, "the L2 reduce is always in place");
  if (dtype != TCPXB_BF16 && dtype != TCPXB_F32) return fail(TCPXB_K_INVALID, "reduce needs bf16 or f32");
  const void* a = acc ? acc : dst;
  return run({static_cast<const uint8_t*>(pool), pool_bytes, static_cast<const uint8_t*>(a), static_cast<uint8_t*>(dst), dst_bytes,
              nullptr, 0, descs, count, dtype, false, status, opts});
}

int tcpxb_unpack_fanout(const void* pool, uint64_t pool_bytes, void* dst, uint64_t dst_bytes, void* const* peers, int npeers,
                        const tcpxbLoadMeta* descs, uint32_t count, uint32_t* status, const tcpxbUnpackOpts* opts, void*) {
  return run({static_cast<const uint8_t*>(pool), pool_bytes, nullptr, static_cast<uint8_t*>(dst), dst_bytes, peers, npeers, descs,
              count, TCPXB_U8, false, status, opts});
}

int tcpxb_unpack_reduce_fanout(const void* pool, uint64_t pool_bytes, const void* acc, void* dst, uint64_t dst_bytes,
                               void* const* peers, int npeers, const tcpxbLoadMeta* descs, uint32_t count, int dtype, int impl,
                               uint32_t* status, const tcpxbUnpackOpts* opts, void*) {
  if (impl == TCPXB_REDUCE_L2 && acc != nullptr && acc != dst) return fail(TCPXB_K_INVALID, "the L2 reduce is always in place");
  if (dtype != TCPXB_BF16 && dtype != TCPXB_F32) return fail(TCPXB_K_INVALID, "reduce needs bf16 or f32");
  const void* a = acc ? acc : dst;
  return run({static_cast<const uint8_t*>(pool), pool_bytes, static_cast<const uint8_t*>(a), static_cast<uint8_t*>(dst), dst_bytes,
              peers, npeers, descs, count, dtype, impl == TCPXB_REDUCE_L2, status, opts});
}

int tcpxb_unpack_fanout_nvls(const void* pool, uint64_t pool_bytes, void* dst, void* /*mc_dst*/, uint64_t dst_bytes,
                             void* const* peers, int npeers, const tcpxbLoadMeta* descs, uint32_t count, uint32_t* status,
                             const tcpxbUnpackOpts* opts, void* stream) {
  return tcpxb_unpack_fanout(pool, pool_bytes, dst, dst_bytes, peers, npeers, descs, count, status, opts, stream);
}

int tcpxb_unpack_reduce_fanout_nvls(const void* pool, uint64_t pool_bytes, const void* acc, void* dst, void* /*mc_dst*/,
                                    uint64_t dst_bytes, void* const* peers, int npeers, const tcpxbLoadMeta* descs,
                                    uint32_t count, int dtype, uint32_t* status, const tcpxbUnpackOpts* opts, void* stream) {
  return tcpxb_unpack_reduce_fanout(pool, pool_bytes, acc, dst, dst_bytes, peers, npeers, descs, count, dtype, TCPXB_REDUCE_SM,
                                    status, opts, stream);
}

int tcpxb_wait_flags(const uint32_t* flags, int n, uint32_t value, uint64_t wait_ns, uint32_t* status, void*) {
  if (flags == nullptr || n < 0) return fail(TCPXB_K_INVALID, "null flag array");
  const uint64_t limit = wait_ns ? wait_ns : kDefaultWaitNs;
  const uint64_t t0 = nowNs();
  for (int i = 0; i < n; ++i) {
    for (;;) {
      const uint32_t v = __atomic_load_n(&flags[i], __ATOMIC_ACQUIRE);
      if ((int32_t)(v - value) >= 0) break;
      if (nowNs() - t0 > limit) { report(status, TCPXB_ST_TIMEOUT, (uint32_t)i); break; }
    }
  }
  return TCPXB_K_OK;
}

int tcpxb_signal_flags(uint32_t* const* peer_flags, int n, uint32_t value, void*) {
  if (peer_flags == nullptr || n < 0 || n > TCPXB_MAX_PEERS + 1) return fail(TCPXB_K_INVALID, "bad flag list");
  for (int i = 0; i < n; ++i)
    if (peer_flags[i] != nullptr) __atomic_store_n(peer_flags[i], value, __ATOMIC_RELEASE);
  return TCPXB_K_OK;
}

int tcpxb_peer_reduce(void* out, void* const* srcs, int nsrcs, uint64_t shard_off, uint64_t bytes, int dtype, void*) {
  if (out == nullptr || srcs == nullptr || nsrcs < 1 || nsrcs > TCPXB_MAX_PEERS) return fail(TCPXB_K_INVALID, "bad source list");
  if (dtype != TCPXB_BF16 && dtype != TCPXB_F32) return fail(TCPXB_K_INVALID, "reduce needs bf16 or f32");
  if ((bytes | shard_off) & 15) return fail(TCPXB_K_INVALID, "shard offset and size must be multiples of 16 bytes");
  uint8_t* o = static_cast<uint8_t*>(out);
  if (!tcpxb::gpu::standinMovesData()) return TCPXB_K_OK;  // timing mode
  if (dtype == TCPXB_BF16) {
    // one rounding, after all addends are summed in fp32
    for (uint64_t i = 0; i < bytes; i += 2) {
      float sum = 0.f;
      for (int r = 0; r < nsrcs; ++r) {
        uint16_t x;
        memcpy(&x, static_cast<const uint8_t*>(srcs[r]) + shard_off + i, 2);
        sum += bf16ToFloat(x);
      }
      const uint16_t h = floatToBf16(sum);
      memcpy(o + i, &h, 2);
    }
  } else {
    for (uint64_t i = 0; i < bytes; i += 4) {
      float sum = 0.f;
      for (int r = 0; r < nsrcs; ++r) {
        float x;
        memcpy(&x, static_cast<const uint8_t*>(srcs[r]) + shard_off + i, 4);
        sum += x;
      }
      memcpy(o + i, &sum, 4);
    }
  }
  return TCPXB_K_OK;
}

size_t tcpxb_checksum_scratch_bytes(void) { return 16; }

static int checksumWords(const void* buf, uint64_t bytes, uint64_t* out) {
  if (out == nullptr || (buf == nullptr && bytes != 0)) return fail(TCPXB_K_INVALID, "null buffer or output");
  if (reinterpret_cast<uintptr_t>(buf) & 3) return fail(TCPXB_K_INVALID, "checksum buffer must be 4-byte aligned");
  const uint8_t* p = static_cast<const uint8_t*>(buf);
  uint64_t sum = 0;
  uint64_t i = 0;
  for (; i + 4 <= bytes; i += 4) {
    uint32_t w;
    memcpy(&w, p + i, 4);
    sum += w;
  }
  if (i < bytes) {
    uint32_t w = 0;
    memcpy(&w, p + i, bytes - i);
    sum += w;
  }
  *out = sum;
  return TCPXB_K_OK;
}

int tcpxb_checksum(const void* buf, uint64_t bytes, uint64_t* out, void* partials, void*) {
  if (partials == nullptr) return fail(TCPXB_K_INVALID, "null buffer, output or scratch");
  return checksumWords(buf, bytes, out);
}

int tcpxb_checksum_noalloc(const void* buf, uint64_t bytes, uint64_t* out, void*) {
  if (bytes > TCPXB_CHECKSUM_NOALLOC_MAX_BYTES) return fail(TCPXB_K_TOO_LARGE, "tcpxb_checksum_noalloc handles at most 16 GiB per call");
  return checksumWords(buf, bytes, out);
}

}  // extern "C"
