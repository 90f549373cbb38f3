// sm_100a unpack kernels: reassemble scattered rx page fragments on the GPU.
//
// One kernel template covers the four products:
//   K1  unpack_copy            pool fragment -> dst
//   K2  unpack_reduce          dst = acc + pool fragment (bf16 with fp32 add, or fp32)
//   K3  unpack_fanout          K1 + the same fragment stored to every local peer GPU
//   K3r unpack_reduce_fanout   K2 + the reduced fragment stored to every local peer GPU
//
// The reference has no counterpart: with it, NCCL's collective kernels walk the
// scatter list (reference: src/net_tcpx.cc:739-740 declares NCCL_NET_DEVICE_UNPACK;
// src/sock/tcpx.h:136-228 builds the list).  The list format is kept.
//
// Structure.  Persistent grid, one CTA per SM, twelve warps per CTA.  Each warp owns
// a private ring of D shared-memory slots and D mbarriers and walks descriptors
// gw, gw+G, gw+2G, ... (G = warps in the grid).  Per fragment, one elected lane
// issues a bulk-async copy global -> shared (cp.async.bulk, completion counted in
// bytes on the slot's mbarrier); when it lands, the warp optionally adds the
// accumulator tile (also bulk-loaded), and the elected lane issues bulk-async
// stores shared -> global to the local destination and to each peer's mapping.
// D fragments are in flight per warp (4 for the copy, 2 fragment + accumulator
// pairs for the reduce), so an SM keeps 192 KB of loads in the air, which is what
// HBM3e needs to stay busy with 4 KB transfers.  Twelve warps of depth 4 / 2
// measured 2 - 3 % faster on the fused reduce than eight warps of depth 6 / 3.
// Fragments whose addresses are not 16-byte aligned, or that are longer than a
// slot, take a warp-cooperative ld/st path; ragged tails (< 16 B) likewise.
//
// Every wait is bounded: on expiry the kernel records TCPXB_ST_TIMEOUT in the
// status block, stops issuing, waits only for the loads already in flight and
// returns; it never traps and never spins forever.  A launch that recorded any error
// does not publish its fan-out completion flag: the peers then run into their own
// bounded flag wait instead of taking partly written output for complete.
// No load in this file is a cluster-wide one; peers are reached by stores only.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "tcpxb/kernels.h"

namespace {

#ifndef TCPXB_WARPS
#define TCPXB_WARPS 12
#endif
#ifndef TCPXB_DEPTH_COPY
#define TCPXB_DEPTH_COPY 4
#endif
#ifndef TCPXB_DEPTH_REDUCE
#define TCPXB_DEPTH_REDUCE 2
#endif
constexpr int kWarps = TCPXB_WARPS;
constexpr int kThreads = kWarps * 32;
constexpr int kSlot = TCPXB_FRAG_BYTES;
constexpr uint64_t kDefaultWaitNs = 2000000000ull;

enum FanMode { FAN_NONE = 0, FAN_PEER = 1, FAN_NVLS = 2 };

struct UnpackParams {
  const uint8_t* pool;
  uint64_t pool_bytes;
  uint8_t* dst;
  uint64_t dst_bytes;
  const uint8_t* acc;
  uint8_t* mc_dst;
  const tcpxbLoadMeta* descs;
  uint32_t count;
  int npeers;
  uint8_t* peers[TCPXB_MAX_PEERS];
  uint32_t* peer_flags[TCPXB_MAX_PEERS];
  uint32_t flag_value;
  uint32_t* ticket;
  uint32_t* status;
  const uint32_t* ready;
  uint64_t wait_ns;
};

struct SlotInfo {
  uint32_t src_off;
  uint32_t len;
  uint64_t dst_off;
  uint32_t bulk;   // bytes moved by the bulk path (multiple of 16, may be 0)
  uint32_t pad[3];
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst_smem),
      "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
      : "memory");
}
// The same load with an L2 eviction-priority hint: rx pool pages are read exactly once.
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst_smem, const void* src, uint32_t bytes,
                                              uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
          "r"(dst_smem),
      "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                   __cvta_generic_to_global(dst)),
               "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_red_bf16(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile(
      "cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.bf16 [%0], [%1], %2;" ::"l"(
          __cvta_generic_to_global(dst)),
      "r"(src_smem), "r"(bytes)
      : "memory");
}
__device__ __forceinline__ void bulk_red_f32(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(
                   __cvta_generic_to_global(dst)),
               "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_v4(void* mc, uint4 v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ void multimem_red_bf16x8(void* mc, uint4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void multimem_red_f32x4(void* mc, uint4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

__device__ __forceinline__ void report(uint32_t* status, uint32_t code, uint32_t index) {
  if (status == nullptr) return;
  if (atomicCAS(&status[0], 0u, code) == 0u) status[1] = index;
  atomicAdd(&status[2], 1u);
}

// Bounded mbarrier wait: every lane polls, so every lane observes the phase and
// with it the bytes the async proxy wrote.  Returns false when time ran out.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 0xff) == 0xff) {
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
}

// ------------------------------------------------------------ element helpers
__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
  // bf16 -> fp32 is a 16-bit shift; add in fp32; round to nearest even once.
  float a0 = __uint_as_float(a << 16), a1 = __uint_as_float(a & 0xffff0000u);
  float b0 = __uint_as_float(b << 16), b1 = __uint_as_float(b & 0xffff0000u);
  __nv_bfloat162 r = __floats2bfloat162_rn(a0 + b0, a1 + b1);
  return *reinterpret_cast<uint32_t*>(&r);
}
template <int RED>
__device__ __forceinline__ uint4 add_vec(uint4 a, uint4 b) {
  uint4 r;
  if (RED == TCPXB_BF16) {
    r.x = add_bf16x2(a.x, b.x); r.y = add_bf16x2(a.y, b.y);
    r.z = add_bf16x2(a.z, b.z); r.w = add_bf16x2(a.w, b.w);
  } else {
    r.x = __float_as_uint(__uint_as_float(a.x) + __uint_as_float(b.x));
    r.y = __float_as_uint(__uint_as_float(a.y) + __uint_as_float(b.y));
    r.z = __float_as_uint(__uint_as_float(a.z) + __uint_as_float(b.z));
    r.w = __float_as_uint(__uint_as_float(a.w) + __uint_as_float(b.w));
  }
  return r;
}

template <typename T>
__device__ __forceinline__ void store_all(uint8_t* dst, const UnpackParams& p, int fan,
                                          uint64_t off, T v) {
  *reinterpret_cast<T*>(dst + off) = v;
  if (fan) {
    for (int i = 0; i < p.npeers; ++i) *reinterpret_cast<T*>(p.peers[i] + off) = v;
  }
}

template <typename T>
__device__ __forceinline__ void copy_units(const uint8_t* src, const UnpackParams& p, int fan,
                                           uint64_t dst_off, uint32_t n_units, int lane) {
  for (uint32_t i = lane; i < n_units; i += 32) {
    T v = *reinterpret_cast<const T*>(src + (uint64_t)i * sizeof(T));
    store_all<T>(p.dst, p, fan, dst_off + (uint64_t)i * sizeof(T), v);
  }
}

// Warp-cooperative generic path for `n` bytes of any alignment: plain loads and
// stores, widest unit the common alignment of source and destination allows.
template <int RED, bool L2RED, int FAN>
__device__ void warp_generic(const UnpackParams& p, uint32_t src_off, uint64_t dst_off, uint32_t n,
                             uint32_t desc_index, int lane, uint32_t* cta_err) {
  if (n == 0) return;
  const uint8_t* src = p.pool + src_off;
  const int fan = (FAN != FAN_NONE);
  if (RED == TCPXB_U8) {
    uintptr_t s = reinterpret_cast<uintptr_t>(src);
    uintptr_t d = reinterpret_cast<uintptr_t>(p.dst + dst_off);
    if (((s ^ d) & 15) == 0) {
      uint32_t head = static_cast<uint32_t>((16 - (s & 15)) & 15);
      if (head > n) head = n;
      copy_units<uint8_t>(src, p, fan, dst_off, head, lane);
      uint32_t body = (n - head) >> 4;
      copy_units<uint4>(src + head, p, fan, dst_off + head, body, lane);
      uint32_t done = head + (body << 4);
      copy_units<uint8_t>(src + done, p, fan, dst_off + done, n - done, lane);
    } else {
      uint32_t a = static_cast<uint32_t>((s | d) & 15);
      uint32_t w = a & (~a + 1);  // lowest set bit: 1, 2, 4 or 8
      uint32_t units, done;
      if (w == 8) { units = n >> 3; copy_units<uint2>(src, p, fan, dst_off, units, lane); done = units << 3; }
      else if (w == 4) { units = n >> 2; copy_units<uint32_t>(src, p, fan, dst_off, units, lane); done = units << 2; }
      else if (w == 2) { units = n >> 1; copy_units<uint16_t>(src, p, fan, dst_off, units, lane); done = units << 1; }
      else { done = 0; }
      copy_units<uint8_t>(src + done, p, fan, dst_off + done, n - done, lane);
    }
  } else {
    constexpr uint32_t es = (RED == TCPXB_BF16) ? 2 : 4;
    uintptr_t s = reinterpret_cast<uintptr_t>(src);
    uintptr_t d = reinterpret_cast<uintptr_t>(p.dst + dst_off);
    uintptr_t a = reinterpret_cast<uintptr_t>(p.acc + dst_off);
    if (((s | d | a | n) & (es - 1)) != 0) {
      if (lane == 0) { report(p.status, TCPXB_ST_ALIGN, desc_index); atomicOr(cta_err, 1u); }
      return;
    }
    uint32_t elems = n / es;
    for (uint32_t i = lane; i < elems; i += 32) {
      uint64_t off = dst_off + (uint64_t)i * es;
      if (RED == TCPXB_BF16) {
        float x = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(src + (uint64_t)i * es));
        if (L2RED) {
          // reduce-into-all form: each buffer adds the fragment to its own value
          __nv_bfloat16* q = reinterpret_cast<__nv_bfloat16*>(p.dst + off);
          *q = __float2bfloat16_rn(__bfloat162float(*q) + x);
          if (fan) for (int r = 0; r < p.npeers; ++r) {
            __nv_bfloat16* pq = reinterpret_cast<__nv_bfloat16*>(p.peers[r] + off);
            *pq = __float2bfloat16_rn(__bfloat162float(*pq) + x);
          }
        } else {
          float y = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p.acc + off));
          store_all<__nv_bfloat16>(p.dst, p, fan, off, __float2bfloat16_rn(x + y));
        }
      } else {
        float x = *reinterpret_cast<const float*>(src + (uint64_t)i * es);
        if (L2RED) {
          float* q = reinterpret_cast<float*>(p.dst + off);
          *q = *q + x;
          if (fan) for (int r = 0; r < p.npeers; ++r) {
            float* pq = reinterpret_cast<float*>(p.peers[r] + off);
            *pq = *pq + x;
          }
        } else {
          float y = *reinterpret_cast<const float*>(p.acc + off);
          store_all<float>(p.dst, p, fan, off, x + y);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ the kernel
template <int RED, bool L2RED, int FAN>
struct Cfg {
  static constexpr bool kAccSlot = (RED != TCPXB_U8) && !L2RED;
  static constexpr int kStride = kAccSlot ? 2 * kSlot : kSlot;
  static constexpr int kDepth = kAccSlot ? TCPXB_DEPTH_REDUCE : TCPXB_DEPTH_COPY;
  static_assert(kWarps * kDepth * kStride + kWarps * kDepth * 40 <= 227 * 1024, "slot rings must fit one CTA's shared memory");
  static constexpr int kDataBytes = kWarps * kDepth * kStride;
  static constexpr int kSmemBytes = kDataBytes + kWarps * kDepth * (8 + (int)sizeof(SlotInfo));
};

template <int RED, bool L2RED, int FAN>
__global__ void __launch_bounds__(kThreads, 1)
unpack_kernel(const __grid_constant__ UnpackParams p) {
  using C = Cfg<RED, L2RED, FAN>;
  constexpr int D = C::kDepth;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* wbuf = smem + warp * D * C::kStride;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kDataBytes) + warp * D;
  SlotInfo* infos = reinterpret_cast<SlotInfo*>(smem + C::kDataBytes + kWarps * D * 8) + warp * D;

  // Programmatic dependent launch, both roles.  As the earlier kernel: let a dependent
  // launch be scheduled from now on (its CTAs still need this one's shared memory to
  // be released before they fit).  As the later kernel: everything up to the wait
  // below touches only this CTA's shared memory; the wait returns when the previous
  // kernel of the stream has completed and its writes are visible (at once when the
  // launch did not ask for an early start).
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ uint32_t cta_err;  // any warp of this CTA recorded an error
  if (threadIdx.x == 0) cta_err = 0;
  if (lane == 0) {
    for (int s = 0; s < D; ++s) mbar_init(smem_u32(&bars[s]), 1);
    fence_mbar_init();
  }
  __syncthreads();
  asm volatile("griddepcontrol.wait;" ::: "memory");
  auto record = [&](uint32_t code, uint32_t index) {  // one lane calls this
    report(p.status, code, index);
    atomicOr(&cta_err, 1u);
  };

  // Consecutive descriptors go to different SMs first, then to different warps.
  const uint32_t G = gridDim.x * kWarps;
  const uint32_t gw = warp * gridDim.x + blockIdx.x;
  const uint32_t n = (gw < p.count) ? (p.count - gw + G - 1) / G : 0;
  const uint64_t wait_ns = p.wait_ns ? p.wait_ns : kDefaultWaitNs;

  const uint64_t pool_policy = policy_evict_first();
  uint32_t cached_blk = 0xffffffffu;
  uint4 cached = make_uint4(0, 0, 0, 0);
  uint32_t ready_seen = 0;
  uint64_t ready_t0 = 0;
  bool dead = false;  // a bounded wait ran out: stop issuing, drain what is in flight
  uint32_t issued = 0;  // local iterations whose loads were issued

  // Issue the loads of local iteration k into slot k % D.  Warp-uniform.
  auto issue = [&](uint32_t k) {
    const uint32_t slot = k % D;
    const uint32_t idx = gw + k * G;
    issued = k + 1;
    uint32_t so, ln, dlo, dhi;
    if (p.ready != nullptr) {
      // Streaming: descriptor idx exists once the producer's counter passed it.
      if (lane == 0 && ready_seen <= idx) {
        for (uint32_t spin = 0;; ++spin) {
          const uint32_t before = ready_seen;
          ready_seen = ld_acquire_sys(p.ready);
          if (ready_seen != before) ready_t0 = 0;  // the producer moved: the limit bounds its silence, not the launch
          if (ready_seen > idx) break;
          if ((spin & 0x3f) == 0x3f) {
            uint64_t now = globaltimer_ns();
            if (ready_t0 == 0) ready_t0 = now;
            else if (now - ready_t0 > wait_ns) break;
          }
          __nanosleep(200);
        }
      }
      ready_seen = __shfl_sync(0xffffffffu, ready_seen, 0);
      uint4 d = make_uint4(0, 0, 0, 0);
      if (ready_seen <= idx) {
        if (lane == 0) record(TCPXB_ST_TIMEOUT, idx);
        dead = true;
      } else if (lane == 0) {
        d = ld_volatile_v4(&p.descs[idx]);
      }
      so = __shfl_sync(0xffffffffu, d.x, 0);
      ln = __shfl_sync(0xffffffffu, d.y, 0);
      dlo = __shfl_sync(0xffffffffu, d.z, 0);
      dhi = __shfl_sync(0xffffffffu, d.w, 0);
    } else {
      const uint32_t blk = k >> 5;
      if (blk != cached_blk) {
        const uint32_t kk = (blk << 5) + lane;
        if (kk < n) cached = __ldg(reinterpret_cast<const uint4*>(&p.descs[gw + (uint64_t)kk * G]));
        cached_blk = blk;
      }
      so = __shfl_sync(0xffffffffu, cached.x, k & 31);
      ln = __shfl_sync(0xffffffffu, cached.y, k & 31);
      dlo = __shfl_sync(0xffffffffu, cached.z, k & 31);
      dhi = __shfl_sync(0xffffffffu, cached.w, k & 31);
    }
    const uint64_t dof = (static_cast<uint64_t>(dhi) << 32) | dlo;
    if (dead) ln = 0;
    if ((uint64_t)so + ln > p.pool_bytes || dof + ln > p.dst_bytes || dof + ln < dof) {
      if (lane == 0) record(TCPXB_ST_BOUNDS, idx);
      ln = 0;
    }
    uintptr_t al = reinterpret_cast<uintptr_t>(p.pool + so) | reinterpret_cast<uintptr_t>(p.dst + dof);
    if (C::kAccSlot) al |= reinterpret_cast<uintptr_t>(p.acc + dof);
    const uint32_t bulk = ((al & 15) == 0 && ln <= (uint32_t)kSlot) ? (ln & ~15u) : 0u;
    if (lane == 0) {
      infos[slot].src_off = so;
      infos[slot].len = ln;
      infos[slot].dst_off = dof;
      infos[slot].bulk = bulk;
      const uint32_t bar = smem_u32(&bars[slot]);
      if (bulk) {
        mbar_expect_tx(bar, C::kAccSlot ? 2 * bulk : bulk);
        bulk_g2s_hint(smem_u32(wbuf + slot * C::kStride), p.pool + so, bulk, bar, pool_policy);
        if (C::kAccSlot) bulk_g2s(smem_u32(wbuf + slot * C::kStride + kSlot), p.acc + dof, bulk, bar);
      } else {
        mbar_arrive(bar);
      }
    }
    __syncwarp();
  };

  const uint32_t pro = n < (uint32_t)D ? n : (uint32_t)D;
  for (uint32_t k = 0; k < pro && !dead; ++k) issue(k);  // a wait that ran out is not repeated for the next slot

  for (uint32_t k = 0; k < n; ++k) {
    // After a time-out only the loads already issued are waited for (at most D of
    // them, each with a shortened limit): the drain takes about one wait, not n of them.
    if (dead && k >= issued) break;
    const uint32_t slot = k % D;
    const uint32_t parity = (k / D) & 1;
    const uint32_t bar = smem_u32(&bars[slot]);
    if (!mbar_wait_bounded(bar, parity, dead ? (wait_ns >> 3) + 1 : wait_ns)) {
      if (lane == 0 && !dead) record(TCPXB_ST_TIMEOUT, gw + k * G);
      dead = true;
    }
    dead = __any_sync(0xffffffffu, dead);
    const SlotInfo info = infos[slot];
    uint8_t* sfrag = wbuf + slot * C::kStride;
    uint8_t* sout = sfrag;
    if (info.bulk && !dead) {
      if (C::kAccSlot) {
        sout = sfrag + kSlot;
        const uint32_t vecs = info.bulk >> 4;
        for (uint32_t i = lane; i < vecs; i += 32) {
          uint4 a = *reinterpret_cast<const uint4*>(sfrag + (i << 4));
          uint4 b = *reinterpret_cast<const uint4*>(sout + (i << 4));
          *reinterpret_cast<uint4*>(sout + (i << 4)) = add_vec<RED>(b, a);
        }
        if (FAN != FAN_NVLS) fence_proxy_async_smem();
        __syncwarp();
      }
      if (FAN == FAN_NVLS) {
        // One multimem instruction per 16 B reaches every GPU of the group,
        // this one included, through the switch.
        const uint32_t vecs = info.bulk >> 4;
        for (uint32_t i = lane; i < vecs; i += 32) {
          uint4 v = *reinterpret_cast<const uint4*>(sout + (i << 4));
          void* mc = p.mc_dst + info.dst_off + (i << 4);
          if (L2RED) {
            if (RED == TCPXB_BF16) multimem_red_bf16x8(mc, v);
            else multimem_red_f32x4(mc, v);
          } else {
            multimem_st_v4(mc, v);
          }
        }
        __syncwarp();
      } else if (lane == 0) {
        const uint32_t s = smem_u32(sout);
        if (L2RED) {
          if (RED == TCPXB_BF16) bulk_red_bf16(p.dst + info.dst_off, s, info.bulk);
          else bulk_red_f32(p.dst + info.dst_off, s, info.bulk);
          if (FAN == FAN_PEER) {
            for (int r = 0; r < p.npeers; ++r) {
              if (RED == TCPXB_BF16) bulk_red_bf16(p.peers[r] + info.dst_off, s, info.bulk);
              else bulk_red_f32(p.peers[r] + info.dst_off, s, info.bulk);
            }
          }
        } else {
          bulk_s2g(p.dst + info.dst_off, s, info.bulk);
          if (FAN == FAN_PEER) {
            for (int r = 0; r < p.npeers; ++r) bulk_s2g(p.peers[r] + info.dst_off, s, info.bulk);
          }
        }
      }
    }
    // An (often empty) group per iteration keeps "all but the newest group" equal
    // to "every store of the iterations before this one".
    if (lane == 0) bulk_commit();
    if (info.len > info.bulk && !dead) {
      warp_generic<RED, L2RED, FAN>(p, info.src_off + info.bulk, info.dst_off + info.bulk,
                                    info.len - info.bulk, gw + k * G, lane, &cta_err);
    }
    // Refill the slot of the previous iteration: its store has had one iteration
    // to read shared memory, so this wait rarely blocks.
    if (k >= 1 && (k - 1) + D < n && !dead) {
      if (lane == 0) bulk_wait_read<1>();
      __syncwarp();
      issue((k - 1) + D);
    }
  }
  if (lane == 0) bulk_wait_all();

  if (FAN != FAN_NONE && p.flag_value != 0 && p.ticket != nullptr) {
    // Publish completion to the peers once every CTA's stores are done.
    // The ticket counts CTAs in its low half and CTAs with errors in its high half.
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const uint32_t mine = 1u + (cta_err ? 0x10000u : 0u);
      const uint32_t t = atomicAdd(p.ticket, mine) + mine;
      if ((t & 0xffffu) == gridDim.x) {
        *p.ticket = 0;
        __threadfence_system();
        if ((t >> 16) == 0) {
          for (int r = 0; r < TCPXB_MAX_PEERS; ++r) {
            if (p.peer_flags[r] != nullptr) st_release_sys(p.peer_flags[r], p.flag_value);
          }
        }
      }
    }
  }
}

// Bounded wait for peer completion flags; one warp, lane i watches flags[i].
__global__ void wait_flags_kernel(const uint32_t* flags, int n, uint32_t value, uint64_t wait_ns,
                                  uint32_t* status) {
  const int i = threadIdx.x;
  if (i >= n) return;
  uint64_t t0 = globaltimer_ns();
  for (;;) {
    uint32_t v = ld_acquire_sys(&flags[i]);
    if ((int32_t)(v - value) >= 0) return;
    if (globaltimer_ns() - t0 > wait_ns) {
      report(status, TCPXB_ST_TIMEOUT, (uint32_t)i);
      return;
    }
    __nanosleep(100);
  }
}

struct SignalParams {
  uint32_t* flags[TCPXB_MAX_PEERS + 1];
  int n;
  uint32_t value;
};
__global__ void signal_flags_kernel(const __grid_constant__ SignalParams p) {
  const int i = threadIdx.x;
  if (i < p.n && p.flags[i] != nullptr) {
    __threadfence_system();
    st_release_sys(p.flags[i], p.value);
  }
}

// out[i] = sum_r srcs[r][shard_off + i]; 16 B per thread per step, fp32 adds.
struct PeerReduceParams {
  const uint8_t* srcs[TCPXB_MAX_PEERS + 1];
  int nsrcs;
  uint8_t* out;
  uint64_t shard_off;
  uint64_t vecs;
};
template <int RED>
__global__ void __launch_bounds__(256) peer_reduce_kernel(const __grid_constant__ PeerReduceParams p) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.vecs; i += stride) {
    const uint64_t off = p.shard_off + (i << 4);
    uint4 v[TCPXB_MAX_PEERS + 1];
#pragma unroll
    for (int r = 0; r < TCPXB_MAX_PEERS + 1; ++r) {
      if (r < p.nsrcs) v[r] = *reinterpret_cast<const uint4*>(p.srcs[r] + off);
    }
    if (RED == TCPXB_BF16) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int r = 0; r < TCPXB_MAX_PEERS + 1; ++r) {
        if (r < p.nsrcs) {
          const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] += __uint_as_float(w[j] << 16);
            acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
          }
        }
      }
      uint4 o;
      __nv_bfloat162 t;
      t = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&t);
      t = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&t);
      t = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&t);
      t = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&t);
      *reinterpret_cast<uint4*>(p.out + (i << 4)) = o;
    } else {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < TCPXB_MAX_PEERS + 1; ++r) {
        if (r < p.nsrcs) {
          acc.x += __uint_as_float(v[r].x); acc.y += __uint_as_float(v[r].y);
          acc.z += __uint_as_float(v[r].z); acc.w += __uint_as_float(v[r].w);
        }
      }
      *reinterpret_cast<float4*>(p.out + (i << 4)) = acc;
    }
  }
}

// Checksum: per-block partial sums into scratch; the last block to arrive adds them.
// The sum is over 64-bit integers (wrapping), so its value depends neither on the order
// of the additions nor on scheduling.
constexpr int kCsumBlocks = 592;  // 4 per SM on a 148-SM part
constexpr int kCsumThreads = 256;
struct CsumScratch {
  uint32_t ticket;
  uint32_t pad;
  uint64_t partial[kCsumBlocks];
};
__global__ void __launch_bounds__(kCsumThreads)
checksum_kernel(const uint8_t* buf, uint64_t bytes, uint64_t* out, CsumScratch* scratch) {
  const uint64_t words = bytes >> 2;
  const uint32_t* w = reinterpret_cast<const uint32_t*>(buf);
  uint64_t sum = 0;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(buf) & 15) == 0;
  const uint64_t vecs = vec_ok ? (words >> 2) : 0;
  // Eight independent 16-byte streaming loads per thread and trip: at four CTAs of 256
  // threads per SM that is 128 KiB in flight per SM, several times what the HBM latency
  // asks for; one load per trip (16 KiB per SM) left the kernel latency-bound at a third
  // of the copy rate.  The data is read once: `ld.global.cs` keeps it from displacing L2 lines.
  const uint4* v16 = reinterpret_cast<const uint4*>(buf);
  uint64_t i = tid;
  constexpr int kUnroll = 8;
  for (; i + (kUnroll - 1) * stride < vecs; i += kUnroll * stride) {
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      // volatile: the eight loads are issued back to back, ahead of the first add
      asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                   : "l"(v16 + i + (uint64_t)u * stride));
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) sum += (uint64_t)v[u].x + v[u].y + v[u].z + v[u].w;
  }
  for (; i < vecs; i += stride) {
    const uint4 v = __ldcs(v16 + i);
    sum += (uint64_t)v.x + v.y + v.z + v.w;
  }
  for (uint64_t i = (vecs << 2) + tid; i < words; i += stride) sum += w[i];
  if (tid == 0 && (bytes & 3)) {
    uint32_t last = 0;
    for (uint32_t b = 0; b < (bytes & 3); ++b) last |= (uint32_t)buf[(words << 2) + b] << (8 * b);
    sum += last;
  }
  __shared__ uint64_t red[kCsumThreads / 32];
  __shared__ uint32_t is_last;
  auto block_sum = [&](uint64_t v) -> uint64_t {  // valid in thread 0
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    __syncthreads();  // red[] may still be read from the previous use
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    uint64_t s = 0;
    if (threadIdx.x == 0)
      for (int i = 0; i < kCsumThreads / 32; ++i) s += red[i];
    return s;
  };
  const uint64_t mine = block_sum(sum);
  if (threadIdx.x == 0) {
    scratch->partial[blockIdx.x] = mine;
    __threadfence();
    is_last = atomicAdd(&scratch->ticket, 1u) == gridDim.x - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (is_last) {
    // The last block to arrive adds the partial sums, all threads at once: one thread
    // walking 592 dependent-latency loads cost 20 us, twice the time of the 64 MiB pass.
    __threadfence();
    uint64_t part = 0;
    for (uint32_t b = threadIdx.x; b < gridDim.x; b += blockDim.x)
      part += *reinterpret_cast<volatile uint64_t*>(&scratch->partial[b]);
    const uint64_t total = block_sum(part);
    if (threadIdx.x == 0) {
      *out = total;
      scratch->ticket = 0;
    }
  }
}

// Scratch of the allocation-free checksum entry point: one CsumScratch per GPU,
// resident from library load to process exit.
static_assert(sizeof(CsumScratch) <= TCPXB_CHECKSUM_NOALLOC_SCRATCH_BYTES, "stated scratch size");
static __device__ __align__(256) unsigned char g_csum_static[TCPXB_CHECKSUM_NOALLOC_SCRATCH_BYTES];

// ------------------------------------------------------------------ host side
thread_local char g_err[256] = "";
int fail(int code, const char* fmt, const char* a = "") {
  snprintf(g_err, sizeof g_err, fmt, a);
  return code;
}
#define CUDA_TRY(expr)                                                  \
  do {                                                                  \
    cudaError_t e_ = (expr);                                            \
    if (e_ != cudaSuccess) return fail(TCPXB_K_CUDA, #expr ": %s", cudaGetErrorString(e_)); \
  } while (0)

constexpr int kMaxDevices = 64;
struct DeviceInfo {
  int sms = 0;
  bool attr_done[3][2][3] = {};
};
DeviceInfo g_dev[kMaxDevices];

// Applies the shared-memory attribute of one variant on `dev` (this also makes the
// runtime load the kernel) and records that it is done.
template <int RED, bool L2RED, int FAN>
int prepareVariant(int dev) {
  using C = Cfg<RED, L2RED, FAN>;
  DeviceInfo& di = g_dev[dev];
  if (di.attr_done[RED][L2RED][FAN]) return TCPXB_K_OK;
  CUDA_TRY(cudaFuncSetAttribute(unpack_kernel<RED, L2RED, FAN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                C::kSmemBytes));
  di.attr_done[RED][L2RED][FAN] = true;
  return TCPXB_K_OK;
}

int deviceInfo(int* dev_out) {
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(TCPXB_K_INVALID, "device ordinal out of range");
  if (g_dev[dev].sms == 0) {
    int sms = 0;
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    g_dev[dev].sms = sms;
  }
  *dev_out = dev;
  return TCPXB_K_OK;
}

template <int RED, bool L2RED, int FAN>
int launch(const UnpackParams& p, int max_ctas, bool early, cudaStream_t stream) {
  using C = Cfg<RED, L2RED, FAN>;
  int dev = 0;
  int rc = deviceInfo(&dev);
  if (rc) return rc;
  rc = prepareVariant<RED, L2RED, FAN>(dev);
  if (rc) return rc;
  if (p.count == 0) return TCPXB_K_OK;
  int ctas = (int)((p.count + kWarps - 1) / kWarps);
  int cap = g_dev[dev].sms;
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (ctas > cap) ctas = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early ? 1 : 0;
  CUDA_TRY(cudaLaunchKernelEx(&cfg, unpack_kernel<RED, L2RED, FAN>, p));
  return TCPXB_K_OK;
}

// Device address of the allocation-free checksum's scratch on `dev` (the current
// device).  In host code `g_csum_static` is only a handle for the runtime, not an
// address a kernel could use, so the address is resolved once per device and kept.
int csumStaticScratch(int dev, void** out) {
  static std::mutex mu;
  static void* scratch_of_device[kMaxDevices] = {};
  std::lock_guard<std::mutex> l(mu);
  if (scratch_of_device[dev] == nullptr) {
    void* p = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&p, g_csum_static));
    scratch_of_device[dev] = p;
  }
  *out = scratch_of_device[dev];
  return TCPXB_K_OK;
}

template <int FAN>
int prepareFan(int dev) {
  int rc = prepareVariant<TCPXB_U8, false, FAN>(dev);
  if (!rc) rc = prepareVariant<TCPXB_BF16, false, FAN>(dev);
  if (!rc) rc = prepareVariant<TCPXB_BF16, true, FAN>(dev);
  if (!rc) rc = prepareVariant<TCPXB_F32, false, FAN>(dev);
  if (!rc) rc = prepareVariant<TCPXB_F32, true, FAN>(dev);
  return rc;
}

template <int FAN>
int dispatch(const UnpackParams& p, int dtype, int impl, int max_ctas, bool early, cudaStream_t s) {
  const bool l2 = (impl == TCPXB_REDUCE_L2);
  switch (dtype) {
    case TCPXB_U8: return launch<TCPXB_U8, false, FAN>(p, max_ctas, early, s);
    case TCPXB_BF16:
      return l2 ? launch<TCPXB_BF16, true, FAN>(p, max_ctas, early, s)
                : launch<TCPXB_BF16, false, FAN>(p, max_ctas, early, s);
    case TCPXB_F32:
      return l2 ? launch<TCPXB_F32, true, FAN>(p, max_ctas, early, s)
                : launch<TCPXB_F32, false, FAN>(p, max_ctas, early, s);
    default: return fail(TCPXB_K_INVALID, "unknown dtype");
  }
}

int fill(UnpackParams& p, const void* pool, uint64_t pool_bytes, const void* acc, void* dst,
         void* mc_dst, uint64_t dst_bytes, void* const* peers, int npeers,
         const tcpxbLoadMeta* descs, uint32_t count, uint32_t* status,
         const tcpxbUnpackOpts* opts) {
  memset(&p, 0, sizeof p);
  if (count != 0 && (pool == nullptr || dst == nullptr || descs == nullptr))
    return fail(TCPXB_K_INVALID, "null pool, dst or descriptor pointer");
  if (npeers < 0 || npeers > TCPXB_MAX_PEERS) return fail(TCPXB_K_INVALID, "npeers out of range");
  if (npeers > 0 && peers == nullptr) return fail(TCPXB_K_INVALID, "null peer table");
  if (reinterpret_cast<uintptr_t>(descs) & 15)
    return fail(TCPXB_K_INVALID, "descriptor array must be 16-byte aligned");
  p.pool = static_cast<const uint8_t*>(pool);
  p.pool_bytes = pool_bytes;
  p.dst = static_cast<uint8_t*>(dst);
  p.dst_bytes = dst_bytes;
  p.acc = static_cast<const uint8_t*>(acc ? acc : dst);
  p.mc_dst = static_cast<uint8_t*>(mc_dst);
  p.descs = descs;
  p.count = count;
  p.npeers = npeers;
  const uintptr_t base_mis = reinterpret_cast<uintptr_t>(dst) & 15;
  for (int i = 0; i < npeers; ++i) {
    if (peers[i] == nullptr) return fail(TCPXB_K_INVALID, "null peer pointer");
    // The fast path decides alignment from the local address; peers must agree.
    if ((reinterpret_cast<uintptr_t>(peers[i]) & 15) != base_mis)
      return fail(TCPXB_K_INVALID, "peer buffers must share the local buffer's 16-byte phase");
    p.peers[i] = static_cast<uint8_t*>(peers[i]);
  }
  if (mc_dst != nullptr && (reinterpret_cast<uintptr_t>(mc_dst) & 15) != base_mis)
    return fail(TCPXB_K_INVALID, "multicast mapping must share the local buffer's 16-byte phase");
  p.status = status;
  if (opts != nullptr) {
    p.ready = opts->ready_count;
    p.wait_ns = opts->wait_ns;
    p.flag_value = opts->flag_value;
    p.ticket = opts->ticket;
    for (int i = 0; i < TCPXB_MAX_PEERS; ++i) p.peer_flags[i] = opts->peer_flags[i];
  }
  return TCPXB_K_OK;
}

}  // namespace

extern "C" {

const char* tcpxb_kernel_last_error(void) { return g_err; }

int tcpxb_kernels_preload(void) {
  static std::mutex mu;
  static bool done[kMaxDevices] = {};
  std::lock_guard<std::mutex> l(mu);
  int dev = 0;
  int rc = deviceInfo(&dev);
  if (rc) return rc;
  if (done[dev]) return TCPXB_K_OK;
  rc = prepareFan<FAN_NONE>(dev);
  if (!rc) rc = prepareFan<FAN_PEER>(dev);
  if (!rc) rc = prepareFan<FAN_NVLS>(dev);
  if (rc) return rc;
  // Setting an attribute does not make the runtime load a kernel; an empty launch
  // does.  Every kernel runs once with nothing to do, on a private stream.
  cudaStream_t s = nullptr;
  CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  UnpackParams p;
  memset(&p, 0, sizeof p);
#define TCPXB_DRY(RED, L2, FAN) \
  unpack_kernel<RED, L2, FAN><<<1, kThreads, Cfg<RED, L2, FAN>::kSmemBytes, s>>>(p)
#define TCPXB_DRY_FAN(FAN)                                                      \
  TCPXB_DRY(TCPXB_U8, false, FAN); TCPXB_DRY(TCPXB_BF16, false, FAN); TCPXB_DRY(TCPXB_BF16, true, FAN); \
  TCPXB_DRY(TCPXB_F32, false, FAN); TCPXB_DRY(TCPXB_F32, true, FAN)
  TCPXB_DRY_FAN(FAN_NONE);
  TCPXB_DRY_FAN(FAN_PEER);
  TCPXB_DRY_FAN(FAN_NVLS);
#undef TCPXB_DRY_FAN
#undef TCPXB_DRY
  wait_flags_kernel<<<1, 32, 0, s>>>(nullptr, 0, 0, 1, nullptr);
  SignalParams sp;
  memset(&sp, 0, sizeof sp);
  signal_flags_kernel<<<1, 32, 0, s>>>(sp);
  PeerReduceParams pp;
  memset(&pp, 0, sizeof pp);
  peer_reduce_kernel<TCPXB_BF16><<<1, 256, 0, s>>>(pp);
  peer_reduce_kernel<TCPXB_F32><<<1, 256, 0, s>>>(pp);
  // The checksum kernel and the address of the allocation-free entry point's scratch:
  // one launch over zero bytes, its result written into the scratch itself, so that
  // the first real tcpxb_checksum_noalloc on this device only clears and launches.
  void* cs = nullptr;
  rc = csumStaticScratch(dev, &cs);
  if (rc) return rc;
  CUDA_TRY(cudaMemsetAsync(cs, 0, 8, s));
  checksum_kernel<<<1, kCsumThreads, 0, s>>>(nullptr, 0, &static_cast<CsumScratch*>(cs)->partial[kCsumBlocks - 1],
                                             static_cast<CsumScratch*>(cs));
  CUDA_TRY(cudaGetLastError());
  CUDA_TRY(cudaStreamSynchronize(s));
  CUDA_TRY(cudaStreamDestroy(s));
  done[dev] = true;
  return TCPXB_K_OK;
}

int tcpxb_unpack_copy(const void* pool, uint64_t pool_bytes, void* dst, uint64_t dst_bytes,
                      const tcpxbLoadMeta* descs, uint32_t count, uint32_t* status,
                      const tcpxbUnpackOpts* opts, void* stream) {
  UnpackParams p;
  int rc = fill(p, pool, pool_bytes, nullptr, dst, nullptr, dst_bytes, nullptr, 0, descs, count,
                status, opts);
  if (rc) return rc;
  return dispatch<FAN_NONE>(p, TCPXB_U8, 0, opts ? opts->max_ctas : 0, opts != nullptr && opts->early_launch != 0,
                            static_cast<cudaStream_t>(stream));
}

int tcpxb_unpack_reduce(const void* pool, uint64_t pool_bytes, const void* acc, void* dst,
                        uint64_t dst_bytes, const tcpxbLoadMeta* descs, uint32_t count, int dtype,
                        int impl, uint32_t* status, const tcpxbUnpackOpts* opts, void* stream) {
  if (dtype != TCPXB_BF16 && dtype != TCPXB_F32)
    return fail(TCPXB_K_INVALID, "reduce needs dtype bf16 or f32");
  if (impl == TCPXB_REDUCE_L2 && acc != nullptr && acc != dst)
    return fail(TCPXB_K_INVALID, "the L2 reduce form is in place: acc must be NULL or dst");
  UnpackParams p;
  int rc = fill(p, pool, pool_bytes, acc, dst, nullptr, dst_bytes, nullptr, 0, descs, count, status,
                opts);
  if (rc) return rc;
  return dispatch<FAN_NONE>(p, dtype, impl, opts ? opts->max_ctas : 0, opts != nullptr && opts->early_launch != 0,
                            static_cast<cudaStream_t>(stream));
}

int tcpxb_unpack_fanout(const void* pool, uint64_t pool_bytes, void* dst, uint64_t dst_bytes,
                        void* const* peers, int npeers, const tcpxbLoadMeta* descs, uint32_t count,
                        uint32_t* status, const tcpxbUnpackOpts* opts, void* stream) {
  UnpackParams p;
  int rc = fill(p, pool, pool_bytes, nullptr, dst, nullptr, dst_bytes, peers, npeers, descs, count,
                status, opts);
  if (rc) return rc;
  return dispatch<FAN_PEER>(p, TCPXB_U8, 0, opts ? opts->max_ctas : 0, opts != nullptr && opts->early_launch != 0,
                            static_cast<cudaStream_t>(stream));
}

int tcpxb_unpack_reduce_fanout(const void* pool, uint64_t pool_bytes, const void* acc, void* dst,
                               uint64_t dst_bytes, void* const* peers, int npeers,
                               const tcpxbLoadMeta* descs, uint32_t count, int dtype, int impl,
                               uint32_t* status, const tcpxbUnpackOpts* opts, void* stream) {
  if (dtype != TCPXB_BF16 && dtype != TCPXB_F32)
    return fail(TCPXB_K_INVALID, "reduce needs dtype bf16 or f32");
  if (impl == TCPXB_REDUCE_L2 && acc != nullptr && acc != dst)
    return fail(TCPXB_K_INVALID, "the L2 reduce form is in place: acc must be NULL or dst");
  UnpackParams p;
  int rc = fill(p, pool, pool_bytes, acc, dst, nullptr, dst_bytes, peers, npeers, descs, count,
                status, opts);
  if (rc) return rc;
  return dispatch<FAN_PEER>(p, dtype, impl, opts ? opts->max_ctas : 0, opts != nullptr && opts->early_launch != 0,
                            static_cast<cudaStream_t>(stream));
}

int tcpxb_unpack_fanout_nvls(const void* pool, uint64_t pool_bytes, void* dst, void* mc_dst,
                             uint64_t dst_bytes, void* const* peers, int npeers,
                             const tcpxbLoadMeta* descs, uint32_t count, uint32_t* status,
                             const tcpxbUnpackOpts* opts, void* stream) {
  if (mc_dst == nullptr) return fail(TCPXB_K_INVALID, "null multicast mapping");
  UnpackParams p;
  int rc = fill(p, pool, pool_bytes, nullptr, dst, mc_dst, dst_bytes, peers, npeers, descs, count,
                status, opts);
  if (rc) return rc;
  return dispatch<FAN_NVLS>(p, TCPXB_U8, 0, opts ? opts->max_ctas : 0, opts != nullptr && opts->early_launch != 0,
                            static_cast<cudaStream_t>(stream));
}

int tcpxb_unpack_reduce_fanout_nvls(const void* pool, uint64_t pool_bytes, const void* acc,
                                    void* dst, void* mc_dst, uint64_t dst_bytes,
                                    void* const* peers, int npeers, const tcpxbLoadMeta* descs,
                                    uint32_t count, int dtype, uint32_t* status,
                                    const tcpxbUnpackOpts* opts, void* stream) {
  if (mc_dst == nullptr) return fail(TCPXB_K_INVALID, "null multicast mapping");
  if (dtype != TCPXB_BF16 && dtype != TCPXB_F32)
    return fail(TCPXB_K_INVALID, "reduce needs dtype bf16 or f32");
  UnpackParams p;
  int rc = fill(p, pool, pool_bytes, acc, dst, mc_dst, dst_bytes, peers, npeers, descs, count,
                status, opts);
  if (rc) return rc;
  // acc == NULL selects the reduce-into-all form (multimem.red into every accumulator).
  return dispatch<FAN_NVLS>(p, dtype, acc == nullptr ? TCPXB_REDUCE_L2 : TCPXB_REDUCE_SM,
                            opts ? opts->max_ctas : 0, opts != nullptr && opts->early_launch != 0, static_cast<cudaStream_t>(stream));
}

int tcpxb_wait_flags(const uint32_t* flags, int n, uint32_t value, uint64_t wait_ns,
                     uint32_t* status, void* stream) {
  if (flags == nullptr || n < 0 || n > 32) return fail(TCPXB_K_INVALID, "bad flag table");
  if (n == 0) return TCPXB_K_OK;
  wait_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      flags, n, value, wait_ns ? wait_ns : kDefaultWaitNs, status);
  CUDA_TRY(cudaGetLastError());
  return TCPXB_K_OK;
}

int tcpxb_signal_flags(uint32_t* const* peer_flags, int n, uint32_t value, void* stream) {
  if (n < 0 || n > TCPXB_MAX_PEERS + 1 || (n > 0 && peer_flags == nullptr))
    return fail(TCPXB_K_INVALID, "bad flag table");
  if (n == 0) return TCPXB_K_OK;
  SignalParams p;
  memset(&p, 0, sizeof p);
  for (int i = 0; i < n; ++i) p.flags[i] = peer_flags[i];
  p.n = n;
  p.value = value;
  signal_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  CUDA_TRY(cudaGetLastError());
  return TCPXB_K_OK;
}

int tcpxb_peer_reduce(void* out, void* const* srcs, int nsrcs, uint64_t shard_off, uint64_t bytes,
                      int dtype, void* stream) {
  if (out == nullptr || srcs == nullptr || nsrcs < 1 || nsrcs > TCPXB_MAX_PEERS + 1)
    return fail(TCPXB_K_INVALID, "bad source table");
  if (dtype != TCPXB_BF16 && dtype != TCPXB_F32)
    return fail(TCPXB_K_INVALID, "reduce needs dtype bf16 or f32");
  if ((bytes & 15) || (shard_off & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return fail(TCPXB_K_INVALID, "peer_reduce works on 16-byte aligned spans");
  PeerReduceParams p;
  memset(&p, 0, sizeof p);
  for (int i = 0; i < nsrcs; ++i) {
    if (srcs[i] == nullptr || (reinterpret_cast<uintptr_t>(srcs[i]) & 15))
      return fail(TCPXB_K_INVALID, "null or misaligned source");
    p.srcs[i] = static_cast<const uint8_t*>(srcs[i]);
  }
  p.nsrcs = nsrcs;
  p.out = static_cast<uint8_t*>(out);
  p.shard_off = shard_off;
  p.vecs = bytes >> 4;
  if (p.vecs == 0) return TCPXB_K_OK;
  int dev = 0, sms = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  uint64_t want = (p.vecs + 255) / 256;
  int blocks = (int)(want < (uint64_t)sms * 8 ? want : (uint64_t)sms * 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == TCPXB_BF16) peer_reduce_kernel<TCPXB_BF16><<<blocks, 256, 0, s>>>(p);
  else peer_reduce_kernel<TCPXB_F32><<<blocks, 256, 0, s>>>(p);
  CUDA_TRY(cudaGetLastError());
  return TCPXB_K_OK;
}

size_t tcpxb_checksum_scratch_bytes(void) { return sizeof(CsumScratch); }

int tcpxb_checksum(const void* buf, uint64_t bytes, uint64_t* out, void* partials, void* stream) {
  if (out == nullptr || partials == nullptr || (buf == nullptr && bytes != 0))
    return fail(TCPXB_K_INVALID, "null buffer, output or scratch");
  if (reinterpret_cast<uintptr_t>(buf) & 3)
    return fail(TCPXB_K_INVALID, "checksum buffer must be 4-byte aligned");
  uint64_t want = (bytes / 16 + kCsumThreads - 1) / kCsumThreads;
  int blocks = (int)(want < 1 ? 1 : (want > (uint64_t)kCsumBlocks ? kCsumBlocks : want));
  checksum_kernel<<<blocks, kCsumThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(buf), bytes, out, static_cast<CsumScratch*>(partials));
  CUDA_TRY(cudaGetLastError());
  return TCPXB_K_OK;
}

int tcpxb_checksum_noalloc(const void* buf, uint64_t bytes, uint64_t* out, void* stream) {
  if (out == nullptr || (buf == nullptr && bytes != 0))
    return fail(TCPXB_K_INVALID, "null buffer or output");
  if (reinterpret_cast<uintptr_t>(buf) & 3)
    return fail(TCPXB_K_INVALID, "checksum buffer must be 4-byte aligned");
  if (bytes > TCPXB_CHECKSUM_NOALLOC_MAX_BYTES)
    return fail(TCPXB_K_TOO_LARGE,
                "tcpxb_checksum_noalloc handles at most 16 GiB per call; split the buffer or use tcpxb_checksum");
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(TCPXB_K_INVALID, "device ordinal out of range");
  void* scratch = nullptr;
  const int rc = csumStaticScratch(dev, &scratch);  // a table look-up after tcpxb_kernels_preload or a first call
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the completion counter must start at zero even if an earlier launch was cut short
  CUDA_TRY(cudaMemsetAsync(scratch, 0, 8, s));
  uint64_t want = (bytes / 16 + kCsumThreads - 1) / kCsumThreads;
  int blocks = (int)(want < 1 ? 1 : (want > (uint64_t)kCsumBlocks ? kCsumBlocks : want));
  checksum_kernel<<<blocks, kCsumThreads, 0, s>>>(static_cast<const uint8_t*>(buf), bytes, out,
                                                  static_cast<CsumScratch*>(scratch));
  CUDA_TRY(cudaGetLastError());
  return TCPXB_K_OK;
}

}  // extern "C"
