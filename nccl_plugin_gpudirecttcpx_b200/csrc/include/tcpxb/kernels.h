// C ABI of the sm_100a device kernels: GPU unpack of scattered rx page fragments.
//
// The reference plugin ships no GPU kernel; it hands NCCL a scatter list of
// {src_off, len, dst_off} records (reference: src/sock/tcpx.h:178-180,
// src/devcomm/nccl/unpack1.cu:52-63) and NCCL's own collective kernels copy
// pool -> user buffer.  Here the same scatter list is consumed by our own
// kernels, which also fuse the receive-side reduction and the NVLink fan-out.
//
// All functions return 0 on success or a negative tcpxbKernelError; the text of
// the last failure on the calling thread is available from tcpxb_kernel_last_error().
#ifndef TCPXB_KERNELS_H_
#define TCPXB_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// One fragment of received payload: `len` bytes at `src_off` in the rx page pool
// belong at `dst_off` in the destination buffer.  Same 16-byte layout as NCCL's
// `union loadMeta` so one descriptor array serves both consumers.
typedef struct tcpxbLoadMeta {
  uint32_t src_off;
  uint32_t len;
  uint64_t dst_off;
} tcpxbLoadMeta;

// Largest fragment the bulk-copy fast path moves in one piece (one rx page,
// NCCL_NET_MTU_SIZE).  Longer descriptors are legal and take the generic path.
#define TCPXB_FRAG_BYTES 4096
#define TCPXB_MAX_PEERS 8

typedef enum tcpxbDtype {
  TCPXB_U8 = 0,    // plain bytes (copy only)
  TCPXB_BF16 = 1,  // sum in fp32, round once to bf16
  TCPXB_F32 = 2,
} tcpxbDtype;

typedef enum tcpxbReduceImpl {
  TCPXB_REDUCE_SM = 0,  // addend tile and fragment both staged in shared memory, added by the warp
  TCPXB_REDUCE_L2 = 1,  // cp.reduce.async.bulk: the add happens at the L2 / destination
} tcpxbReduceImpl;

typedef enum tcpxbKernelError {
  TCPXB_K_OK = 0,
  TCPXB_K_INVALID = -1,    // bad argument (null pointer, misaligned base, too many peers)
  TCPXB_K_CUDA = -2,       // a CUDA runtime call failed
  TCPXB_K_TOO_LARGE = -3,  // size beyond a stated maximum
} tcpxbKernelError;

// Device-side status block, written by the kernels (never trapped on).
// word[0] = first error code (0 = none), word[1] = index of the offending
// descriptor, word[2] = count of skipped descriptors, word[3] = reserved.
typedef enum tcpxbDeviceStatus {
  TCPXB_ST_OK = 0,
  TCPXB_ST_BOUNDS = 1,     // src_off+len > pool_bytes or dst_off+len > dst_bytes: fragment skipped
  TCPXB_ST_ALIGN = 2,      // reduce fragment not aligned to the element size: fragment skipped
  TCPXB_ST_TIMEOUT = 3,    // a bounded wait (mbarrier / ready counter / peer flag) ran out
} tcpxbDeviceStatus;
#define TCPXB_STATUS_WORDS 4

// Optional extras shared by every unpack entry point; zero-initialise for defaults.
typedef struct tcpxbUnpackOpts {
  // Streaming: when non-null the kernel treats descriptor i as published once
  // *ready_count > i (a host-mapped or device counter the producer advances with
  // release semantics) and waits for it; the wait gives up when the counter has not
  // moved for wait_ns nanoseconds (a producer that keeps advancing never trips the
  // limit, however long the launch lasts).
  const uint32_t* ready_count;
  uint64_t wait_ns;        // 0 = default (2 s)
  // Fan-out completion: when flag_value != 0, after every store of the launch has
  // completed the kernel writes flag_value (release, system scope) to every
  // non-null peer_flags[i], unless the launch recorded an error in `status`: then
  // no flag is written and the peers' own bounded waits run out.  `ticket` is one
  // zero-initialised uint32 of scratch on the launching GPU (at most 65535 CTAs per
  // launch); the kernel leaves it zero again.
  uint32_t* peer_flags[TCPXB_MAX_PEERS];
  uint32_t flag_value;
  uint32_t* ticket;
  int max_ctas;            // 0 = one CTA per SM
  // Programmatic dependent launch: when non-zero the launch may be scheduled while the
  // previous kernel of the stream is still running; its CTAs become resident as SMs free
  // up, set up their barriers, and wait for that kernel to complete (and its writes to
  // be visible) before they touch any memory.  Results are the same; back-to-back
  // launches lose the gap between kernels.
  int early_launch;
} tcpxbUnpackOpts;

// K1: dst[dst_off .. +len) = pool[src_off .. +len) for every descriptor.
int tcpxb_unpack_copy(const void* pool, uint64_t pool_bytes, void* dst, uint64_t dst_bytes,
                      const tcpxbLoadMeta* descs, uint32_t count, uint32_t* status,
                      const tcpxbUnpackOpts* opts, void* stream);

// K2: dst[..] = acc[..] + pool[..] element-wise (acc may equal dst for in-place).
// With impl == TCPXB_REDUCE_L2, acc must be NULL or equal dst (always in place).
int tcpxb_unpack_reduce(const void* pool, uint64_t pool_bytes, const void* acc, void* dst,
                        uint64_t dst_bytes, const tcpxbLoadMeta* descs, uint32_t count,
                        int dtype, int impl, uint32_t* status, const tcpxbUnpackOpts* opts,
                        void* stream);

// K3: as K1, and every unpacked fragment is also stored at the same dst_off in
// each peers[i] (peer-mapped device pointers reached over NVLink).
int tcpxb_unpack_fanout(const void* pool, uint64_t pool_bytes, void* dst, uint64_t dst_bytes,
                        void* const* peers, int npeers, const tcpxbLoadMeta* descs,
                        uint32_t count, uint32_t* status, const tcpxbUnpackOpts* opts,
                        void* stream);

// K3r: as K2, and the reduced fragment is also stored to each peer.  With
// impl == TCPXB_REDUCE_L2 the fragment is instead added into dst and into every
// peer's buffer (each peer keeps its own accumulator).
int tcpxb_unpack_reduce_fanout(const void* pool, uint64_t pool_bytes, const void* acc, void* dst,
                               uint64_t dst_bytes, void* const* peers, int npeers,
                               const tcpxbLoadMeta* descs, uint32_t count, int dtype, int impl,
                               uint32_t* status, const tcpxbUnpackOpts* opts, void* stream);

// NVLS variants: the fan-out goes through one multimem store (or multimem.red for
// the reduce-into-all form) on `mc_dst`, a multicast mapping of the same buffer on
// every GPU of the group (the local GPU included).  `dst` is the local unicast
// mapping of that buffer, used for ragged head/tail bytes together with `peers`.
int tcpxb_unpack_fanout_nvls(const void* pool, uint64_t pool_bytes, void* dst, void* mc_dst,
                             uint64_t dst_bytes, void* const* peers, int npeers,
                             const tcpxbLoadMeta* descs, uint32_t count, uint32_t* status,
                             const tcpxbUnpackOpts* opts, void* stream);
int tcpxb_unpack_reduce_fanout_nvls(const void* pool, uint64_t pool_bytes, const void* acc,
                                    void* dst, void* mc_dst, uint64_t dst_bytes,
                                    void* const* peers, int npeers, const tcpxbLoadMeta* descs,
                                    uint32_t count, int dtype, uint32_t* status,
                                    const tcpxbUnpackOpts* opts, void* stream);

// Loads every kernel of this library on the current device and applies their
// launch attributes.  CUDA loads kernels lazily, and a first launch may have to
// wait for running kernels to finish; a receive path that launches its first
// unpack kernel while a collective kernel is spinning on that very data would
// never return.  Call this at set-up time, before such kernels exist.
int tcpxb_kernels_preload(void);

// Waits (bounded) until flags[i] >= value for i in [0, n); on time-out writes
// TCPXB_ST_TIMEOUT to status and returns.  Runs on the GPU that owns `flags`.
int tcpxb_wait_flags(const uint32_t* flags, int n, uint32_t value, uint64_t wait_ns,
                     uint32_t* status, void* stream);

// Writes `value` (release, system scope) to each peer_flags[i]: "my buffers are
// ready for epoch `value`".  The counterpart of tcpxb_wait_flags.
int tcpxb_signal_flags(uint32_t* const* peer_flags, int n, uint32_t value, void* stream);

// Intra-node reduce-scatter stage over peer memory: out[i] = sum over r of
// srcs[r][shard_off + i], element-wise, for `bytes` bytes.  srcs are peer-mapped
// device pointers (the local one included); plain peer loads, no library call.
int tcpxb_peer_reduce(void* out, void* const* srcs, int nsrcs, uint64_t shard_off,
                      uint64_t bytes, int dtype, void* stream);

// 64-bit checksum of a buffer (sum of its 32-bit words, little-endian, the ragged
// tail zero-padded), written to *out on the device.  `partials` is scratch:
// tcpxb_checksum_scratch_bytes() bytes, of which the first 4 must be zero before
// the first use; the kernel leaves them zero again.
size_t tcpxb_checksum_scratch_bytes(void);
int tcpxb_checksum(const void* buf, uint64_t bytes, uint64_t* out, void* partials, void* stream);

// Checksum for callers that must not allocate device memory.
//
// Same result as tcpxb_checksum, but the scratch for the per-block partial sums
// lives in a fixed array inside this library instead of a buffer the caller
// provides, so the call performs no cudaMalloc / cudaFree and uses no allocating
// library routine.  It is meant for code that runs where an allocation is
// forbidden or dangerous: the transport's progress loop on NCCL's proxy thread
// (a cudaMalloc there synchronises the device and can deadlock against a
// collective kernel that is waiting for that same thread), completion callbacks,
// and processes that were handed a fixed amount of device memory and may not grow it.
// The reference has nothing like it (it owns no kernel at all).
//
//  * The array takes TCPXB_CHECKSUM_NOALLOC_SCRATCH_BYTES on every GPU that loads
//    the library, from load until the process exits.
//  * Buffers larger than TCPXB_CHECKSUM_NOALLOC_MAX_BYTES are refused with
//    TCPXB_K_TOO_LARGE and an explanatory message; nothing is launched.
//  * The array's device address is looked up once per device (cudaGetSymbolAddress
//    with that device current): by tcpxb_kernels_preload if it ran on the device,
//    else by the first call there.  Do whichever comes first before any stream
//    capture begins on the device, and off the path that must not block: the
//    look-up may load the module.  Later calls only clear the counter and launch.
//  * All calls on one GPU share the array: the counter it starts from is cleared
//    on the stream at the head of every call, and the partial sums keep the
//    previous call's values until overwritten.  Two calls that overlap in time on
//    the same GPU (different streams) race on it and may both return garbage;
//    issue them on one stream or order them with events.
// `buf`, `out` and `stream` are as for tcpxb_checksum; `out` is device memory the
// caller owns.
#define TCPXB_CHECKSUM_NOALLOC_MAX_BYTES (1ull << 34)
#define TCPXB_CHECKSUM_NOALLOC_SCRATCH_BYTES 4864
int tcpxb_checksum_noalloc(const void* buf, uint64_t bytes, uint64_t* out, void* stream);

const char* tcpxb_kernel_last_error(void);

#ifdef __cplusplus
}
#endif
#endif  // TCPXB_KERNELS_H_
