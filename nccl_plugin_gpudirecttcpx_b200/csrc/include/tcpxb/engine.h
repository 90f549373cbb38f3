// Hierarchical collective engine: drives the transport's isend/irecv for the
// inter-node stage and the fused unpack kernels for the receive-side reduction and
// the intra-node NVLink stage.
//
// The reference has no counterpart (it sits below NCCL and owns no collective;
// reference: src/nccl_plugin.cc:22-42 is its whole upward interface).  It exists
// here because NCCL cannot call this library's kernels from inside its own: the
// product path "network receive fused with reduction and NVLink fan-out" has to be
// driven by something that sees both the scatter lists and the peer mappings.
//
// Topology.  `world` ranks, one GPU each, grouped into emulated nodes of
// `gpus_per_node` consecutive ranks.  Rank r talks over the network only to the
// ranks with the same local index in the neighbouring nodes ("rails").  With
// world == 1 the single rank is its own network peer (a twin node holding the same
// data), which runs the identical code path on one GPU.
//
// all_reduce of S bytes per GPU:
//   1. intra-node reduce-scatter by peer loads (tcpxb_peer_reduce): GPU l owns shard l;
//   2. inter-node stage on the shard: two nodes exchange whole shards and each adds
//      the received fragments (unpack_reduce_fanout); more nodes run a ring
//      reduce-scatter (unpack_reduce) then a ring all-gather (unpack_fanout);
//   3. the kernels of step 2 store every finished fragment into all local GPUs'
//      output buffers, so the intra-node all-gather rides on the receive path.
// Synchronous calls block the host until every network transfer is done and every kernel
// is queued on the caller's stream; the asynchronous forms below hand the same work to a
// thread of the engine's own.
#ifndef TCPXB_ENGINE_H_
#define TCPXB_ENGINE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TCPXB_ENGINE_MAX_RAILS 16
#define TCPXB_ENGINE_HANDLE_BYTES 128

typedef struct tcpxbEngineConfig {
  int rank, world, gpus_per_node;
  int gpu_dev;            // CUDA device of this rank
  int request_bytes;      // bytes per network request (<= 4 MiB, multiple of 4096); 0 = 1 MiB
  int max_inflight;       // requests in flight per rail (<= 12); 0 = 4 (little in flight stays in the CPU's caches)
  int unpack_ctas;        // CTAs per unpack launch; 0 = 16
  int reduce_impl;        // TCPXB_REDUCE_SM or TCPXB_REDUCE_L2
  int use_nvls;           // use the multimem fan-out when a multicast mapping is given
  int plain_mode;         // 1 = baseline: unpack_copy to a bounce buffer, separate add, no fused fan-out
  // The driving thread of an exchange spins for idle_spin_us without progress, then sleeps
  // idle_sleep_us at a time.  0 = defaults (20 / 30); idle_sleep_us < 0 = never sleep.
  // By default the sleep is a plain nap that nobody ends early; with wake_on_events it is a
  // ppoll on the control sockets and on an eventfd that helper threads write when a task
  // finishes (lower latency per event, one system call per wake-up on both sides).
  int idle_spin_us, idle_sleep_us, wake_on_events;
} tcpxbEngineConfig;

typedef struct tcpxbEngineStats {
  uint64_t bytes_sent, bytes_received;   // over the network, this rank
  uint64_t requests, unpack_launches, fragments;
  uint64_t kernel_launches;              // every kernel of this library the engine queued
  double seconds_net_wait;               // host time spent inside exchanges
  // where the driving thread spends that time (seconds): posting receives, posting
  // sends (staging copies included), testing receives, launching unpack kernels,
  // returning pages, testing sends, idle spinning, and asleep waiting for a wake-up
  double t_post_recv, t_post_send, t_test_recv, t_launch, t_consume, t_test_send, t_idle, t_sleep;
  uint64_t sleeps;                       // times the driving thread blocked
  // helper threads of all rails, seconds: sending helpers asleep without a task / in poll()
  // on a full socket; receiving helpers asleep without a task / in poll() on an empty socket
  double tx_idle, tx_blocked, rx_idle, rx_blocked;
} tcpxbEngineStats;

// Creates the engine and initialises the transport (flags are read from the
// environment as for the plugin).  Returns NULL on failure.
void* tcpxb_engine_create(const tcpxbEngineConfig* cfg);
void tcpxb_engine_destroy(void* engine);
// Number of rails (network devices) the engine stripes over.
int tcpxb_engine_rails(void* engine);
// Opens one listening endpoint per rail; writes rails x 128 bytes of handles.
int tcpxb_engine_listen(void* engine, void* handles_out);
// Connects to the next node's handles and accepts the previous node's connection.
// `next_handles` are the bytes the next neighbour's tcpxb_engine_listen produced.
int tcpxb_engine_connect(void* engine, const void* next_handles);
// Intra-node peer mappings, all indexed by local rank (the own entry included):
// work buffers (inputs are staged here), output buffers, flag blocks
// (>= 64 uint32 each, zero-initialised) and optionally a multicast mapping of the
// output buffer.  Every buffer holds at least `buffer_bytes`.
int tcpxb_engine_set_peers(void* engine, void* const* work_ptrs, void* const* out_ptrs,
                           uint32_t* const* flag_ptrs, void* mc_out, uint64_t buffer_bytes);

// Collectives.  With gpus_per_node > 1 the peers read and write the buffers registered
// with tcpxb_engine_set_peers: all_gather and reduce_scatter take exactly those (`in` =
// this rank's work buffer where it is read by peers, `out` = its output buffer);
// all_reduce also takes any other device pointers, `out` == `in` included, and stages them
// through the registered buffers with one device copy each way.  With one GPU per node,
// `out` may be `in` (in place; between two nodes that costs one device copy).
int tcpxb_engine_all_reduce(void* engine, const void* in, void* out, uint64_t bytes, int dtype, void* stream);
// all_gather: `in` holds bytes_per_rank; out receives world x bytes_per_rank in rank order.
int tcpxb_engine_all_gather(void* engine, const void* in, void* out, uint64_t bytes_per_rank, void* stream);
// reduce_scatter: `in` holds world x bytes_per_rank; out receives this rank's reduced part.
int tcpxb_engine_reduce_scatter(void* engine, const void* in, void* out, uint64_t bytes_per_rank, int dtype, void* stream);
// Point-to-point over rail 0..n to the next / from the previous node (same local index).
int tcpxb_engine_send_next(void* engine, const void* buf, uint64_t bytes, void* stream);
int tcpxb_engine_recv_prev(void* engine, void* buf, uint64_t bytes, void* stream);

// Asynchronous forms.  The call queues the collective on a thread and a stream of the
// engine's own and returns a ticket (> 0; 0 = failure) at once, so the caller's thread is
// free and may queue more: jobs run in the order they were queued.  `after_event` (a CUDA
// event, or NULL) is what the engine's stream waits for before it touches the buffers.
//   tcpxb_engine_test / _wait   has the job finished its network part and queued its last
//                               kernel?  (_wait blocks.)  Return -1 when the job failed.
//   tcpxb_engine_stream_wait    makes `stream` wait for the job's kernels (after _wait).
//   tcpxb_engine_release        forgets a finished job.
// Synchronous and asynchronous calls must not be mixed while jobs are queued.
uint64_t tcpxb_engine_all_reduce_async(void* engine, const void* in, void* out, uint64_t bytes, int dtype, void* after_event);
uint64_t tcpxb_engine_all_gather_async(void* engine, const void* in, void* out, uint64_t bytes_per_rank, void* after_event);
uint64_t tcpxb_engine_reduce_scatter_async(void* engine, const void* in, void* out, uint64_t bytes_per_rank, int dtype, void* after_event);
int tcpxb_engine_test(void* engine, uint64_t ticket, int* done);
int tcpxb_engine_wait(void* engine, uint64_t ticket);
int tcpxb_engine_stream_wait(void* engine, uint64_t ticket, void* stream);
int tcpxb_engine_release(void* engine, uint64_t ticket);

int tcpxb_engine_stats(void* engine, tcpxbEngineStats* out);
// First device-side status word the unpack kernels reported (0 = clean).
int tcpxb_engine_device_status(void* engine, uint32_t* words4);
const char* tcpxb_engine_last_error(void);

#ifdef __cplusplus
}
#endif
#endif  // TCPXB_ENGINE_H_
