// Fixed-capacity ring whose items walk through an ordered list of stages.
//
// Same job as the reference's multi-cursor item queue (reference:
// src/work_queue.h:78-130, states in src/work_queue_states.h:22-39): one array,
// one monotonically increasing cursor per stage boundary, FIFO within every
// stage.  boundary[0] counts items ever admitted; boundary[s] counts items that
// have left stage s.  The items currently in stage s (1-based: stage 1 is the
// first after admission) are those with index in [boundary[s], boundary[s-1]).
// A slot is free again once the item left the last stage.
//
// Each boundary has exactly one writer thread, so the ring is lock-free when the
// stages are split between threads: a writer publishes with release, readers of
// other boundaries use acquire.  With `Atomic = false` the cursors are plain
// integers for single-threaded rings.
//
// Cursors are 64-bit: a slot is `cursor % capacity`, and with a capacity that does
// not divide 2^32 (the task ring holds 6) a 32-bit cursor would jump to another
// slot when it wraps, after about 4e9 chunks.  A 64-bit cursor never wraps in practice.
#ifndef TCPXB_STAGE_RING_H_
#define TCPXB_STAGE_RING_H_

#include <atomic>
#include <stdint.h>

namespace tcpxb {

template <bool Atomic>
struct RingCursor;
template <>
struct RingCursor<true> {
  std::atomic<uint64_t> v{0};
  uint64_t load() const { return v.load(std::memory_order_acquire); }
  void bump() { v.store(v.load(std::memory_order_relaxed) + 1, std::memory_order_release); }
  void reset(uint64_t to = 0) { v.store(to, std::memory_order_relaxed); }
};
template <>
struct RingCursor<false> {
  uint64_t v = 0;
  uint64_t load() const { return v; }
  void bump() { ++v; }
  void reset(uint64_t to = 0) { v = to; }
};

// kStages counts the live stages; the "free" state is implicit.
template <typename Item, uint32_t kCapacity, int kStages, bool Atomic>
class StageRing {
  static_assert(kCapacity >= 1 && kStages >= 1, "a ring needs at least one slot and one stage");
 public:
  static constexpr uint32_t capacity() { return kCapacity; }

  // ----- admission (free -> stage 1)
  uint32_t numFree() const { return kCapacity - (uint32_t)(edge_[0].load() - edge_[kStages].load()); }
  bool hasFree() const { return numFree() > 0; }
  bool empty() const { return edge_[0].load() == edge_[kStages].load(); }
  // The slot the next admitted item will occupy; fill it, then call admit().
  Item& nextFree() { return items_[edge_[0].load() % kCapacity]; }
  uint64_t nextFreeIndex() const { return edge_[0].load(); }
  void admit() { edge_[0].bump(); }

  // ----- stage s in [1, kStages]
  uint32_t count(int s) const { return (uint32_t)(edge_[s - 1].load() - edge_[s].load()); }
  bool has(int s) const { return count(s) > 0; }
  // Oldest item in stage s.
  Item& front(int s) { return items_[edge_[s].load() % kCapacity]; }
  uint64_t frontIndex(int s) const { return edge_[s].load(); }
  // k-th oldest item in stage s (k < count(s)).
  Item& at(int s, uint32_t k) { return items_[(edge_[s].load() + k) % kCapacity]; }
  // Moves the oldest item of stage s to stage s+1 (or frees it after the last stage).
  void advance(int s) { edge_[s].bump(); }

  Item& slot(uint64_t index) { return items_[index % kCapacity]; }
  uint32_t inFlight() const { return (uint32_t)(edge_[0].load() - edge_[kStages].load()); }

  // Empties the ring; every cursor restarts at `at` (tests start near 2^32).
  void reset(uint64_t at = 0) { for (auto& e : edge_) e.reset(at); }

 private:
  Item items_[kCapacity];
  RingCursor<Atomic> edge_[kStages + 1];
};

}  // namespace tcpxb
#endif  // TCPXB_STAGE_RING_H_
