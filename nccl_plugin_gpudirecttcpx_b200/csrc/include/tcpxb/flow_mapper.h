// Chooses the data socket ("flow") that carries the next chunk of a message.
//
// Two policies, selectable with NCCL_GPUDIRECTTCPX_SCHED_ALG like the reference
// (reference: src/flow_mapper.h:51-157):
//   RR    the turn passes round the sockets that have a free task slot (the
//         reference keeps them on a stack and takes the most recently offered).
//   KATY  least-loaded first: a 64-bit occupancy map with one bit per
//         (busy-slot count, socket); the lowest set bit is the emptiest socket
//         with the lowest index.  A picked socket is offered again one load level
//         up, and at most two picks are granted per progress round so one
//         request cannot monopolise the sockets.
// Each progress round calls reset(), then offer() for every socket with room,
// then pick() until it returns -1.
#ifndef TCPXB_FLOW_MAPPER_H_
#define TCPXB_FLOW_MAPPER_H_

#include <stdint.h>

#include <memory>

namespace tcpxb {

constexpr int kMaxSockets = 8;
constexpr int kMaxThreads = 16;
constexpr int kMaxTasks = 6;      // per data socket
constexpr int kMaxRequests = 16;  // per comm

class FlowMapper {
 public:
  virtual ~FlowMapper() = default;
  virtual void reset() = 0;
  // Socket `flow` has kMaxTasks - busy free task slots (busy < kMaxTasks).
  virtual void offer(int flow, int busy) = 0;
  virtual bool hasFlow() const = 0;
  // Next socket to use, or -1.
  virtual int pick() = 0;
  virtual const char* name() const = 0;
};

class FlowMapperRR final : public FlowMapper {
 public:
  void reset() override {
    for (int& f : free_) f = 0;
    total_ = 0;
  }
  void offer(int flow, int busy) override {
    if (busy >= kMaxTasks) return;
    total_ += (kMaxTasks - busy) - free_[flow];
    free_[flow] = kMaxTasks - busy;
  }
  bool hasFlow() const override { return total_ > 0; }
  int pick() override {
    if (total_ <= 0) return -1;
    // the turn passes round the sockets and survives reset(), so consecutive
    // chunks - also those of different rounds - land on different sockets
    for (int i = 0; i < kMaxSockets; ++i) {
      const int flow = (turn_ + i) % kMaxSockets;
      if (free_[flow] > 0) {
        --free_[flow];
        --total_;
        turn_ = (flow + 1) % kMaxSockets;
        return flow;
      }
    }
    return -1;
  }
  const char* name() const override { return "RR"; }

 private:
  int free_[kMaxSockets] = {};
  int total_ = 0;
  int turn_ = 0;
};

class FlowMapperKaty final : public FlowMapper {
 public:
  static constexpr int kPicksPerRound = 2;
  void reset() override { map_ = 0; picks_ = 0; }
  void offer(int flow, int busy) override {
    if (busy < kMaxTasks) map_ |= 1ull << (flow + kMaxSockets * busy);
  }
  bool hasFlow() const override { return map_ != 0 && picks_ < kPicksPerRound; }
  int pick() override {
    if (!hasFlow()) return -1;
    const int bit = __builtin_ffsll((long long)map_) - 1;
    map_ &= ~(1ull << bit);
    const int flow = bit % kMaxSockets, busy = bit / kMaxSockets;
    if (busy + 1 < kMaxTasks) map_ |= 1ull << (flow + kMaxSockets * (busy + 1));
    ++picks_;
    return flow;
  }
  const char* name() const override { return "KATY"; }

 private:
  static_assert(kMaxSockets * kMaxTasks <= 64, "occupancy map must fit 64 bits");
  uint64_t map_ = 0;
  int picks_ = 0;
};

inline std::unique_ptr<FlowMapper> makeFlowMapper(int sched_alg) {
  if (sched_alg == 1) return std::make_unique<FlowMapperKaty>();
  return std::make_unique<FlowMapperRR>();
}

}  // namespace tcpxb
#endif  // TCPXB_FLOW_MAPPER_H_
