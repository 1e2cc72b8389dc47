// Host-driven ring AllReduce over a OneSidedTransport: the network data plane
// (used between hosts, without NVLink, or without any GPU).  It keeps the
// reference pipeline's shape (reference: src/mini_nccl.cu:107-198): phase 1
// scatter-reduce and phase 2 all-gather of N-1 steps each, chunks cut into
// SLICE_SIZE slices pushed to rank+1, one-sided payload write followed by a
// flag write, every SIGNAL_BATCH-th flag write signalled, at most WINDOW
// signalled requests in flight.
//
// What is different, on purpose:
//  * sequence numbers continue across calls (the reference restarts at 1 while
//    the flags keep their old values, so later calls never wait);
//  * the receiver returns credits, so a scratch slot is never overwritten
//    before it was consumed (the reference has two slots and no credit);
//  * a slice is forwarded only after its reduction has finished (the
//    reference posts the network write without waiting for the GPU reduce);
//  * count need not divide by the rank count (the reference drops count % N
//    trailing elements) and may be smaller than it;
//  * both phases land in scratch, so no buffer address is exchanged per call;
//  * every wait is bounded and observes the abort word;
//  * for messages of 4 MB and more (and a provider that allows posting from two threads) the sends of
//    a call run in a second thread while the caller's thread receives, reduces and returns credits:
//    a slice is sent as soon as the slice it forwards has been received, so copying out and reducing
//    in overlap instead of taking turns (MINI_NCCL_RING_SENDER_THREAD=0: one thread, as before).
#pragma once
#include <atomic>
#include <cstdint>
#include <deque>
#include <memory>

#include "core/config.h"
#include "core/dtype.h"
#include "net/transport.h"

namespace mnccl {

class BootstrapStore;

struct RingStats {
  uint64_t calls = 0, slices_sent = 0, slices_received = 0, bytes_sent = 0;
  uint64_t credit_stalls = 0, window_stalls = 0;
  uint64_t threaded_calls = 0;   // calls whose sends ran in the second thread
};

class RingAllReduce {
 public:
  // `abort_word` (may be null) is polled inside every wait.
  RingAllReduce(int rank, int size, OneSidedTransport* transport, BootstrapStore* store,
                const Config& cfg, const volatile uint32_t* abort_word);
  ~RingAllReduce();

  // In place on host-accessible memory.  Throws Error on timeout / abort.
  void run(void* data, size_t count, DType dtype, RedOp op);

  const RingStats& stats() const { return stats_; }
  size_t slice_bytes() const { return slice_bytes_; }
  int slots() const { return nslots_; }

 private:
  enum : uint32_t { kDataFlag = 0, kCreditFlag = 1 };
  void send_slice(const char* src, const MemoryRegion& mr, size_t bytes, bool signaled);
  void recv_slice(char* dst, size_t elems, DType dtype, RedOp op, bool reduce);
  void wait_flag(uint32_t index, uint32_t target, const char* what);
  void drain();
  void run_threaded(char* bytes, size_t count, size_t esz, size_t slice_elems, DType dtype, RedOp op, const MemoryRegion& mr);
  std::atomic<bool> cancel_{false};   // set when one of the two threads of a call failed: the other one's waits give up

  int rank_, size_, next_, prev_;
  OneSidedTransport* t_;
  Config cfg_;
  const volatile uint32_t* abort_word_;
  size_t slice_bytes_;
  int nslots_;
  char* scratch_ = nullptr;
  std::shared_ptr<MemoryRegion> scratch_mr_;
  RemoteBuffer next_scratch_, next_flags_, prev_flags_;
  uint32_t sent_total_ = 0, recv_total_ = 0;
  std::deque<Request*> pending_;
  RingStats stats_;
};

}  // namespace mnccl
