// Host watchdog: one thread per communicator.  It reads the progress words the
// kernels write into host-mapped memory ({started, done, status, detail}); when
// a collective has been in flight for longer than the configured bound without
// finishing, or a kernel reported a failed wait, it sets the abort word.  That
// word is shared by every rank of the host and polled by every device-side
// wait, so all local kernels return promptly with an error status instead of
// spinning.  Optionally the trip is forwarded (Hera GLOBAL_ABORT) to other
// hosts through a callback.
//
// The reference runs this check on the calling thread inside every AllReduce,
// which makes the call host-blocking, with a fixed 10 s bound, an abort flag
// local to one rank and no way to learn of the failure except the thrown
// exception (reference: src/mini_nccl.cu:200-216).  The bound is
// MINI_NCCL_WATCHDOG_TIMEOUT_MS here (default 10000).
#pragma once
#include <atomic>
#include <chrono>
#include <cstdint>
#include <functional>
#include <thread>

namespace mnccl {

struct WatchdogStats {
  std::atomic<uint64_t> polls{0}, trips{0}, device_failures{0}, remote_aborts{0};
};

class Watchdog {
 public:
  // progress: this rank's {started, done, status, detail} words (host view).
  // abort_word: the shared abort word (host view).
  Watchdog(volatile uint32_t* progress, volatile uint32_t* abort_word, int timeout_ms, int rank);
  ~Watchdog();
  void start();
  void stop();
  // Called once, from the watchdog thread, when this rank trips (not when it
  // merely observes somebody else's abort).
  void set_on_trip(std::function<void(uint32_t reason)> cb) { on_trip_ = std::move(cb); }
  bool tripped() const { return tripped_.load(); }
  bool saw_abort() const { return saw_abort_.load(); }
  const WatchdogStats& stats() const { return stats_; }
  // One evaluation step with an explicit clock, for unit tests.
  void step(std::chrono::steady_clock::time_point now);

 private:
  void loop();
  volatile uint32_t* progress_;
  volatile uint32_t* abort_;
  int timeout_ms_;
  int rank_;
  std::atomic<bool> run_{false}, tripped_{false}, saw_abort_{false};
  std::thread thread_;
  std::function<void(uint32_t)> on_trip_;
  WatchdogStats stats_;
  uint32_t last_done_ = 0;
  bool in_flight_ = false;
  std::chrono::steady_clock::time_point since_;
};

}  // namespace mnccl
