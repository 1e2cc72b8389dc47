#include "watchdog/watchdog.h"

#include "core/log.h"

namespace mnccl {

Watchdog::Watchdog(volatile uint32_t* progress, volatile uint32_t* abort_word, int timeout_ms, int rank)
    : progress_(progress), abort_(abort_word), timeout_ms_(timeout_ms), rank_(rank) {}

Watchdog::~Watchdog() { stop(); }

void Watchdog::start() {
  if (run_.exchange(true)) return;
  thread_ = std::thread([this] { loop(); });
}

void Watchdog::stop() {
  run_.store(false);
  if (thread_.joinable()) thread_.join();
}

void Watchdog::step(std::chrono::steady_clock::time_point now) {
  stats_.polls++;
  const uint32_t started = __atomic_load_n(progress_ + 0, __ATOMIC_ACQUIRE);
  const uint32_t done = __atomic_load_n(progress_ + 1, __ATOMIC_ACQUIRE);
  const uint32_t status = __atomic_load_n(progress_ + 2, __ATOMIC_ACQUIRE);
  // kernels that fuse a GEMM with a collective count themselves in words 4 and 5
  const uint32_t fused_started = __atomic_load_n(progress_ + 4, __ATOMIC_ACQUIRE);
  const uint32_t fused_done = __atomic_load_n(progress_ + 5, __ATOMIC_ACQUIRE);
  if (__atomic_load_n(abort_, __ATOMIC_ACQUIRE) != 0 && !saw_abort_.exchange(true)) {
    if (!tripped_.load()) stats_.remote_aborts++;
  }
  if (status != 0 && !tripped_.load()) {
    // A device-side wait gave up: make every other local kernel give up too.
    stats_.device_failures++;
    tripped_.store(true);
    log_always("Watchdog", "rank %d: a kernel reported status %u (detail 0x%x). Aborting GPU kernels...", rank_, status,
               __atomic_load_n(progress_ + 3, __ATOMIC_ACQUIRE));
    __atomic_store_n(abort_, 1u, __ATOMIC_RELEASE);
    if (on_trip_) on_trip_(status);
    return;
  }
  const bool busy = started != done || fused_started != fused_done;
  const uint32_t finished = done + fused_done;  // any kernel finishing is progress
  if (!busy) {
    in_flight_ = false;
    last_done_ = finished;
    return;
  }
  if (!in_flight_ || finished != last_done_) {
    in_flight_ = true;
    last_done_ = finished;
    since_ = now;
    return;
  }
  const auto stuck_ms = std::chrono::duration_cast<std::chrono::milliseconds>(now - since_).count();
  if (stuck_ms > timeout_ms_ && !tripped_.load()) {
    stats_.trips++;
    tripped_.store(true);
    log_always("Watchdog", "TIMEOUT DETECTED! Aborting GPU kernels... (rank %d, collective %u in flight for %lld ms)", rank_,
               started, static_cast<long long>(stuck_ms));
    __atomic_store_n(abort_, 1u, __ATOMIC_RELEASE);
    if (on_trip_) on_trip_(1);
  }
}

void Watchdog::loop() {
  while (run_.load()) {
    step(std::chrono::steady_clock::now());
    std::this_thread::sleep_for(std::chrono::milliseconds(timeout_ms_ < 200 ? 1 : 5));
  }
}

}  // namespace mnccl
