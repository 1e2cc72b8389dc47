#include "net/ring.h"

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <thread>
#include <vector>

#include "bootstrap/store.h"
#include "core/error.h"
#include "core/log.h"
#include "ref/oracle.h"

namespace mnccl {
namespace {
struct RingEndpoint {
  RemoteBuffer scratch;
  RemoteBuffer flags;
};
}  // namespace

RingAllReduce::RingAllReduce(int rank, int size, OneSidedTransport* transport, BootstrapStore* store,
                             const Config& cfg, const volatile uint32_t* abort_word)
    : rank_(rank), size_(size), next_((rank + 1) % size), prev_((rank - 1 + size) % size), t_(transport),
      cfg_(cfg), abort_word_(abort_word) {
  // Slices hold whole elements of every type: round down to 8 bytes, at least 8.
  slice_bytes_ = std::max<size_t>(8, cfg.slice_size & ~size_t(7));
  nslots_ = std::min(std::max(cfg.window_size, 2), 64);
  size_t total = slice_bytes_ * static_cast<size_t>(nslots_);
  if (posix_memalign(reinterpret_cast<void**>(&scratch_), 4096, total) != 0)
    fail(Result::SystemError, "cannot allocate ring scratch");
  memset(scratch_, 0, total);
  scratch_mr_ = t_->register_memory(scratch_, total);
  RingEndpoint me;
  me.scratch.addr = reinterpret_cast<uint64_t>(scratch_);
  me.scratch.rkey = scratch_mr_->rkey;
  me.flags = t_->flags_remote();
  std::vector<RingEndpoint> all(size);
  store->all_gather(&me, all.data(), sizeof(me));
  next_scratch_ = all[next_].scratch;
  next_flags_ = all[next_].flags;
  prev_flags_ = all[prev_].flags;
}

RingAllReduce::~RingAllReduce() {
  for (Request* r : pending_) t_->release(r);
  pending_.clear();
  if (scratch_) t_->invalidate(scratch_, 0);
  scratch_mr_.reset();
  free(scratch_);
}

void RingAllReduce::wait_flag(uint32_t index, uint32_t target, const char* what) {
  volatile uint32_t* f = t_->flags() + index;
  auto reached = [&] { return static_cast<int32_t>(__atomic_load_n(f, __ATOMIC_ACQUIRE) - target) >= 0; };
  if (reached()) return;
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(cfg_.watchdog_timeout_ms);
  unsigned spins = 0;
  while (!reached()) {
    if (cancel_.load(std::memory_order_relaxed)) fail(Result::InternalError, std::string("the call's other thread failed while waiting for ") + what);
    if (abort_word_ && *abort_word_) fail(Result::InternalError, std::string("aborted while waiting for ") + what);
    if (t_->aborted()) fail(Result::InternalError, std::string("transport aborted while waiting for ") + what);
    if ((++spins & 0x3f) == 0) {
      t_->poll();
      if (std::chrono::steady_clock::now() >= deadline) {
        log_always("Watchdog", "TIMEOUT DETECTED! Aborting the ring (waiting for %s, flag %u < %u)", what,
                   __atomic_load_n(f, __ATOMIC_ACQUIRE), target);
        t_->abort();
        fail(Result::InternalError, "NCCL Watchdog Timeout: Communication hang detected.");
      }
      if (spins > 4096) std::this_thread::yield();
    }
  }
}

void RingAllReduce::send_slice(const char* src, const MemoryRegion& mr, size_t bytes, bool signaled) {
  uint32_t seq = ++sent_total_;
  uint32_t slot = (seq - 1) % static_cast<uint32_t>(nslots_);
  // Credit: the slot is free once the receiver consumed slice seq - nslots.
  uint32_t need = seq - static_cast<uint32_t>(nslots_);
  volatile uint32_t* credit = t_->flags() + kCreditFlag;
  if (static_cast<int32_t>(__atomic_load_n(credit, __ATOMIC_ACQUIRE) - need) < 0) {
    ++stats_.credit_stalls;
    wait_flag(kCreditFlag, need, "a scratch-slot credit");
  }
  t_->write(next_, src, mr, next_scratch_, size_t(slot) * slice_bytes_, bytes, false);
  Request* r = t_->write_flag(next_, next_flags_, kDataFlag, seq, signaled);
  if (r) pending_.push_back(r);
  while (static_cast<int>(pending_.size()) > cfg_.window_size) {
    ++stats_.window_stalls;
    Request* oldest = pending_.front();
    pending_.pop_front();
    bool ok = t_->wait(oldest, cfg_.watchdog_timeout_ms);
    t_->release(oldest);
    if (!ok) fail(Result::InternalError, "NCCL Watchdog Timeout: a send completion never arrived.");
  }
  ++stats_.slices_sent;
  stats_.bytes_sent += bytes;
}

void RingAllReduce::recv_slice(char* dst, size_t elems, DType dtype, RedOp op, bool reduce) {
  uint32_t seq = ++recv_total_;
  uint32_t slot = (seq - 1) % static_cast<uint32_t>(nslots_);
  wait_flag(kDataFlag, seq, "a data slice");
  const char* src = scratch_ + size_t(slot) * slice_bytes_;
  if (reduce) host_reduce_pair(dtype, op, dst, src, elems);
  else memcpy(dst, src, elems * dtype_size(dtype));
  // Tell the sender the slot is free again.
  t_->write_flag(prev_, prev_flags_, kCreditFlag, seq, false);
  ++stats_.slices_received;
}

void RingAllReduce::drain() {
  while (!pending_.empty()) {
    Request* r = pending_.front();
    pending_.pop_front();
    bool ok = t_->wait(r, cfg_.watchdog_timeout_ms);
    t_->release(r);
    if (!ok) fail(Result::InternalError, "NCCL Watchdog Timeout: a send completion never arrived.");
  }
}

void RingAllReduce::run(void* data, size_t count, DType dtype, RedOp op) {
  ++stats_.calls;
  if (count == 0) return;
  const int n = size_;
  if (n == 1) return;  // sum / prod / max / min / avg of one operand is the operand
  const size_t esz = dtype_size(dtype);
  const size_t slice_elems = std::max<size_t>(1, slice_bytes_ / esz);
  const size_t base = count / n, rem = count % n;
  auto chunk_off = [&](int c) { return size_t(c) * base + std::min<size_t>(c, rem); };
  auto chunk_len = [&](int c) { return base + (size_t(c) < rem ? 1 : 0); };
  char* bytes = static_cast<char*>(data);
  std::shared_ptr<MemoryRegion> mr = t_->register_memory(data, count * esz);
  if (cfg_.ring_sender_thread && t_->concurrent_posting() && count * esz >= (size_t(4) << 20)) {
    run_threaded(bytes, count, esz, slice_elems, dtype, op, *mr);
    if (op == RedOp::Avg) host_avg_finalize(dtype, data, count, n);
    return;
  }

  for (int step = 0; step < 2 * (n - 1); ++step) {
    const bool phase1 = step < n - 1;
    const int i = phase1 ? step : step - (n - 1);
    const int send_chunk = phase1 ? (rank_ - i + n) % n : (rank_ + 1 - i + n) % n;
    const int recv_chunk = phase1 ? (rank_ - i - 1 + 2 * n) % n : (rank_ - i + n) % n;
    const size_t send_len = chunk_len(send_chunk), recv_len = chunk_len(recv_chunk);
    const size_t ns_send = (send_len + slice_elems - 1) / slice_elems;
    const size_t ns_recv = (recv_len + slice_elems - 1) / slice_elems;
    const size_t ns = std::max(ns_send, ns_recv);
    // Sends run a few slices ahead of the receives (never more than half the scratch slots), so
    // that the peer always has a slice to work on instead of one slice per round trip.  The chunk
    // sent in a step was completed in the step before, so sending ahead reads final data.
    const size_t ahead = std::min<size_t>(4, static_cast<size_t>(nslots_) / 2);
    size_t sent = 0;
    for (size_t s = 0; s < ns; ++s) {
      while (sent < ns_send && sent <= s + ahead) {
        size_t off = sent * slice_elems;
        size_t ne = std::min(slice_elems, send_len - off);
        bool signaled = (sent % static_cast<size_t>(cfg_.signal_batch) == 0) || (sent + 1 == ns_send);
        send_slice(bytes + (chunk_off(send_chunk) + off) * esz, *mr, ne * esz, signaled);
        ++sent;
      }
      if (s < ns_recv) {
        size_t off = s * slice_elems;
        size_t ne = std::min(slice_elems, recv_len - off);
        recv_slice(bytes + (chunk_off(recv_chunk) + off) * esz, ne, dtype, op, phase1);
      }
    }
    if (step == n - 2 || step == 2 * (n - 1) - 1) drain();  // end of each phase, as the reference does
  }
  if (op == RedOp::Avg) host_avg_finalize(dtype, data, count, n);
}

// The same schedule with the two halves of the work in two threads.  The chunk a rank sends in step s
// is the chunk it received (and, in phase 1, reduced) in step s - 1, cut into the same slices, so slice
// k of step s may go as soon as slice k of step s - 1 has been consumed: the sender thread waits for
// the receiver's counter to reach that slice and otherwise runs freely (credits and the window bound
// it as before).  The sender owns sent_total_, pending_ and the send counters, the receiver owns
// recv_total_; they share the counter and cancel_.
void RingAllReduce::run_threaded(char* bytes, size_t count, size_t esz, size_t slice_elems, DType dtype, RedOp op,
                                 const MemoryRegion& mr) {
  const int n = size_;
  const size_t base = count / n, rem = count % n;
  auto chunk_off = [&](int c) { return size_t(c) * base + std::min<size_t>(c, rem); };
  auto chunk_len = [&](int c) { return base + (size_t(c) < rem ? 1 : 0); };
  auto slices_of = [&](size_t len) { return (len + slice_elems - 1) / slice_elems; };
  const int steps = 2 * (n - 1);
  auto send_chunk_of = [&](int step) { return step < n - 1 ? (rank_ - step + n) % n : (rank_ + 1 - (step - (n - 1)) + n) % n; };
  auto recv_chunk_of = [&](int step) { return step < n - 1 ? (rank_ - step - 1 + 2 * n) % n : (rank_ - (step - (n - 1)) + n) % n; };
  // slices this rank has received before each step
  std::vector<uint64_t> recv_before(steps + 1, 0);
  for (int s = 0; s < steps; ++s) recv_before[s + 1] = recv_before[s] + slices_of(chunk_len(recv_chunk_of(s)));

  std::atomic<uint64_t> received{0};
  std::exception_ptr sender_error;
  bool sender_first = false;   // the sender failed first (the receiver's error is then only the echo); read after join
  cancel_.store(false);
  ++stats_.threaded_calls;
  std::thread sender([&] {
    try {
      for (int step = 0; step < steps; ++step) {
        const int c = send_chunk_of(step);
        const size_t len = chunk_len(c), ns = slices_of(len);
        for (size_t k = 0; k < ns; ++k) {
          if (step > 0) {
            const uint64_t need = recv_before[step - 1] + k + 1;
            unsigned spins = 0;
            while (received.load(std::memory_order_acquire) < need) {
              if (cancel_.load(std::memory_order_relaxed)) fail(Result::InternalError, "the receiving thread of the call failed");
              if ((++spins & 0x3ff) == 0) {
                if ((abort_word_ && *abort_word_) || t_->aborted()) fail(Result::InternalError, "aborted while waiting for a slice to forward");
                std::this_thread::yield();
              }
            }
          }
          const size_t off = k * slice_elems;
          const size_t ne = std::min(slice_elems, len - off);
          const bool signaled = (k % static_cast<size_t>(cfg_.signal_batch) == 0) || (k + 1 == ns);
          send_slice(bytes + (chunk_off(c) + off) * esz, mr, ne * esz, signaled);
        }
        if (step == n - 2 || step == steps - 1) drain();  // end of each phase, as the reference does
      }
    } catch (...) {
      sender_error = std::current_exception();
      if (!cancel_.exchange(true)) sender_first = true;
    }
  });
  std::exception_ptr receiver_error;
  try {
    for (int step = 0; step < steps; ++step) {
      const int c = recv_chunk_of(step);
      const size_t len = chunk_len(c), ns = slices_of(len);
      for (size_t k = 0; k < ns; ++k) {
        const size_t off = k * slice_elems;
        const size_t ne = std::min(slice_elems, len - off);
        recv_slice(bytes + (chunk_off(c) + off) * esz, ne, dtype, op, step < n - 1);
        received.fetch_add(1, std::memory_order_release);
      }
    }
  } catch (...) {
    receiver_error = std::current_exception();
    cancel_.store(true);
  }
  sender.join();
  cancel_.store(false);
  if (sender_error && (sender_first || !receiver_error)) std::rethrow_exception(sender_error);
  if (receiver_error) std::rethrow_exception(receiver_error);
}

}  // namespace mnccl
