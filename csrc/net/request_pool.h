// Pre-allocated completion requests: no allocation on the send path.  The
// reference keeps 4096 pre-built requests and an SPSC queue of free indices
// (reference: src/transport/RDMATransport.h:336-347,394-400); so does this
// pool.  Differences: exhaustion is an error the caller sees (the reference
// returns nullptr and the caller drops it), completion carries a status (the
// reference ignores the CQE status), and wait() is bounded.
#pragma once
#include <atomic>
#include <chrono>
#include <cstdint>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "core/error.h"
#include "net/spsc_queue.h"

namespace mnccl {

class RequestPool;

class Request {
 public:
  uint64_t wr_id() const { return wr_id_; }
  bool completed() const { return done_.load(std::memory_order_acquire); }
  int status() const { return status_.load(std::memory_order_acquire); }  // 0 = ok
  // Provider side.
  void complete(int status) {
    status_.store(status, std::memory_order_release);
    done_.store(true, std::memory_order_release);
  }

 private:
  friend class RequestPool;
  uint64_t wr_id_ = 0;
  uint32_t index_ = 0;
  std::atomic<bool> done_{false};
  std::atomic<int> status_{0};
};

class RequestPool {
 public:
  explicit RequestPool(size_t n = 4096) : slots_(n), free_(n) {
    for (uint32_t i = 0; i < n; ++i) {
      slots_[i].index_ = i;
      free_.push(i);
    }
  }
  // nullptr when exhausted; callers turn that into an error.
  Request* acquire(uint64_t wr_id) {
    std::lock_guard<std::mutex> lk(acquire_mu_);  // many posting threads -> one consumer at a time
    uint32_t idx;
    if (!free_.pop(&idx)) return nullptr;
    Request* r = &slots_[idx];
    r->wr_id_ = wr_id;
    r->done_.store(false, std::memory_order_relaxed);
    r->status_.store(0, std::memory_order_relaxed);
    return r;
  }
  void release(Request* r) {
    std::lock_guard<std::mutex> lk(release_mu_);
    free_.push(r->index_);
  }
  size_t available() const { return free_.size(); }
  size_t capacity() const { return slots_.size(); }

 private:
  std::vector<Request> slots_;
  SpscQueue<uint32_t> free_;
  std::mutex acquire_mu_, release_mu_;
};

}  // namespace mnccl
