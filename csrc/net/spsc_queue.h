// Bounded single-producer / single-consumer ring.  Same contract as the
// reference's queue (reference: src/transport/LockFreeQueue.h:9-61): capacity
// N usable slots, non-blocking push / pop, acquire-release ordering, head and
// tail on separate cache lines.  Capacity is rounded up to a power of two here
// so that the wrap is a mask instead of a modulo.
#pragma once
#include <atomic>
#include <cstddef>
#include <memory>
#include <new>
#include <utility>

namespace mnccl {

template <typename T>
class SpscQueue {
 public:
  explicit SpscQueue(size_t capacity) {
    size_t n = 2;
    while (n < capacity + 1) n <<= 1;  // one slot stays empty to tell full from empty
    mask_ = n - 1;
    slots_.reset(new T[n]);
  }
  SpscQueue(const SpscQueue&) = delete;
  SpscQueue& operator=(const SpscQueue&) = delete;

  // Producer side.  False when full.
  bool push(const T& v) {
    const size_t t = tail_.load(std::memory_order_relaxed);
    const size_t next = (t + 1) & mask_;
    if (__builtin_expect(next == head_.load(std::memory_order_acquire), 0)) return false;
    slots_[t] = v;
    tail_.store(next, std::memory_order_release);
    return true;
  }
  // Consumer side.  False when empty.
  bool pop(T* out) {
    const size_t h = head_.load(std::memory_order_relaxed);
    if (h == tail_.load(std::memory_order_acquire)) return false;
    *out = std::move(slots_[h]);
    head_.store((h + 1) & mask_, std::memory_order_release);
    return true;
  }
  bool empty() const {
    return head_.load(std::memory_order_acquire) == tail_.load(std::memory_order_acquire);
  }
  size_t size() const {
    const size_t h = head_.load(std::memory_order_acquire);
    const size_t t = tail_.load(std::memory_order_acquire);
    return (t - h) & mask_;
  }
  size_t capacity() const { return mask_; }

 private:
  alignas(64) std::atomic<size_t> head_{0};
  alignas(64) std::atomic<size_t> tail_{0};
  alignas(64) size_t mask_ = 0;
  std::unique_ptr<T[]> slots_;
};

}  // namespace mnccl
