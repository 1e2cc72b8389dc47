// Registration cache: pointer -> registration handle, so that a buffer that is
// used again costs a map lookup instead of a registration.  Same role as the
// reference's MR cache (reference: src/transport/RDMATransport.h:316-334): a
// hit needs the cached range to cover the request, otherwise the entry is
// replaced.  Added here: interval lookup (a pointer inside a cached range
// hits), a capacity with least-recently-used eviction, explicit invalidation
// for freed buffers (the reference documents their absence as a limitation,
// reference: README.md:157) and hit / miss counters.  Used for soft-transport
// keys, verbs MRs and CUDA IPC handles of user buffers alike.
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <list>
#include <map>
#include <memory>
#include <mutex>

namespace mnccl {

template <typename Handle>
class RegistrationCache {
 public:
  using Factory = std::function<std::shared_ptr<Handle>(void* base, size_t size)>;

  explicit RegistrationCache(size_t capacity = 1024) : capacity_(capacity ? capacity : 1) {}

  // Returns a handle whose range covers [ptr, ptr+size).  `make` is called on
  // a miss with the exact range requested.
  std::shared_ptr<Handle> get(void* ptr, size_t size, const Factory& make) {
    std::lock_guard<std::mutex> lk(mu_);
    const uintptr_t p = reinterpret_cast<uintptr_t>(ptr);
    auto it = entries_.upper_bound(p);
    if (it != entries_.begin()) {
      --it;
      Entry& e = it->second;
      if (p >= it->first && p + size <= it->first + e.size) {
        ++hits_;
        lru_.splice(lru_.begin(), lru_, e.lru_it);
        return e.handle;
      }
      // Same base but too small: replace (the reference's "erase and re-register").
      if (it->first == p) erase_locked(it);
    }
    ++misses_;
    std::shared_ptr<Handle> h = make(ptr, size);
    // Drop entries the new range overlaps: they describe memory that has been
    // freed and reallocated.
    for (auto ov = entries_.lower_bound(p); ov != entries_.end() && ov->first < p + size;) {
      auto dead = ov++;
      erase_locked(dead);
    }
    while (entries_.size() >= capacity_ && !lru_.empty()) {
      auto victim = entries_.find(lru_.back());
      if (victim == entries_.end()) { lru_.pop_back(); continue; }
      ++evictions_;
      erase_locked(victim);
    }
    lru_.push_front(p);
    entries_[p] = Entry{size, h, lru_.begin()};
    return h;
  }

  // Forget every entry that overlaps [ptr, ptr+size) (size 0: the entry
  // containing ptr).  Call when the buffer is freed.
  size_t invalidate(void* ptr, size_t size = 0) {
    std::lock_guard<std::mutex> lk(mu_);
    const uintptr_t p = reinterpret_cast<uintptr_t>(ptr);
    const uintptr_t end = p + (size ? size : 1);
    size_t n = 0;
    auto it = entries_.upper_bound(p);
    if (it != entries_.begin()) --it;
    while (it != entries_.end() && it->first < end) {
      auto cur = it++;
      if (cur->first + cur->second.size > p) {
        erase_locked(cur);
        ++n;
      }
    }
    return n;
  }

  void clear() {
    std::lock_guard<std::mutex> lk(mu_);
    entries_.clear();
    lru_.clear();
  }
  size_t size() const { std::lock_guard<std::mutex> lk(mu_); return entries_.size(); }
  uint64_t hits() const { return hits_; }
  uint64_t misses() const { return misses_; }
  uint64_t evictions() const { return evictions_; }

 private:
  struct Entry {
    size_t size;
    std::shared_ptr<Handle> handle;
    std::list<uintptr_t>::iterator lru_it;
  };
  void erase_locked(typename std::map<uintptr_t, Entry>::iterator it) {
    lru_.erase(it->second.lru_it);
    entries_.erase(it);
  }
  mutable std::mutex mu_;
  size_t capacity_;
  std::map<uintptr_t, Entry> entries_;
  std::list<uintptr_t> lru_;
  uint64_t hits_ = 0, misses_ = 0, evictions_ = 0;
};

}  // namespace mnccl
