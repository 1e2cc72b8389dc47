#include "net/soft_transport.h"

#include <cstdlib>
#include <cstring>
#include <poll.h>

#include "bootstrap/store.h"
#include "core/config.h"
#include "core/error.h"
#include "core/log.h"

namespace mnccl {
namespace {
constexpr uint32_t kFrameMagic = 0x4d4e5346;  // "MNSF"
enum : uint32_t { kWrite = 1, kFlag = 2 };
struct Frame {
  uint32_t magic;
  uint32_t kind;
  uint32_t rkey;
  uint32_t value;
  uint64_t addr;
  uint64_t len;
};
struct Endpoint {
  char ip[64];
  int32_t port;
};
struct Hello {
  uint32_t magic;
  int32_t rank;
};
}  // namespace

SoftTransport::Region::~Region() {
  if (owner) owner->unregister_key(rkey);
}

SoftTransport::SoftTransport(int rank, int size) : rank_(rank), size_(size) {
  timeout_ms_ = Config::get().socket_timeout_ms;
  flags_.reset(new uint32_t[kNumFlags]);
  memset(flags_.get(), 0, sizeof(uint32_t) * kNumFlags);
  if (const char* e = std::getenv("MINI_NCCL_SOFT_DROP_FLAG_AT")) drop_at_.store(std::strtoull(e, nullptr, 10));
}

SoftTransport::~SoftTransport() {
  run_.store(false);
  if (nic_.joinable()) nic_.join();
  flags_mr_.reset();
  cache_.clear();
}

void SoftTransport::connect(BootstrapStore& store) {
  socks_.resize(size_);
  send_mu_.resize(size_);
  for (auto& m : send_mu_) m.reset(new std::mutex);
  dead_ = std::vector<std::atomic<bool>>(size_);
  for (auto& d : dead_) d.store(false);
  flags_mr_ = register_memory(flags_.get(), sizeof(uint32_t) * kNumFlags);
  flags_remote_.addr = reinterpret_cast<uint64_t>(flags_.get());
  flags_remote_.rkey = flags_mr_->rkey;
  if (size_ > 1) {
    TcpListener lis;
    lis.listen_on(0);
    Endpoint me{};
    me.port = lis.port();
    std::vector<Endpoint> all(size_);
    store.all_gather(&me, all.data(), sizeof(me));
    // Lower rank listens, higher rank dials.
    for (int peer = 0; peer < rank_; ++peer) {
      socks_[peer] = TcpSocket::connect_to(store.peer_ips()[peer], all[peer].port, Config::get().connect_retries, 200);
      Hello h{kFrameMagic, rank_};
      socks_[peer].send_all(&h, sizeof(h), timeout_ms_);
    }
    for (int n = rank_ + 1; n < size_; ++n) {
      TcpSocket s = lis.accept_one(timeout_ms_);
      Hello h{};
      s.recv_all(&h, sizeof(h), timeout_ms_);
      if (h.magic != kFrameMagic || h.rank <= rank_ || h.rank >= size_ || socks_[h.rank].valid())
        fail(Result::SystemError, "soft transport: unexpected peer hello");
      socks_[h.rank] = std::move(s);
    }
    store.barrier();
  }
  run_.store(true);
  nic_ = std::thread([this] { nic_loop(); });
}

std::shared_ptr<MemoryRegion> SoftTransport::register_memory(void* ptr, size_t size) {
  uint64_t before = cache_.misses();
  auto mr = cache_.get(ptr, size, [this](void* base, size_t sz) {
    auto r = std::make_shared<Region>();
    r->ptr = base;
    r->size = sz;
    r->owner = this;
    std::lock_guard<std::mutex> lk(key_mu_);
    r->lkey = r->rkey = next_key_++;
    keys_[r->rkey] = {reinterpret_cast<uintptr_t>(base), sz};
    return std::static_pointer_cast<MemoryRegion>(r);
  });
  if (cache_.misses() != before) stats_.reg_misses++; else stats_.reg_hits++;
  return mr;
}

void SoftTransport::invalidate(void* ptr, size_t size) { cache_.invalidate(ptr, size); }

void SoftTransport::unregister_key(uint32_t rkey) {
  std::lock_guard<std::mutex> lk(key_mu_);
  keys_.erase(rkey);
}

void SoftTransport::send_frame(int peer, uint32_t kind, uint32_t rkey, uint32_t value, uint64_t addr,
                               const void* payload, uint64_t len) {
  if (peer < 0 || peer >= size_ || peer == rank_) fail(Result::InvalidArgument, "soft transport: bad peer");
  if (aborted()) fail(Result::InternalError, "transport aborted");
  Frame f{kFrameMagic, kind, rkey, value, addr, len};
  std::lock_guard<std::mutex> lk(*send_mu_[peer]);
  socks_[peer].send_all(&f, sizeof(f), timeout_ms_);
  if (kind == kWrite && len) socks_[peer].send_all(payload, len, timeout_ms_);
}

Request* SoftTransport::write(int peer, const void* local, const MemoryRegion& local_mr, RemoteBuffer remote,
                              size_t remote_offset, size_t len, bool signaled) {
  const uintptr_t l = reinterpret_cast<uintptr_t>(local);
  const uintptr_t b = reinterpret_cast<uintptr_t>(local_mr.ptr);
  if (l < b || l + len > b + local_mr.size) fail(Result::InvalidArgument, "write: local range outside its registered region");
  Request* req = nullptr;
  if (signaled) {
    req = pool_.acquire(stats_.writes.load());
    if (!req) fail(Result::InternalError, "request pool exhausted");
  }
  try {
    send_frame(peer, kWrite, remote.rkey, 0, remote.addr + remote_offset, local, len);
  } catch (...) {
    if (req) pool_.release(req);
    throw;
  }
  stats_.writes++;
  stats_.bytes_written += len;
  if (req) {
    stats_.signaled++;
    req->complete(0);
    reaped_.fetch_add(1);
  }
  return req;
}

Request* SoftTransport::write_flag(int peer, RemoteBuffer remote_flags, uint32_t index, uint32_t value,
                                   bool signaled) {
  if (index >= kNumFlags) fail(Result::InvalidArgument, "flag index out of range");
  Request* req = nullptr;
  if (signaled) {
    req = pool_.acquire(stats_.flag_writes.load());
    if (!req) fail(Result::InternalError, "request pool exhausted");
  }
  uint64_t nth = flag_posts_.fetch_add(1) + 1;
  const bool drop = drop_at_.load() != 0 && nth >= drop_at_.load();
  try {
    if (!drop) send_frame(peer, kFlag, remote_flags.rkey, value, remote_flags.addr + 4ull * index, nullptr, 4);
    else MNCCL_INFO("Mini-NCCL", "soft transport: dropping flag write #%llu (fault injection)", (unsigned long long)nth);
  } catch (...) {
    if (req) pool_.release(req);
    throw;
  }
  stats_.flag_writes++;
  if (req) {
    stats_.signaled++;
    req->complete(0);
    reaped_.fetch_add(1);
  }
  return req;
}

int SoftTransport::poll() { return reaped_.exchange(0); }

bool SoftTransport::handle_frame(int peer) {
  Frame f{};
  if (!socks_[peer].recv_all_or_eof(&f, sizeof(f), timeout_ms_)) return false;
  if (f.magic != kFrameMagic) fail(Result::InternalError, "soft transport: bad frame magic");
  bool ok = false;
  {
    std::lock_guard<std::mutex> lk(key_mu_);
    auto it = keys_.find(f.rkey);
    if (it != keys_.end()) {
      uintptr_t base = it->second.first;
      size_t sz = it->second.second;
      ok = f.addr >= base && f.addr + f.len <= base + sz && f.addr + f.len >= f.addr;
    }
  }
  if (f.kind == kWrite) {
    if (ok) {
      socks_[peer].recv_all(reinterpret_cast<void*>(f.addr), f.len, timeout_ms_);
    } else {
      // Remote access error: swallow the payload, count it (a real NIC would
      // move the QP to the error state).
      access_errors_++;
      stats_.completion_errors++;
      std::vector<char> sink(64 * 1024);
      uint64_t left = f.len;
      while (left) {
        size_t n = left < sink.size() ? static_cast<size_t>(left) : sink.size();
        socks_[peer].recv_all(sink.data(), n, timeout_ms_);
        left -= n;
      }
      MNCCL_WARN("Mini-NCCL", "soft transport: rejected a write from rank %d (bad key or range)", peer);
    }
  } else if (f.kind == kFlag) {
    if (ok && f.len == 4 && (f.addr & 3) == 0) {
      __atomic_store_n(reinterpret_cast<uint32_t*>(f.addr), f.value, __ATOMIC_RELEASE);
    } else {
      access_errors_++;
      stats_.completion_errors++;
    }
  } else {
    fail(Result::InternalError, "soft transport: unknown frame kind");
  }
  return true;
}

void SoftTransport::nic_loop() {
  std::vector<struct pollfd> fds;
  std::vector<int> who;
  while (run_.load()) {
    fds.clear();
    who.clear();
    for (int p = 0; p < size_; ++p) {
      if (p != rank_ && socks_[p].valid() && !dead_[p].load()) {
        fds.push_back({socks_[p].fd(), POLLIN, 0});
        who.push_back(p);
      }
    }
    if (fds.empty()) {
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
      continue;
    }
    int r = ::poll(fds.data(), fds.size(), 20);
    if (r <= 0) continue;
    for (size_t i = 0; i < fds.size(); ++i) {
      if (!(fds[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
      try {
        if (!handle_frame(who[i])) dead_[who[i]].store(true);  // peer went away (destroy or death)
      } catch (const std::exception& e) {
        if (run_.load()) MNCCL_WARN("Mini-NCCL", "soft transport: connection to rank %d failed: %s", who[i], e.what());
        dead_[who[i]].store(true);
      }
    }
  }
}

bool OneSidedTransport::wait(Request* r, int timeout_ms) {
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (!r->completed()) {
    poll();
    if (r->completed()) break;
    if (aborted()) fail(Result::InternalError, "transport aborted while waiting for a completion");
    if (std::chrono::steady_clock::now() >= deadline) return false;
    std::this_thread::yield();
  }
  if (r->status() != 0) {
    stats_.completion_errors++;
    fail(Result::RemoteError, "work request completed with error status " + std::to_string(r->status()));
  }
  return true;
}

}  // namespace mnccl
