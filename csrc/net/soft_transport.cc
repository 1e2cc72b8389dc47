#include "net/soft_transport.h"

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <poll.h>
#include <sys/mman.h>
#include <sys/uio.h>
#include <unistd.h>

#include <fstream>
#include <functional>
#include <string>

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
struct CmaInfo {      // what a rank tells the others about its address space
  uint64_t host_id;   // same value = same boot of the same host and the same pid namespace
  uint64_t table_addr;
  int32_t pid;
  int32_t enabled;
  uint64_t flags_addr;   // the flag array in the owner's address space, and its key
  uint32_t flags_rkey;
  uint32_t flags_shared; // 1: the array is the shared-memory object flags_name
  char flags_name[48];
};
constexpr size_t kFlagPageBytes = 2 * 4096;            // flags, then a page with the header below
struct FlagPageHeader {
  uint64_t magic;
  int32_t rank, pid;
};
constexpr uint64_t kFlagPageMagic = 0x4d4e43434c464c47ull;

uint64_t cma_host_id() {
  std::string key;
  char name[256] = {0};
  if (gethostname(name, sizeof(name) - 1) == 0) key += name;
  std::ifstream boot("/proc/sys/kernel/random/boot_id");
  std::string line;
  if (boot && std::getline(boot, line)) key += line;
  char buf[128];
  ssize_t n = readlink("/proc/self/ns/pid", buf, sizeof(buf) - 1);
  if (n > 0) key.append(buf, static_cast<size_t>(n));
  return std::hash<std::string>{}(key) | 1ull;
}
}  // namespace

SoftTransport::Region::~Region() {
  if (owner) owner->unregister_key(rkey);
}

SoftTransport::SoftTransport(int rank, int size) : rank_(rank), size_(size) {
  timeout_ms_ = Config::get().socket_timeout_ms;
  static_assert(sizeof(uint32_t) * kNumFlags <= 4096, "the flag array fits the first page");
  // The flag array: a shared-memory page that same-host peers can map (see the header), else heap memory.
  snprintf(flags_name_, sizeof(flags_name_), "/mnccl-fl-%d-%d-%08x", static_cast<int>(getpid()), rank,
           static_cast<unsigned>(std::chrono::steady_clock::now().time_since_epoch().count()));
  int fd = shm_open(flags_name_, O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd >= 0) {
    void* m = ftruncate(fd, kFlagPageBytes) == 0 ? mmap(nullptr, kFlagPageBytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0) : MAP_FAILED;
    close(fd);
    if (m != MAP_FAILED) {
      flags_ = static_cast<uint32_t*>(m);
      flags_shm_ = true;
      memset(m, 0, kFlagPageBytes);
      FlagPageHeader* h = reinterpret_cast<FlagPageHeader*>(static_cast<char*>(m) + 4096);
      h->rank = rank;
      h->pid = static_cast<int32_t>(getpid());
      __atomic_store_n(&h->magic, kFlagPageMagic, __ATOMIC_RELEASE);
    } else {
      shm_unlink(flags_name_);
    }
  }
  if (!flags_shm_) {
    flags_name_[0] = 0;
    flags_ = new uint32_t[kNumFlags];
    memset(flags_, 0, sizeof(uint32_t) * kNumFlags);
  }
  table_.reset(new KeyTable());
  memset(table_.get(), 0, sizeof(KeyTable));
  if (const char* e = std::getenv("MINI_NCCL_SOFT_DROP_FLAG_AT")) drop_at_.store(std::strtoull(e, nullptr, 10));
}

SoftTransport::~SoftTransport() {
  run_.store(false);
  if (nic_.joinable()) nic_.join();
  flags_mr_.reset();
  cache_.clear();
  for (uint32_t* p : peer_flags_)
    if (p) munmap(p, kFlagPageBytes);
  if (flags_shm_) {
    if (flags_name_[0]) shm_unlink(flags_name_);
    munmap(flags_, kFlagPageBytes);
  } else {
    delete[] flags_;
  }
}

void SoftTransport::connect(BootstrapStore& store) {
  socks_.resize(size_);
  send_mu_.resize(size_);
  for (auto& m : send_mu_) m.reset(new std::mutex);
  dead_ = std::vector<std::atomic<bool>>(size_);
  for (auto& d : dead_) d.store(false);
  flags_mr_ = register_memory(flags_, sizeof(uint32_t) * kNumFlags);
  flags_remote_.addr = reinterpret_cast<uint64_t>(flags_);
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
    // Same-host fast path: who shares this host's memory, and may we touch it?
    const char* env = std::getenv("MINI_NCCL_SOFT_CMA");
    CmaInfo mine{};
    mine.host_id = cma_host_id();
    mine.table_addr = reinterpret_cast<uint64_t>(table_.get());
    mine.pid = static_cast<int32_t>(getpid());
    mine.enabled = (env && env[0] == '0') ? 0 : 1;
    mine.flags_addr = flags_remote_.addr;
    mine.flags_rkey = flags_remote_.rkey;
    mine.flags_shared = flags_shm_ ? 1 : 0;
    memcpy(mine.flags_name, flags_name_, sizeof(mine.flags_name));
    std::vector<CmaInfo> infos(size_);
    store.all_gather(&mine, infos.data(), sizeof(mine));
    cma_.assign(size_, CmaPeer());
    peer_flags_.assign(size_, nullptr);
    peer_flags_remote_.assign(size_, RemoteBuffer());
    int n_cma = 0;
    for (int p = 0; p < size_; ++p) {
      if (p == rank_ || !mine.enabled || !infos[p].enabled || infos[p].host_id != mine.host_id) continue;
      cma_[p].pid = infos[p].pid;
      cma_[p].table_addr = infos[p].table_addr;
      cma_[p].ok = true;
      if (!cma_refresh(cma_[p])) cma_[p].ok = false;  // the probe: not permitted here (ptrace policy) -> sockets
      if (cma_[p].ok) ++n_cma;
      // the peer's flag page: only together with the payload fast path (a flag must never overtake a
      // payload that is still in a socket)
      if (cma_[p].ok && infos[p].flags_shared) {
        infos[p].flags_name[sizeof(infos[p].flags_name) - 1] = 0;
        int pfd = shm_open(infos[p].flags_name, O_RDWR, 0600);
        if (pfd >= 0) {
          void* m = mmap(nullptr, kFlagPageBytes, PROT_READ | PROT_WRITE, MAP_SHARED, pfd, 0);
          close(pfd);
          if (m != MAP_FAILED) {
            const FlagPageHeader* h = reinterpret_cast<const FlagPageHeader*>(static_cast<const char*>(m) + 4096);
            if (__atomic_load_n(&h->magic, __ATOMIC_ACQUIRE) == kFlagPageMagic && h->rank == p && h->pid == infos[p].pid) {
              peer_flags_[p] = static_cast<uint32_t*>(m);
              peer_flags_remote_[p].addr = infos[p].flags_addr;
              peer_flags_remote_[p].rkey = infos[p].flags_rkey;
            } else {
              munmap(m, kFlagPageBytes);
            }
          }
        }
      }
    }
    if (n_cma) MNCCL_INFO("Mini-NCCL", "soft transport: cross-memory attach to %d same-host peer(s)", n_cma);
    store.barrier();
    // every peer that wanted the page has mapped it: the name can go
    if (flags_shm_ && flags_name_[0]) {
      shm_unlink(flags_name_);
      flags_name_[0] = 0;
    }
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
    table_add(r->rkey, reinterpret_cast<uintptr_t>(base), sz);
    return std::static_pointer_cast<MemoryRegion>(r);
  });
  if (cache_.misses() != before) stats_.reg_misses++; else stats_.reg_hits++;
  return mr;
}

void SoftTransport::invalidate(void* ptr, size_t size) { cache_.invalidate(ptr, size); }

void SoftTransport::unregister_key(uint32_t rkey) {
  std::lock_guard<std::mutex> lk(key_mu_);
  keys_.erase(rkey);
  table_remove(rkey);
}

// ---- same-host fast path ------------------------------------------------------------------------

// Callers hold key_mu_.  Entry fields are written before the key that makes the entry valid, and a
// key is only handed to a peer after the registration returned, so a reader never needs a lock.
void SoftTransport::table_add(uint32_t rkey, uintptr_t base, size_t size) {
  KeyTable* t = table_.get();
  const uint32_t cap = static_cast<uint32_t>(sizeof(t->entry) / sizeof(t->entry[0]));
  uint32_t slot = t->count;
  for (uint32_t i = 0; i < t->count; ++i)
    if (__atomic_load_n(&t->entry[i].rkey, __ATOMIC_RELAXED) == 0) { slot = i; break; }
  if (slot >= cap) return;  // table full: writes with this key fall back to the socket (key not found)
  t->entry[slot].base = base;
  t->entry[slot].size = size;
  __atomic_store_n(&t->entry[slot].rkey, rkey, __ATOMIC_RELEASE);
  if (slot == t->count) __atomic_store_n(&t->count, t->count + 1, __ATOMIC_RELEASE);
}

void SoftTransport::table_remove(uint32_t rkey) {
  KeyTable* t = table_.get();
  for (uint32_t i = 0; i < t->count; ++i)
    if (t->entry[i].rkey == rkey) {
      __atomic_store_n(&t->entry[i].rkey, 0u, __ATOMIC_RELEASE);
      __atomic_store_n(&t->generation, t->generation + 1, __ATOMIC_RELEASE);
      return;
    }
}

bool SoftTransport::cma_read(const CmaPeer& p, uint64_t remote_addr, void* dst, size_t len) const {
  size_t done = 0;
  while (done < len) {
    struct iovec l{static_cast<char*>(dst) + done, len - done};
    struct iovec r{reinterpret_cast<void*>(remote_addr + done), len - done};
    ssize_t n = process_vm_readv(p.pid, &l, 1, &r, 1, 0);
    if (n <= 0) return false;
    done += static_cast<size_t>(n);
  }
  return true;
}

// Fetch the peer's region table (header first, then the live entries) into the cache.
bool SoftTransport::cma_refresh(CmaPeer& p) {
  struct { uint64_t generation; uint32_t count, pad; } head;
  if (!cma_read(p, p.table_addr, &head, sizeof(head))) return false;
  const uint32_t cap = static_cast<uint32_t>(sizeof(KeyTable::entry) / sizeof(KeyEntry));
  if (head.count > cap) return false;
  std::vector<KeyEntry> entries(head.count);
  if (head.count && !cma_read(p, p.table_addr + offsetof(KeyTable, entry), entries.data(), sizeof(KeyEntry) * head.count))
    return false;
  p.keys.clear();
  for (const KeyEntry& e : entries)
    if (e.rkey != 0) p.keys[e.rkey] = {e.base, e.size};
  p.generation = head.generation;
  return true;
}

int SoftTransport::cma_write(int peer, const void* local, uint32_t rkey, uint64_t addr, size_t len) {
  CmaPeer& p = cma_[peer];
  // A removed region bumps the generation: one 8-byte read tells whether the cached table is current.
  uint64_t gen = 0;
  if (!cma_read(p, p.table_addr, &gen, sizeof(gen))) return -1;
  auto it = p.keys.find(rkey);
  if (gen != p.generation || it == p.keys.end()) {
    if (!cma_refresh(p)) return -1;
    it = p.keys.find(rkey);
  }
  if (it == p.keys.end()) return 0;
  const uint64_t base = it->second.first, size = it->second.second;
  if (addr < base || addr + len > base + size || addr + len < addr) return 0;
  size_t done = 0;
  while (done < len) {
    struct iovec l{const_cast<char*>(static_cast<const char*>(local)) + done, len - done};
    struct iovec r{reinterpret_cast<void*>(addr + done), len - done};
    ssize_t n = process_vm_writev(p.pid, &l, 1, &r, 1, 0);
    if (n <= 0) return done == 0 ? -1 : 0;  // nothing moved: try the socket; partly moved: report an error
    done += static_cast<size_t>(n);
  }
  return 1;
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
  int status = 0;
  try {
    int fast = -1;
    if (len && peer >= 0 && peer < static_cast<int>(cma_.size()) && cma_[peer].ok) {
      if (aborted()) fail(Result::InternalError, "transport aborted");
      std::lock_guard<std::mutex> lk(*send_mu_[peer]);  // the cached table copy belongs to one poster at a time
      fast = cma_write(peer, local, remote.rkey, remote.addr + remote_offset, len);
      if (fast < 0) cma_[peer].ok = false;              // not permitted after all: sockets from now on
    }
    if (fast == 1) {
      cma_writes_++;
      stats_.direct_writes++;
    } else if (fast == 0) {
      // what the receiver's check would have found: a remote access error, seen by the poster
      access_errors_++;
      stats_.completion_errors++;
      status = 10;
      MNCCL_WARN("Mini-NCCL", "soft transport: write to rank %d rejected (bad key or range)", peer);
    } else {
      send_frame(peer, kWrite, remote.rkey, 0, remote.addr + remote_offset, local, len);
    }
  } catch (...) {
    if (req) pool_.release(req);
    throw;
  }
  stats_.writes++;
  stats_.bytes_written += len;
  if (req) {
    stats_.signaled++;
    req->complete(status);
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
    // Same-host peer whose payloads go straight into its memory: so does the flag, with one release
    // store (every payload posted before it was copied by a system call that has returned).
    uint32_t* page = (!drop && peer >= 0 && peer < static_cast<int>(peer_flags_.size()) && cma_[peer].ok) ? peer_flags_[peer] : nullptr;
    if (page && remote_flags.addr == peer_flags_remote_[peer].addr && remote_flags.rkey == peer_flags_remote_[peer].rkey) {
      if (aborted()) fail(Result::InternalError, "transport aborted");
      __atomic_store_n(page + index, value, __ATOMIC_RELEASE);
      stats_.direct_flags++;
    } else if (!drop) send_frame(peer, kFlag, remote_flags.rkey, value, remote_flags.addr + 4ull * index, nullptr, 4);
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
  auto last_frame = std::chrono::steady_clock::now() - std::chrono::seconds(1);
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
    // While frames keep coming the thread looks again at once: waking a sleeping thread costs more
    // than a whole slice takes.  After kSpinUs without traffic it blocks in poll() again.
    constexpr int kSpinUs = 100;
    int r = ::poll(fds.data(), fds.size(), 0);
    if (r <= 0) {
      if (std::chrono::steady_clock::now() - last_frame < std::chrono::microseconds(kSpinUs)) continue;
      r = ::poll(fds.data(), fds.size(), 20);
      if (r <= 0) continue;
    }
    last_frame = std::chrono::steady_clock::now();
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
