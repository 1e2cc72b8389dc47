// Soft one-sided provider: emulates an RDMA NIC over TCP.  A background "NIC"
// thread owns the receive side: it reads {key, address, length} frames from
// every peer connection, checks them against the table of registered regions
// (as a real NIC checks the rkey and bounds) and deposits the payload straight
// into the target memory; a flag frame becomes a 4-byte release store.  TCP
// keeps frames of one connection in order, which gives the "payload before
// flag" guarantee that the reference takes from RC queue pairs (reference:
// src/transport/RDMATransport.h:259-311).  Works between hosts as well as on
// loopback, needs no RDMA hardware, and is the provider the CPU tests use.
//
// Same-host fast path: when a peer runs on this host (same boot, same pid namespace) and the kernel
// permits it, the PAYLOAD of a write goes straight into the peer's memory with process_vm_writev
// (cross-memory attach: one copy instead of two through a socket), after the sender has checked key
// and range against a copy of the peer's region table.  The flag array of every rank lives in a
// POSIX shared-memory page that same-host peers map: a flag for such a peer is ONE release store into
// that page (the payload before it was copied by a system call that has returned, so it is in place),
// instead of a frame that a thread of the receiver has to wake up for; measured on the 8-core build
// machine, 2 processes: 4 MiB fp32 in 2.3 ms with flag frames.  A peer whose payloads have to go
// through the socket (fast path refused) gets its flags through the socket too, behind them.
// MINI_NCCL_SOFT_CMA=0 switches the fast path off.  (The reference's same-host path is CUDA IPC,
// reference: src/transport/RDMATransport.h:583-590; between processes without a GPU this is its
// counterpart.)
#pragma once
#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "bootstrap/socket.h"
#include "net/reg_cache.h"
#include "net/transport.h"

namespace mnccl {

class SoftTransport : public OneSidedTransport {
 public:
  SoftTransport(int rank, int size);
  ~SoftTransport() override;

  const char* name() const override { return "soft"; }
  void connect(BootstrapStore& store) override;
  std::shared_ptr<MemoryRegion> register_memory(void* ptr, size_t size) override;
  void invalidate(void* ptr, size_t size) override;
  Request* write(int peer, const void* local, const MemoryRegion& local_mr, RemoteBuffer remote,
                 size_t remote_offset, size_t len, bool signaled) override;
  Request* write_flag(int peer, RemoteBuffer remote_flags, uint32_t index, uint32_t value,
                      bool signaled) override;
  int poll() override;
  volatile uint32_t* flags() override { return flags_; }
  RemoteBuffer flags_remote() const override { return flags_remote_; }
  int max_outstanding() const override { return 1024; }
  bool concurrent_posting() const override { return true; }  // per-peer send lock, atomic counters, flags are atomic stores

  // Host-side fault injection for tests: from the n-th flag write posted by
  // this rank on (1-based) every flag write is dropped silently, as if the
  // link had gone quiet; 0 disables.  (A single lost flag would be healed by
  // the next one: flags are monotonic counters.)
  void drop_flag_write_at(uint64_t n) { drop_at_.store(n); flag_posts_.store(0); }
  uint64_t remote_access_errors() const { return access_errors_.load(); }
  uint64_t cma_writes() const { return cma_writes_.load(); }
  bool cma_enabled(int peer) const { return peer >= 0 && peer < static_cast<int>(cma_.size()) && cma_[peer].ok; }

 private:
  struct Region : MemoryRegion {
    SoftTransport* owner = nullptr;
    ~Region() override;
  };
  void nic_loop();
  bool handle_frame(int peer);
  void unregister_key(uint32_t rkey);
  void send_frame(int peer, uint32_t kind, uint32_t rkey, uint32_t value, uint64_t addr,
                  const void* payload, uint64_t len);

  int rank_, size_;
  int timeout_ms_;
  std::vector<TcpSocket> socks_;
  std::vector<std::unique_ptr<std::mutex>> send_mu_;
  std::vector<std::atomic<bool>> dead_;  // set by the NIC thread when a peer's connection ended
  uint32_t* flags_ = nullptr;          // kNumFlags words: a shared-memory page (flags_shm_) or heap memory
  bool flags_shm_ = false;
  char flags_name_[48] = {0};          // name of the shared-memory object while peers may still open it
  std::vector<uint32_t*> peer_flags_;  // same-host peers' flag pages as mapped here (null: frames)
  std::vector<RemoteBuffer> peer_flags_remote_;  // what those pages are called by their owners
  std::shared_ptr<MemoryRegion> flags_mr_;
  RemoteBuffer flags_remote_;

  std::mutex key_mu_;
  std::map<uint32_t, std::pair<uintptr_t, size_t>> keys_;
  uint32_t next_key_ = 0x1000;
  RegistrationCache<MemoryRegion> cache_{4096};

  // ---- same-host fast path (cross-memory attach)
  struct KeyEntry {            // one registered region, as peers read it
    uint64_t base, size;
    uint32_t rkey, pad;
  };
  struct KeyTable {            // lives at a fixed address for the life of the transport
    uint64_t generation;       // bumped whenever an entry is removed
    uint32_t count, pad;       // entries [0, count) may be valid (rkey != 0)
    KeyEntry entry[4096 + 64];
  };
  struct CmaPeer {
    bool ok = false;
    int pid = 0;
    uint64_t table_addr = 0;
    uint64_t generation = ~0ull;                              // of the cached copy
    std::map<uint32_t, std::pair<uint64_t, uint64_t>> keys;   // cached: rkey -> (base, size)
  };
  bool cma_read(const CmaPeer& p, uint64_t remote_addr, void* dst, size_t len) const;
  bool cma_refresh(CmaPeer& p);
  // 1: written; 0: rejected (bad key or range); -1: the fast path failed, use the socket
  int cma_write(int peer, const void* local, uint32_t rkey, uint64_t addr, size_t len);
  void table_add(uint32_t rkey, uintptr_t base, size_t size);
  void table_remove(uint32_t rkey);
  std::unique_ptr<KeyTable> table_;
  std::vector<CmaPeer> cma_;
  std::atomic<uint64_t> cma_writes_{0};

  std::atomic<bool> run_{false};
  std::thread nic_;
  std::atomic<int> reaped_{0};
  std::atomic<uint64_t> drop_at_{0}, flag_posts_{0}, access_errors_{0};
};

}  // namespace mnccl
