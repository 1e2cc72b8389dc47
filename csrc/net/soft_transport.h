// Soft one-sided provider: emulates an RDMA NIC over TCP.  A background "NIC"
// thread owns the receive side: it reads {key, address, length} frames from
// every peer connection, checks them against the table of registered regions
// (as a real NIC checks the rkey and bounds) and deposits the payload straight
// into the target memory; a flag frame becomes a 4-byte release store.  TCP
// keeps frames of one connection in order, which gives the "payload before
// flag" guarantee that the reference takes from RC queue pairs (reference:
// src/transport/RDMATransport.h:259-311).  Works between hosts as well as on
// loopback, needs no RDMA hardware, and is the provider the CPU tests use.
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
  volatile uint32_t* flags() override { return flags_.get(); }
  RemoteBuffer flags_remote() const override { return flags_remote_; }
  int max_outstanding() const override { return 1024; }

  // Host-side fault injection for tests: from the n-th flag write posted by
  // this rank on (1-based) every flag write is dropped silently, as if the
  // link had gone quiet; 0 disables.  (A single lost flag would be healed by
  // the next one: flags are monotonic counters.)
  void drop_flag_write_at(uint64_t n) { drop_at_.store(n); flag_posts_.store(0); }
  uint64_t remote_access_errors() const { return access_errors_.load(); }

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
  std::unique_ptr<uint32_t[]> flags_;
  std::shared_ptr<MemoryRegion> flags_mr_;
  RemoteBuffer flags_remote_;

  std::mutex key_mu_;
  std::map<uint32_t, std::pair<uintptr_t, size_t>> keys_;
  uint32_t next_key_ = 0x1000;
  RegistrationCache<MemoryRegion> cache_{4096};

  std::atomic<bool> run_{false};
  std::thread nic_;
  std::atomic<int> reaped_{0};
  std::atomic<uint64_t> drop_at_{0}, flag_posts_{0}, access_errors_{0};
};

}  // namespace mnccl
