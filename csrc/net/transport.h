// One-sided transport interface for the network (inter-node / no-NVLink) data
// plane: registered memory, RDMA-style write, a 4-byte inline "flag" write that
// is delivered after every earlier write on the same connection, selective
// completion signalling.  It restates the capability of the reference's
// Transport / MemoryRegion / Request classes (reference:
// include/mini_nccl.h:36-69) without the stubbed isend / irecv, and the ring
// algorithm depends on this interface only (the reference downcasts to its
// concrete verbs class, reference: src/mini_nccl.cu:73-74).
//
// Providers: SoftTransport (TCP emulation of one-sided writes, always
// available) and VerbsTransport (libibverbs RC queue pairs, compiled when
// <infiniband/verbs.h> exists).
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>

#include "net/request_pool.h"

namespace mnccl {

class BootstrapStore;

struct MemoryRegion {
  void* ptr = nullptr;
  size_t size = 0;
  uint32_t lkey = 0;
  uint32_t rkey = 0;
  virtual ~MemoryRegion() = default;
};

// What a peer needs to write into a region of ours.
struct RemoteBuffer {
  uint64_t addr = 0;
  uint32_t rkey = 0;
  uint32_t pad = 0;
};

struct TransportStats {
  std::atomic<uint64_t> writes{0}, flag_writes{0}, bytes_written{0}, signaled{0};
  std::atomic<uint64_t> reg_hits{0}, reg_misses{0}, completion_errors{0};
  std::atomic<uint64_t> direct_writes{0};  // payloads that went straight into a same-host peer's memory
  std::atomic<uint64_t> direct_flags{0};   // flags stored straight into a same-host peer's flag page
};

class OneSidedTransport {
 public:
  virtual ~OneSidedTransport() = default;
  virtual const char* name() const = 0;

  // Establish connections to every peer (collective; uses the store).
  virtual void connect(BootstrapStore& store) = 0;

  // Register through the cache.  The returned region covers [ptr, ptr+size).
  virtual std::shared_ptr<MemoryRegion> register_memory(void* ptr, size_t size) = 0;
  virtual void invalidate(void* ptr, size_t size) = 0;

  // One-sided write.  `local` must lie in a registered region.  Returns a
  // request when `signaled` (owned by the caller: poll it, then release()),
  // nullptr otherwise.  Throws when the request pool is exhausted or the
  // connection failed.
  virtual Request* write(int peer, const void* local, const MemoryRegion& local_mr, RemoteBuffer remote,
                         size_t remote_offset, size_t len, bool signaled) = 0;
  // Inline 4-byte write, ordered after all earlier writes to the same peer.
  virtual Request* write_flag(int peer, RemoteBuffer remote_flags, uint32_t index, uint32_t value,
                              bool signaled) = 0;

  // Drive completions.  Returns the number of completions reaped.
  virtual int poll() = 0;
  // Bounded wait for one request; false on timeout.  Throws on completion error.
  bool wait(Request* r, int timeout_ms);
  void release(Request* r) { pool_.release(r); }

  // Flag array peers write into (host memory, registered).  kNumFlags entries.
  static constexpr uint32_t kNumFlags = 1024;
  virtual volatile uint32_t* flags() = 0;
  virtual RemoteBuffer flags_remote() const = 0;

  // Upper bound of posted-but-unreaped work requests per peer.
  virtual int max_outstanding() const = 0;
  // True when one thread may post writes and wait for their completions while another thread posts
  // unsignalled flag writes and polls (the ring's sender thread, net/ring.cc).
  virtual bool concurrent_posting() const { return false; }

  // Makes every blocked wait in this transport return (sticky).
  void abort() { aborted_.store(true, std::memory_order_release); }
  bool aborted() const { return aborted_.load(std::memory_order_acquire); }

  TransportStats& stats() { return stats_; }
  RequestPool& pool() { return pool_; }

 protected:
  RequestPool pool_{4096};
  TransportStats stats_;
  std::atomic<bool> aborted_{false};
};

// Factory: "soft" | "verbs" | "auto" (verbs when compiled in and a device
// exists, else soft).
std::unique_ptr<OneSidedTransport> make_transport(const std::string& kind, int rank, int size);
bool verbs_compiled_in();

}  // namespace mnccl
