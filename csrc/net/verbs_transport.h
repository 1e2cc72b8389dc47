// libibverbs provider of the one-sided transport: reliable-connected queue pairs in a full
// mesh, RDMA_WRITE for payload, a 4-byte inline RDMA_WRITE for the flag (delivered after the
// payload because one QP keeps order), selective signalling, one completion queue.  Same
// capability as the reference's transport (reference: src/transport/RDMATransport.h:99-627)
// behind the interface the ring algorithm uses.  Differences: peer information travels through
// the bootstrap store once (no per-call exchange, reference :206-220), completion status is
// checked (reference :349-353 ignores it), unsignalled posts are bounded so the send queue cannot
// overflow (reference: 64 * 16 * 2 outstanding against max_send_wr 1024), waits are bounded, NUMA
// pinning touches the calling thread only.  Compiled only when <infiniband/verbs.h> exists.
#pragma once
#include <infiniband/verbs.h>

#include <deque>
#include <mutex>
#include <vector>

#include "net/reg_cache.h"
#include "net/transport.h"

namespace mnccl {

class VerbsTransport : public OneSidedTransport {
 public:
  VerbsTransport(int rank, int size);
  ~VerbsTransport() override;

  const char* name() const override { return "verbs"; }
  void connect(BootstrapStore& store) override;
  std::shared_ptr<MemoryRegion> register_memory(void* ptr, size_t size) override;
  void invalidate(void* ptr, size_t size) override;
  Request* write(int peer, const void* local, const MemoryRegion& local_mr, RemoteBuffer remote, size_t remote_offset,
                 size_t len, bool signaled) override;
  Request* write_flag(int peer, RemoteBuffer remote_flags, uint32_t index, uint32_t value, bool signaled) override;
  int poll() override;
  volatile uint32_t* flags() override { return flags_; }
  RemoteBuffer flags_remote() const override { return flags_remote_; }
  int max_outstanding() const override { return kSendDepth; }
  const std::string& device_name() const { return device_name_; }

  static constexpr int kSendDepth = 1024;   // max_send_wr, as the reference
  static constexpr int kCqDepth = 4096;
  static constexpr int kForceSignalEvery = 128;  // unsignalled posts per peer before one is signalled anyway

 private:
  struct VerbsRegion : MemoryRegion {
    ibv_mr* mr = nullptr;
    ~VerbsRegion() override;
  };
  struct QpInfo {  // what a peer needs to reach one of our queue pairs
    uint32_t qpn;
    uint32_t psn;
    uint16_t lid;
    uint8_t gid[16];
    uint8_t pad[2];
  };
  void post(int peer, ibv_send_wr* wr, bool* signaled_out);
  void to_init(ibv_qp* qp);
  void to_rtr(ibv_qp* qp, const QpInfo& remote);
  void to_rts(ibv_qp* qp);

  int rank_, size_;
  int timeout_ms_;
  std::string device_name_;
  ibv_context* ctx_ = nullptr;
  ibv_pd* pd_ = nullptr;
  ibv_cq* cq_ = nullptr;
  std::vector<ibv_qp*> qps_;
  std::vector<int> unsignaled_;     // per peer, since the last signalled post
  // Send-queue accounting per peer.  A polled completion retires its own request and every earlier
  // one of the queue pair, not the ones posted after it: requests in flight = posted - retired.
  // Completions of one reliable-connected queue pair arrive in posting order, so a FIFO of the
  // post indices of the signalled requests tells which index a completion stands for.
  std::vector<uint64_t> posted_, retired_;
  std::vector<std::deque<uint64_t>> signaled_at_;
  std::mutex post_mu_;
  uint8_t port_ = 1;
  int gid_index_ = 1;
  uint32_t* flags_ = nullptr;
  std::shared_ptr<MemoryRegion> flags_mr_;
  RemoteBuffer flags_remote_;
  RegistrationCache<MemoryRegion> cache_{4096};
};

}  // namespace mnccl
