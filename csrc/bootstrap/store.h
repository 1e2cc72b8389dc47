// Bootstrap store: a star through rank 0 over TCP that gives every rank
// all_gather / broadcast / barrier on small host blobs.  This replaces both
// rendezvous exchanges of the reference: the static N x N registry exchanged
// once at init and the per-call address exchange (reference:
// src/transport/RDMATransport.h:549-573 and :206-220).  Here it is used at
// init, at symmetric allocation and at destroy only; nothing on the
// AllReduce hot path touches it (the reference runs one exchange per call).
// Default port 8888 as in the reference (:551,566).
#pragma once
#include <cstdint>
#include <mutex>
#include <string>
#include <vector>

#include "bootstrap/socket.h"

namespace mnccl {

class BootstrapStore {
 public:
  BootstrapStore(int rank, int size, std::string root_ip, int port, int timeout_ms,
                 int connect_retries);
  ~BootstrapStore();

  // Rank 0 listens and accepts size-1 peers; the others connect (with retry).
  void connect();

  // in: `bytes` bytes; out: size*bytes, ordered by rank.  Collective.
  void all_gather(const void* in, void* out, size_t bytes);
  // Root's buffer is copied to everyone.  Collective.
  void broadcast(void* buf, size_t bytes, int root = 0);
  void barrier();

  int rank() const { return rank_; }
  int size() const { return size_; }
  // IP address of peer `r` as seen by rank 0 (valid after connect()).
  const std::vector<std::string>& peer_ips() const { return ips_; }

 private:
  int rank_, size_;
  std::string root_ip_;
  int port_, timeout_ms_, retries_;
  TcpListener listener_;
  std::vector<TcpSocket> peers_;  // rank 0: socket to each rank (index = rank); others: [0] = root
  std::vector<std::string> ips_;
  std::mutex mu_;
  uint32_t op_seq_ = 0;
};

}  // namespace mnccl
