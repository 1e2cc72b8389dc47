// File-descriptor passing between the ranks of one host over abstract
// Unix-domain sockets (SCM_RIGHTS).  Used to hand CUDA VMM allocation handles
// and NVSwitch multicast handles (exported as POSIX fds) to peer processes.
// The reference has no counterpart: it tries cudaIpc handles on host-pinned
// memory, which cannot work (reference: src/transport/RDMATransport.h:522-529).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace mnccl {

class FdChannel {
 public:
  // `ns` separates jobs sharing a network namespace; the socket name is
  // "\0mnccl-<ns>-<rank>".
  FdChannel(std::string ns, int rank);
  ~FdChannel();
  FdChannel(const FdChannel&) = delete;
  FdChannel& operator=(const FdChannel&) = delete;

  // Bind + listen on this rank's name.  Must complete on every rank (use a
  // store barrier) before anyone calls send_fd.
  void open();
  // Sends `fd` with a 16-byte tag {src rank, user tag} to `dst_rank`.
  void send_fd(int dst_rank, int fd, uint32_t tag, int timeout_ms);
  // Receives one descriptor; fills src rank and tag.  The caller owns the fd.
  int recv_fd(int* src_rank, uint32_t* tag, int timeout_ms);
  void close();

 private:
  std::string name_for(int rank) const;
  std::string ns_;
  int rank_;
  int listen_fd_ = -1;
};

}  // namespace mnccl
