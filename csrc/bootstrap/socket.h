// Blocking TCP sockets with deadlines.  Covers the reference's bootstrap
// sockets (reference: src/transport/Socket.h:16-107): full-length send/recv,
// TCP_NODELAY, SO_REUSEADDR listener, connect with retries.  Every blocking
// call here takes a timeout (the reference blocks forever in recv).
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>

namespace mnccl {

class TcpSocket {
 public:
  TcpSocket() = default;
  explicit TcpSocket(int fd) : fd_(fd) {}
  ~TcpSocket();
  TcpSocket(TcpSocket&& o) noexcept : fd_(o.fd_) { o.fd_ = -1; }
  TcpSocket& operator=(TcpSocket&& o) noexcept;
  TcpSocket(const TcpSocket&) = delete;
  TcpSocket& operator=(const TcpSocket&) = delete;

  bool valid() const { return fd_ >= 0; }
  int fd() const { return fd_; }
  void close();

  // Full-length transfers.  Throw Error(SystemError) on failure / timeout and
  // Error(RemoteError) when the peer closed the connection.
  void send_all(const void* data, size_t len, int timeout_ms) const;
  void recv_all(void* data, size_t len, int timeout_ms) const;
  // Returns false on orderly shutdown before the first byte; true otherwise.
  bool recv_all_or_eof(void* data, size_t len, int timeout_ms) const;
  // True when at least one byte can be read within timeout_ms.
  bool readable(int timeout_ms) const;

  std::string peer_ip() const;

  // Connect with `retries` attempts spaced `retry_ms` apart.
  static TcpSocket connect_to(const std::string& ip, int port, int retries, int retry_ms);

 private:
  int fd_ = -1;
};

class TcpListener {
 public:
  TcpListener() = default;
  ~TcpListener();
  TcpListener(const TcpListener&) = delete;
  TcpListener& operator=(const TcpListener&) = delete;

  // port 0 picks a free port; the bound port is returned by port().
  void listen_on(int port, int backlog = 128);
  // Throws Error(SystemError) when nothing arrives within timeout_ms
  // (timeout_ms < 0 waits forever).
  TcpSocket accept_one(int timeout_ms);
  // Non-throwing variant: returns an invalid socket on timeout.
  TcpSocket try_accept(int timeout_ms);
  int port() const { return port_; }
  void close();
  bool valid() const { return fd_ >= 0; }

 private:
  int fd_ = -1;
  int port_ = 0;
};

}  // namespace mnccl
