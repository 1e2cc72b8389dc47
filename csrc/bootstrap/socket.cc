#include "bootstrap/socket.h"

#include <arpa/inet.h>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <thread>
#include <unistd.h>

#include "core/error.h"

namespace mnccl {
namespace {

using Clock = std::chrono::steady_clock;

int remaining_ms(Clock::time_point deadline) {
  auto now = Clock::now();
  if (now >= deadline) return 0;
  return static_cast<int>(std::chrono::duration_cast<std::chrono::milliseconds>(deadline - now).count()) + 1;
}

// Waits for `events` on fd; returns false on timeout.
bool wait_fd(int fd, short events, Clock::time_point deadline, bool forever) {
  for (;;) {
    struct pollfd p = {fd, events, 0};
    int t = forever ? -1 : remaining_ms(deadline);
    int r = ::poll(&p, 1, t);
    if (r > 0) return true;
    if (r == 0) {
      if (forever) continue;
      if (remaining_ms(deadline) == 0) return false;
      continue;
    }
    if (errno == EINTR) continue;
    fail(Result::SystemError, std::string("poll failed: ") + strerror(errno));
  }
}

void set_nodelay(int fd) {
  int one = 1;
  ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}

}  // namespace

TcpSocket::~TcpSocket() { close(); }

TcpSocket& TcpSocket::operator=(TcpSocket&& o) noexcept {
  if (this != &o) {
    close();
    fd_ = o.fd_;
    o.fd_ = -1;
  }
  return *this;
}

void TcpSocket::close() {
  if (fd_ >= 0) {
    ::close(fd_);
    fd_ = -1;
  }
}

void TcpSocket::send_all(const void* data, size_t len, int timeout_ms) const {
  if (fd_ < 0) fail(Result::SystemError, "send on closed socket");
  const char* p = static_cast<const char*>(data);
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  size_t done = 0;
  while (done < len) {
    ssize_t n = ::send(fd_, p + done, len - done, MSG_NOSIGNAL | MSG_DONTWAIT);
    if (n > 0) {
      done += static_cast<size_t>(n);
      continue;
    }
    if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) {
      if (!wait_fd(fd_, POLLOUT, deadline, timeout_ms < 0)) fail(Result::SystemError, "socket send timed out");
      continue;
    }
    if (n < 0 && errno == EINTR) continue;
    if (n < 0 && (errno == EPIPE || errno == ECONNRESET)) fail(Result::RemoteError, "peer closed connection during send");
    fail(Result::SystemError, std::string("socket send failed: ") + strerror(errno));
  }
}

bool TcpSocket::recv_all_or_eof(void* data, size_t len, int timeout_ms) const {
  if (fd_ < 0) fail(Result::SystemError, "recv on closed socket");
  char* p = static_cast<char*>(data);
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  size_t done = 0;
  while (done < len) {
    ssize_t n = ::recv(fd_, p + done, len - done, MSG_DONTWAIT);
    if (n > 0) {
      done += static_cast<size_t>(n);
      continue;
    }
    if (n == 0) {
      if (done == 0) return false;
      fail(Result::RemoteError, "peer closed connection mid-message");
    }
    if (errno == EAGAIN || errno == EWOULDBLOCK) {
      if (!wait_fd(fd_, POLLIN, deadline, timeout_ms < 0)) fail(Result::SystemError, "socket recv timed out");
      continue;
    }
    if (errno == EINTR) continue;
    if (errno == ECONNRESET) fail(Result::RemoteError, "connection reset by peer");
    fail(Result::SystemError, std::string("socket recv failed: ") + strerror(errno));
  }
  return true;
}

void TcpSocket::recv_all(void* data, size_t len, int timeout_ms) const {
  if (len == 0) return;
  if (!recv_all_or_eof(data, len, timeout_ms)) fail(Result::RemoteError, "peer closed connection");
}

bool TcpSocket::readable(int timeout_ms) const {
  if (fd_ < 0) return false;
  struct pollfd p = {fd_, POLLIN, 0};
  int r;
  do { r = ::poll(&p, 1, timeout_ms); } while (r < 0 && errno == EINTR);
  return r > 0;
}

std::string TcpSocket::peer_ip() const {
  struct sockaddr_in addr;
  socklen_t alen = sizeof(addr);
  if (::getpeername(fd_, reinterpret_cast<struct sockaddr*>(&addr), &alen) != 0) return "127.0.0.1";
  char buf[INET_ADDRSTRLEN] = {0};
  if (!inet_ntop(AF_INET, &addr.sin_addr, buf, sizeof(buf))) return "127.0.0.1";
  return buf;
}

TcpSocket TcpSocket::connect_to(const std::string& ip, int port, int retries, int retry_ms) {
  struct sockaddr_in addr;
  memset(&addr, 0, sizeof(addr));
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (inet_pton(AF_INET, ip.c_str(), &addr.sin_addr) != 1) {
    // Not a dotted quad: resolve the name.
    struct addrinfo hints;
    memset(&hints, 0, sizeof(hints));
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    struct addrinfo* res = nullptr;
    if (getaddrinfo(ip.c_str(), nullptr, &hints, &res) != 0 || !res)
      fail(Result::SystemError, "cannot resolve address '" + ip + "'");
    addr.sin_addr = reinterpret_cast<struct sockaddr_in*>(res->ai_addr)->sin_addr;
    freeaddrinfo(res);
  }
  std::string last;
  for (int attempt = 0; attempt < retries; ++attempt) {
    int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) fail(Result::SystemError, std::string("socket() failed: ") + strerror(errno));
    if (::connect(fd, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) == 0) {
      set_nodelay(fd);
      return TcpSocket(fd);
    }
    last = strerror(errno);
    ::close(fd);
    if (attempt + 1 < retries) std::this_thread::sleep_for(std::chrono::milliseconds(retry_ms));
  }
  fail(Result::SystemError, "connect to " + ip + ":" + std::to_string(port) + " failed after " +
                                std::to_string(retries) + " attempts: " + last);
}

TcpListener::~TcpListener() { close(); }

void TcpListener::close() {
  if (fd_ >= 0) {
    ::close(fd_);
    fd_ = -1;
  }
}

void TcpListener::listen_on(int port, int backlog) {
  close();
  fd_ = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd_ < 0) fail(Result::SystemError, std::string("socket() failed: ") + strerror(errno));
  int one = 1;
  ::setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  struct sockaddr_in addr;
  memset(&addr, 0, sizeof(addr));
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (::bind(fd_, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) != 0) {
    std::string e = strerror(errno);
    close();
    fail(Result::SystemError, "bind to port " + std::to_string(port) + " failed: " + e);
  }
  if (::listen(fd_, backlog) != 0) {
    std::string e = strerror(errno);
    close();
    fail(Result::SystemError, "listen failed: " + e);
  }
  socklen_t alen = sizeof(addr);
  ::getsockname(fd_, reinterpret_cast<struct sockaddr*>(&addr), &alen);
  port_ = ntohs(addr.sin_port);
}

TcpSocket TcpListener::try_accept(int timeout_ms) {
  if (fd_ < 0) fail(Result::SystemError, "accept on closed listener");
  struct pollfd p = {fd_, POLLIN, 0};
  int r;
  do { r = ::poll(&p, 1, timeout_ms); } while (r < 0 && errno == EINTR);
  if (r <= 0) return TcpSocket();
  int cfd = ::accept4(fd_, nullptr, nullptr, SOCK_CLOEXEC);
  if (cfd < 0) return TcpSocket();
  set_nodelay(cfd);
  return TcpSocket(cfd);
}

TcpSocket TcpListener::accept_one(int timeout_ms) {
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
  for (;;) {
    int t = timeout_ms < 0 ? 1000 : remaining_ms(deadline);
    TcpSocket s = try_accept(t);
    if (s.valid()) return s;
    if (timeout_ms >= 0 && remaining_ms(deadline) == 0) fail(Result::SystemError, "accept timed out");
  }
}

}  // namespace mnccl
