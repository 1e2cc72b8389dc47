#include "bootstrap/fdpass.h"

#include <cerrno>
#include <chrono>
#include <cstring>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <thread>
#include <unistd.h>

#include "core/error.h"

namespace mnccl {
namespace {
struct Tag {
  uint32_t magic;
  int32_t src;
  uint32_t tag;
  uint32_t pad;
};
constexpr uint32_t kMagic = 0x4d4e4644;  // "MNFD"

socklen_t fill_addr(struct sockaddr_un* a, const std::string& name) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  // Abstract namespace: sun_path[0] == 0.
  size_t n = name.size();
  if (n + 1 > sizeof(a->sun_path)) n = sizeof(a->sun_path) - 1;
  memcpy(a->sun_path + 1, name.data(), n);
  return static_cast<socklen_t>(offsetof(struct sockaddr_un, sun_path) + 1 + n);
}
}  // namespace

FdChannel::FdChannel(std::string ns, int rank) : ns_(std::move(ns)), rank_(rank) {}
FdChannel::~FdChannel() { close(); }

std::string FdChannel::name_for(int rank) const { return "mnccl-" + ns_ + "-" + std::to_string(rank); }

void FdChannel::open() {
  close();
  listen_fd_ = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (listen_fd_ < 0) fail(Result::SystemError, std::string("unix socket() failed: ") + strerror(errno));
  struct sockaddr_un a;
  socklen_t len = fill_addr(&a, name_for(rank_));
  if (::bind(listen_fd_, reinterpret_cast<struct sockaddr*>(&a), len) != 0) {
    std::string e = strerror(errno);
    close();
    fail(Result::SystemError, "unix bind failed (" + name_for(rank_) + "): " + e);
  }
  if (::listen(listen_fd_, 64) != 0) {
    std::string e = strerror(errno);
    close();
    fail(Result::SystemError, "unix listen failed: " + e);
  }
}

void FdChannel::close() {
  if (listen_fd_ >= 0) {
    ::close(listen_fd_);
    listen_fd_ = -1;
  }
}

void FdChannel::send_fd(int dst_rank, int fd, uint32_t tag, int timeout_ms) {
  int s = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (s < 0) fail(Result::SystemError, std::string("unix socket() failed: ") + strerror(errno));
  struct sockaddr_un a;
  socklen_t len = fill_addr(&a, name_for(dst_rank));
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    if (::connect(s, reinterpret_cast<struct sockaddr*>(&a), len) == 0) break;
    if (std::chrono::steady_clock::now() >= deadline) {
      std::string e = strerror(errno);
      ::close(s);
      fail(Result::SystemError, "unix connect to rank " + std::to_string(dst_rank) + " failed: " + e);
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
  Tag t{kMagic, rank_, tag, 0};
  struct iovec iov = {&t, sizeof(t)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  ssize_t n;
  do { n = ::sendmsg(s, &msg, MSG_NOSIGNAL); } while (n < 0 && errno == EINTR);
  std::string e = n < 0 ? strerror(errno) : "";
  ::close(s);
  if (n != static_cast<ssize_t>(sizeof(t))) fail(Result::SystemError, "sendmsg(SCM_RIGHTS) failed: " + e);
}

int FdChannel::recv_fd(int* src_rank, uint32_t* tag, int timeout_ms) {
  if (listen_fd_ < 0) fail(Result::SystemError, "fd channel not open");
  struct pollfd p = {listen_fd_, POLLIN, 0};
  int r;
  do { r = ::poll(&p, 1, timeout_ms); } while (r < 0 && errno == EINTR);
  if (r <= 0) fail(Result::SystemError, "timed out waiting for a peer's file descriptor");
  int s = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
  if (s < 0) fail(Result::SystemError, std::string("unix accept failed: ") + strerror(errno));
  Tag t{};
  struct iovec iov = {&t, sizeof(t)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  struct pollfd q = {s, POLLIN, 0};
  do { r = ::poll(&q, 1, timeout_ms); } while (r < 0 && errno == EINTR);
  ssize_t n = -1;
  if (r > 0) {
    do { n = ::recvmsg(s, &msg, MSG_CMSG_CLOEXEC); } while (n < 0 && errno == EINTR);
  }
  int fd = -1;
  if (n == static_cast<ssize_t>(sizeof(t)) && t.magic == kMagic) {
    for (struct cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
      if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
        memcpy(&fd, CMSG_DATA(c), sizeof(int));
        break;
      }
    }
  }
  ::close(s);
  if (fd < 0) fail(Result::SystemError, "malformed fd-passing message");
  if (src_rank) *src_rank = t.src;
  if (tag) *tag = t.tag;
  return fd;
}

}  // namespace mnccl
