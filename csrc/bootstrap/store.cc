#include "bootstrap/store.h"

#include <cstring>

#include "core/error.h"
#include "core/log.h"

namespace mnccl {
namespace {
constexpr uint32_t kHelloMagic = 0x4d4e4253;  // "MNBS"
struct Hello {
  uint32_t magic;
  int32_t rank;
  int32_t size;
};
struct OpHeader {
  uint32_t seq;
  uint32_t kind;  // 1 = gather, 2 = bcast
  uint64_t bytes;
};
}  // namespace

BootstrapStore::BootstrapStore(int rank, int size, std::string root_ip, int port, int timeout_ms,
                               int connect_retries)
    : rank_(rank), size_(size), root_ip_(std::move(root_ip)), port_(port),
      timeout_ms_(timeout_ms), retries_(connect_retries) {}

BootstrapStore::~BootstrapStore() = default;

void BootstrapStore::connect() {
  ips_.assign(size_, "127.0.0.1");
  if (size_ == 1) return;
  if (rank_ == 0) {
    listener_.listen_on(port_);
    peers_.resize(size_);
    int have = 0;
    while (have < size_ - 1) {
      TcpSocket s = listener_.accept_one(timeout_ms_);
      Hello h{};
      s.recv_all(&h, sizeof(h), timeout_ms_);
      if (h.magic != kHelloMagic || h.rank <= 0 || h.rank >= size_ || h.size != size_ ||
          peers_[h.rank].valid()) {
        MNCCL_WARN("Mini-NCCL", "bootstrap: rejected a malformed or duplicate hello (rank %d)", h.rank);
        continue;
      }
      ips_[h.rank] = s.peer_ip();
      peers_[h.rank] = std::move(s);
      ++have;
    }
    listener_.close();  // the port is free for the next communicator
  } else {
    peers_.resize(1);
    peers_[0] = TcpSocket::connect_to(root_ip_, port_, retries_, 1000);
    Hello h{kHelloMagic, rank_, size_};
    peers_[0].send_all(&h, sizeof(h), timeout_ms_);
  }
  // Everyone learns everyone's address (as seen by the root).
  std::vector<char> packed(size_ * 64, 0);
  if (rank_ == 0) {
    ips_[0] = root_ip_;
    for (int r = 0; r < size_; ++r) strncpy(&packed[r * 64], ips_[r].c_str(), 63);
  }
  broadcast(packed.data(), packed.size(), 0);
  for (int r = 0; r < size_; ++r) ips_[r] = std::string(&packed[r * 64]);
}

void BootstrapStore::all_gather(const void* in, void* out, size_t bytes) {
  std::lock_guard<std::mutex> lk(mu_);
  char* o = static_cast<char*>(out);
  if (size_ == 1) {
    if (bytes) memcpy(o, in, bytes);
    return;
  }
  uint32_t seq = ++op_seq_;
  if (rank_ == 0) {
    if (bytes) memcpy(o, in, bytes);
    for (int r = 1; r < size_; ++r) {
      OpHeader h{};
      peers_[r].recv_all(&h, sizeof(h), timeout_ms_);
      if (h.seq != seq || h.kind != 1 || h.bytes != bytes)
        fail(Result::InternalError, "bootstrap all_gather out of step with rank " + std::to_string(r));
      peers_[r].recv_all(o + size_t(r) * bytes, bytes, timeout_ms_);
    }
    for (int r = 1; r < size_; ++r) peers_[r].send_all(o, size_t(size_) * bytes, timeout_ms_);
  } else {
    OpHeader h{seq, 1, bytes};
    peers_[0].send_all(&h, sizeof(h), timeout_ms_);
    peers_[0].send_all(in, bytes, timeout_ms_);
    peers_[0].recv_all(o, size_t(size_) * bytes, timeout_ms_);
  }
}

void BootstrapStore::broadcast(void* buf, size_t bytes, int root) {
  if (size_ == 1) return;
  if (root != 0) {
    // Route through the star: gather then pick.
    std::vector<char> all(size_t(size_) * bytes);
    all_gather(buf, all.data(), bytes);
    memcpy(buf, all.data() + size_t(root) * bytes, bytes);
    return;
  }
  std::lock_guard<std::mutex> lk(mu_);
  uint32_t seq = ++op_seq_;
  if (rank_ == 0) {
    OpHeader h{seq, 2, bytes};
    for (int r = 1; r < size_; ++r) {
      peers_[r].send_all(&h, sizeof(h), timeout_ms_);
      peers_[r].send_all(buf, bytes, timeout_ms_);
    }
  } else {
    OpHeader h{};
    peers_[0].recv_all(&h, sizeof(h), timeout_ms_);
    if (h.seq != seq || h.kind != 2 || h.bytes != bytes)
      fail(Result::InternalError, "bootstrap broadcast out of step");
    peers_[0].recv_all(buf, bytes, timeout_ms_);
  }
}

void BootstrapStore::barrier() {
  uint32_t x = 0;
  std::vector<uint32_t> all(size_);
  all_gather(&x, all.data(), sizeof(x));
}

}  // namespace mnccl
