#include "bootstrap/hera.h"

#include <cstring>
#include <poll.h>
#include <unistd.h>

#include "core/error.h"
#include "core/log.h"

namespace mnccl {
namespace hera {
namespace {

uint32_t expected_len(MsgType t, bool* known) {
  *known = true;
  switch (t) {
    case MsgType::RegisterReq: return sizeof(RegisterReq);
    case MsgType::RegisterResp: return sizeof(RegisterResp);
    case MsgType::TopologyInit: return 0;  // request: empty or TopologyInfo
    case MsgType::TopologyAck: return sizeof(TopologyInfo);
    case MsgType::Heartbeat: return sizeof(Heartbeat);
    case MsgType::GlobalAbort: return sizeof(GlobalAbort);
  }
  *known = false;
  return 0;
}

uint32_t now_seconds() {
  using namespace std::chrono;
  return static_cast<uint32_t>(duration_cast<seconds>(steady_clock::now().time_since_epoch()).count());
}

}  // namespace

void send_msg(const TcpSocket& s, MsgType type, const void* payload, uint32_t len, int timeout_ms) {
  if (len > kMaxPayload) fail(Result::InvalidArgument, "Hera payload too large");
  // One buffer, one send: a frame is never interleaved with another sender's.
  std::vector<uint8_t> frame(sizeof(Header) + len);
  Header h;
  h.magic = kMagic;
  h.msg_type = static_cast<uint8_t>(type);
  h.version = kVersion;
  h.reserved = 0;
  h.payload_len = len;
  memcpy(frame.data(), &h, sizeof(h));
  if (len) memcpy(frame.data() + sizeof(h), payload, len);
  s.send_all(frame.data(), frame.size(), timeout_ms);
}

bool recv_msg(const TcpSocket& s, MsgType* type, std::vector<uint8_t>* payload, int timeout_ms) {
  Header h;
  if (!s.recv_all_or_eof(&h, sizeof(h), timeout_ms)) return false;
  if (h.magic != kMagic) fail(Result::InvalidArgument, "Hera: invalid magic number");
  if (h.version != kVersion) fail(Result::InvalidArgument, "Hera: protocol version mismatch");
  if (h.payload_len > kMaxPayload) fail(Result::InvalidArgument, "Hera: payload length out of bounds");
  MsgType t = static_cast<MsgType>(h.msg_type);
  bool known = false;
  uint32_t want = expected_len(t, &known);
  if (!known) fail(Result::InvalidArgument, "Hera: unknown message type");
  if (t == MsgType::TopologyInit) {
    if (h.payload_len != 0 && h.payload_len != sizeof(TopologyInfo))
      fail(Result::InvalidArgument, "Hera: bad TOPOLOGY_INIT length");
  } else if (h.payload_len != want) {
    fail(Result::InvalidArgument, "Hera: payload length does not match message type");
  }
  payload->resize(h.payload_len);
  if (h.payload_len) s.recv_all(payload->data(), h.payload_len, timeout_ms);
  *type = t;
  return true;
}

// ------------------------------------------------------------------ master

Master::Master(int world_size, int port) : world_size_(world_size), port_(port) {
  if (world_size <= 0) fail(Result::InvalidArgument, "Hera master: world size must be positive");
}

Master::~Master() {
  stop();
  if (thread_.joinable()) thread_.join();
}

void Master::stop() { running_.store(false); }

void Master::start_background() {
  listener_.listen_on(port_);
  bound_port_.store(listener_.port());
  thread_ = std::thread([this] { run(); });
}

std::vector<WorkerRecord> Master::workers() const {
  std::lock_guard<std::mutex> lk(mu_);
  return records_;
}

void Master::run() {
  try {
    if (!listener_.valid()) {
      listener_.listen_on(port_);
      bound_port_.store(listener_.port());
    }
    log_always("Hera-Master", "Listening on port %d, waiting for %d workers...", listener_.port(), world_size_);
    while (running_.load() && registered_.load() < world_size_) {
      TcpSocket c = listener_.try_accept(100);
      if (c.valid()) handle_register(std::move(c));
      service_once();
    }
    if (registered_.load() >= world_size_) {
      log_always("Hera-Master", "All %d workers registered! Cluster is Ready.", world_size_);
      std::string root;
      {
        std::lock_guard<std::mutex> lk(mu_);
        root = records_.empty() ? "" : records_[0].ip;
      }
      log_always("Hera-Master", "Root IP (Rank 0) is: %s", root.c_str());
    }
    while (running_.load()) {
      service_once();
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
  } catch (const std::exception& e) {
    log_always("Hera-Master", "Fatal Error: %s", e.what());
  }
  listener_.close();
}

void Master::handle_register(TcpSocket client) {
  MsgType type;
  std::vector<uint8_t> buf;
  std::string peer_ip = client.peer_ip();
  try {
    if (!recv_msg(client, &type, &buf, io_timeout_ms_)) {
      log_always("Hera-Master", "Client disconnected during registration");
      return;
    }
  } catch (const std::exception& e) {
    log_always("Hera-Master", "Rejected a client: %s", e.what());
    return;
  }
  if (type != MsgType::RegisterReq) {
    log_always("Hera-Master", "Unexpected msg type");
    return;
  }
  RegisterReq req;
  memcpy(&req, buf.data(), sizeof(req));
  req.hostname[sizeof(req.hostname) - 1] = '\0';

  RegisterResp resp;
  memset(&resp, 0, sizeof(resp));
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (static_cast<int>(records_.size()) >= world_size_) return;  // world is full
    WorkerRecord w;
    w.rank = static_cast<int>(records_.size());
    w.pid = req.pid;
    w.hostname = req.hostname;
    w.ip = peer_ip;
    w.last_seen = std::chrono::steady_clock::now();
    records_.push_back(w);
    resp.rank = w.rank;
    resp.world_size = world_size_;
    strncpy(resp.root_ip, records_[0].ip.c_str(), sizeof(resp.root_ip) - 1);
    log_always("Hera-Master", "New Worker: Rank=%d Host=%s IP=%s PID=%d", w.rank, w.hostname.c_str(),
               w.ip.c_str(), w.pid);
  }
  try {
    send_msg(client, MsgType::RegisterResp, &resp, sizeof(resp), io_timeout_ms_);
  } catch (const std::exception& e) {
    log_always("Hera-Master", "Could not answer rank %d: %s", resp.rank, e.what());
  }
  std::lock_guard<std::mutex> lk(mu_);
  conns_.push_back(std::move(client));
  keepalive_.push_back(false);
  registered_.fetch_add(1);
}

void Master::fan_out_abort(int origin, uint32_t reason) {
  // mu_ is held by the caller.
  if (abort_sent_.exchange(true)) return;
  GlobalAbort ga{origin, reason};
  log_always("Hera-Master", "GLOBAL_ABORT from rank %d (reason %u): notifying %zu workers", origin, reason,
             conns_.size());
  for (size_t i = 0; i < conns_.size(); ++i) {
    if (!conns_[i].valid()) continue;
    try {
      send_msg(conns_[i], MsgType::GlobalAbort, &ga, sizeof(ga), 1000);
    } catch (const std::exception&) {
      conns_[i].close();
      records_[i].alive = false;
    }
  }
}

void Master::service_once() {
  std::lock_guard<std::mutex> lk(mu_);
  auto now = std::chrono::steady_clock::now();
  for (size_t i = 0; i < conns_.size(); ++i) {
    if (!conns_[i].valid()) continue;
    while (conns_[i].valid() && conns_[i].readable(0)) {
      MsgType type;
      std::vector<uint8_t> buf;
      bool got = false;
      try {
        got = recv_msg(conns_[i], &type, &buf, io_timeout_ms_);
      } catch (const std::exception& e) {
        MNCCL_INFO("Hera-Master", "rank %zu: dropping connection: %s", i, e.what());
        got = false;
      }
      if (!got) {
        // The reference's workers close right after registration; that is
        // normal.  Losing a keep-alive agent is a failure.
        conns_[i].close();
        if (keepalive_[i]) {
          records_[i].alive = false;
          log_always("Hera-Master", "Lost keep-alive worker rank %zu", i);
          fan_out_abort(static_cast<int>(i), 2);
        }
        break;
      }
      records_[i].last_seen = now;
      if (type == MsgType::Heartbeat) {
        Heartbeat hb;
        memcpy(&hb, buf.data(), sizeof(hb));
        keepalive_[i] = true;
        records_[i].last_state = hb.state;
        if (hb.state != 0) fan_out_abort(static_cast<int>(i), 1);
      } else if (type == MsgType::GlobalAbort) {
        GlobalAbort ga;
        memcpy(&ga, buf.data(), sizeof(ga));
        fan_out_abort(static_cast<int>(i), ga.reason);
      } else if (type == MsgType::TopologyInit) {
        TopologyInfo ti;
        memset(&ti, 0, sizeof(ti));
        int n = static_cast<int>(records_.size());
        int r = static_cast<int>(i);
        ti.prev_rank = (r - 1 + n) % n;
        ti.next_rank = (r + 1) % n;
        strncpy(ti.next_ip, records_[ti.next_rank].ip.c_str(), sizeof(ti.next_ip) - 1);
        ti.next_port = 0;
        try {
          send_msg(conns_[i], MsgType::TopologyAck, &ti, sizeof(ti), io_timeout_ms_);
        } catch (const std::exception&) {
          conns_[i].close();
        }
      }
    }
    if (conns_[i].valid() && keepalive_[i] && hb_timeout_ms_ > 0 && records_[i].alive) {
      auto silent = std::chrono::duration_cast<std::chrono::milliseconds>(now - records_[i].last_seen).count();
      if (silent > hb_timeout_ms_) {
        records_[i].alive = false;
        log_always("Hera-Master", "Heartbeat from rank %zu silent for %lld ms", i, static_cast<long long>(silent));
        fan_out_abort(static_cast<int>(i), 3);
      }
    }
  }
}

// ------------------------------------------------------------------ worker

Worker::Worker(std::string master_ip, int port) : master_ip_(std::move(master_ip)), port_(port) {}

Worker::~Worker() {
  stop_agent();
  disconnect();
}

void Worker::disconnect() { sock_.close(); }

void Worker::connect_and_register(int retries, int retry_ms, int timeout_ms) {
  sock_ = TcpSocket::connect_to(master_ip_, port_, retries, retry_ms);
  RegisterReq req;
  memset(&req, 0, sizeof(req));
  if (::gethostname(req.hostname, sizeof(req.hostname) - 1) != 0) strncpy(req.hostname, "unknown", 63);
  req.pid = static_cast<int32_t>(::getpid());
  log_always("Hera-Worker", "Registering with Master...");
  send_msg(sock_, MsgType::RegisterReq, &req, sizeof(req), timeout_ms);
  MsgType type;
  std::vector<uint8_t> buf;
  if (!recv_msg(sock_, &type, &buf, timeout_ms)) fail(Result::RemoteError, "Hera master closed the connection");
  if (type != MsgType::RegisterResp) fail(Result::InternalError, "Hera: unexpected response type");
  RegisterResp resp;
  memcpy(&resp, buf.data(), sizeof(resp));
  resp.root_ip[sizeof(resp.root_ip) - 1] = '\0';
  rank_ = resp.rank;
  size_ = resp.world_size;
  root_ip_ = resp.root_ip;
  log_always("Hera-Worker", "Registered! Rank=%d World=%d Root=%s", rank_, size_, root_ip_.c_str());
}

TopologyInfo Worker::query_topology(int timeout_ms) {
  if (agent_run_.load()) fail(Result::InvalidUsage, "query_topology must precede start_agent");
  {
    std::lock_guard<std::mutex> lk(send_mu_);
    send_msg(sock_, MsgType::TopologyInit, nullptr, 0, timeout_ms);
  }
  MsgType type;
  std::vector<uint8_t> buf;
  if (!recv_msg(sock_, &type, &buf, timeout_ms)) fail(Result::RemoteError, "Hera master closed the connection");
  if (type != MsgType::TopologyAck) fail(Result::InternalError, "Hera: expected TOPOLOGY_ACK");
  TopologyInfo ti;
  memcpy(&ti, buf.data(), sizeof(ti));
  ti.next_ip[sizeof(ti.next_ip) - 1] = '\0';
  return ti;
}

void Worker::send_global_abort(uint32_t reason) {
  GlobalAbort ga{rank_, reason};
  std::lock_guard<std::mutex> lk(send_mu_);
  if (sock_.valid()) send_msg(sock_, MsgType::GlobalAbort, &ga, sizeof(ga), 2000);
}

void Worker::start_agent(int period_ms, std::function<void(int, uint32_t)> on_abort) {
  if (agent_run_.exchange(true)) return;
  agent_ = std::thread([this, period_ms, on_abort] {
    auto next_beat = std::chrono::steady_clock::now();
    while (agent_run_.load()) {
      try {
        auto now = std::chrono::steady_clock::now();
        if (now >= next_beat) {
          Heartbeat hb{rank_, local_state_.load(), now_seconds()};
          std::lock_guard<std::mutex> lk(send_mu_);
          send_msg(sock_, MsgType::Heartbeat, &hb, sizeof(hb), 2000);
          next_beat = now + std::chrono::milliseconds(period_ms);
        }
        if (sock_.readable(10)) {
          MsgType type;
          std::vector<uint8_t> buf;
          if (!recv_msg(sock_, &type, &buf, 2000)) {
            if (agent_run_.load() && on_abort) on_abort(-1, 4);  // master vanished
            break;
          }
          if (type == MsgType::GlobalAbort) {
            GlobalAbort ga;
            memcpy(&ga, buf.data(), sizeof(ga));
            if (on_abort) on_abort(ga.origin_rank, ga.reason);
            break;
          }
        }
      } catch (const std::exception& e) {
        if (agent_run_.load()) {
          MNCCL_WARN("Hera-Worker", "agent stopped: %s", e.what());
          if (on_abort) on_abort(-1, 4);
        }
        break;
      }
    }
  });
}

void Worker::stop_agent() {
  agent_run_.store(false);
  if (agent_.joinable()) agent_.join();
}

}  // namespace hera
}  // namespace mnccl
