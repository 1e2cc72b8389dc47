// Hera-Core control plane: framing, master and worker.
//
// Behaviour kept from the reference (reference: src/hera/hera_master.h:33-102,
// src/hera/hera_worker.h:21-52, src/hera/HeraSocket.h:86-108): the master
// listens (default port 9999), assigns ranks in arrival order, answers each
// registrant at once with {rank, world_size, root_ip = address of the first
// registrant as seen by the master}, keeps every connection open and then
// idles until stopped; the worker connects, registers with {hostname, pid} and
// exposes rank / size / root_ip.  Frames with a bad magic or version are
// rejected.
//
// Beyond the reference: payload length is bounded and checked against the
// message type, the response is zero-initialised, the worker retries its
// connect, every socket call has a deadline, and after registration the master
// serves HEARTBEAT (liveness bookkeeping, peer-loss detection), GLOBAL_ABORT
// (fan-out to every worker) and TOPOLOGY_INIT (ring neighbours) for workers
// that keep their connection (keep-alive agents).
#pragma once
#include <atomic>
#include <chrono>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "bootstrap/hera_wire.h"
#include "bootstrap/socket.h"

namespace mnccl {
namespace hera {

// Framing.  send_msg writes header+payload; recv_msg validates magic, version
// and length and returns false on orderly EOF before a header.
void send_msg(const TcpSocket& s, MsgType type, const void* payload, uint32_t len, int timeout_ms);
bool recv_msg(const TcpSocket& s, MsgType* type, std::vector<uint8_t>* payload, int timeout_ms);

struct WorkerRecord {
  int rank = -1;
  int pid = 0;
  std::string hostname;
  std::string ip;
  bool alive = true;
  uint32_t last_state = 0;
  std::chrono::steady_clock::time_point last_seen;
};

class Master {
 public:
  Master(int world_size, int port = kDefaultPort);
  ~Master();

  // Blocks: registration phase, then the service loop, until stop().
  void run();
  void stop();
  // Runs run() on an internal thread; returns once the port is bound.
  void start_background();

  int port() const { return bound_port_.load(); }
  bool all_registered() const { return registered_.load() >= world_size_; }
  std::vector<WorkerRecord> workers() const;
  bool abort_broadcast() const { return abort_sent_.load(); }
  // Heartbeat silence after which a keep-alive worker is declared lost and a
  // GLOBAL_ABORT is fanned out (0 disables).
  void set_heartbeat_timeout_ms(int ms) { hb_timeout_ms_ = ms; }
  void set_io_timeout_ms(int ms) { io_timeout_ms_ = ms; }

 private:
  void handle_register(TcpSocket client);
  void service_once();
  void fan_out_abort(int origin, uint32_t reason);

  int world_size_;
  int port_;
  std::atomic<int> bound_port_{0};
  std::atomic<bool> running_{true};
  std::atomic<int> registered_{0};
  std::atomic<bool> abort_sent_{false};
  int hb_timeout_ms_ = 0;
  int io_timeout_ms_ = 5000;
  TcpListener listener_;
  mutable std::mutex mu_;
  std::vector<WorkerRecord> records_;
  std::vector<TcpSocket> conns_;
  std::vector<bool> keepalive_;
  std::thread thread_;
};

class Worker {
 public:
  Worker(std::string master_ip, int port = kDefaultPort);
  ~Worker();

  // Connect (with retry), register, receive the assignment.
  void connect_and_register(int retries = 20, int retry_ms = 250, int timeout_ms = 30000);

  int rank() const { return rank_; }
  int size() const { return size_; }
  const std::string& root_ip() const { return root_ip_; }

  // Ask the master for this rank's ring neighbours (needs all_registered).
  TopologyInfo query_topology(int timeout_ms = 5000);

  // Keep-alive agent: sends HEARTBEAT every period_ms and calls on_abort when
  // a GLOBAL_ABORT arrives or the master vanishes.  stop_agent() joins.
  void start_agent(int period_ms, std::function<void(int origin, uint32_t reason)> on_abort);
  void stop_agent();
  // Ask the master to abort every worker (keeps working without an agent).
  void send_global_abort(uint32_t reason);
  void set_local_state(uint32_t s) { local_state_.store(s); }
  // Drop the connection (what the reference does right after registration).
  void disconnect();

 private:
  std::string master_ip_;
  int port_;
  int rank_ = -1, size_ = 0;
  std::string root_ip_;
  TcpSocket sock_;
  std::mutex send_mu_;
  std::atomic<bool> agent_run_{false};
  std::atomic<uint32_t> local_state_{0};
  std::thread agent_;
};

}  // namespace hera
}  // namespace mnccl
