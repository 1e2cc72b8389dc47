// The communicator: what the opaque ncclComm_t points at.  It owns the
// bootstrap store, the data plane (NVLink symmetric memory + kernels, or the
// network ring), the watchdog and the counters.  Plays the role of the
// reference's Context + transport pair (reference: include/mini_nccl.h:71-111,
// src/api.cpp:55-59) with two data planes instead of one.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "algo/select.h"
#include "core/config.h"
#include "core/dtype.h"
#include "core/error.h"
#include "kernels/comm_dev.h"
#include "kernels/launch.h"

namespace mnccl {

class BootstrapStore;
class FdChannel;
class SymmetricMemory;
struct Segment;
class Watchdog;
class OneSidedTransport;
class RingAllReduce;
namespace hera { class Worker; }

struct CommStats {
  uint64_t calls = 0, bytes = 0;
  uint64_t by_algo[12] = {0};
  uint64_t stale_registrations = 0;
  uint64_t zero_copy_in = 0, zero_copy_out = 0, staged_passes = 0, pipelined = 0;
  uint64_t graph_captures_seen = 0, errors = 0;
  uint64_t auto_exports = 0, auto_imports = 0;
};

class Comm {
 public:
  // rank == -1: Hera auto-bootstrap, `ip` names the master.  Throws Error.
  static Comm* create(int nranks, int rank, const char* ip);
  ~Comm();

  int rank() const { return rank_; }
  int size() const { return size_; }
  bool gpu_plane() const { return gpu_plane_; }

  void all_reduce(const void* send, DType send_t, void* recv, DType recv_t, DType wire_t, size_t count, RedOp op,
                  double scale, Algo forced, cudaStream_t stream);
  void reduce_scatter(const void* send, void* recv, size_t recvcount, DType t, RedOp op, cudaStream_t stream);
  void all_gather(const void* send, void* recv, size_t sendcount, DType t, cudaStream_t stream);

  void* mem_alloc(size_t bytes);
  void mem_free(void* ptr);
  void peer_pointers(void* ptr, void** peers, void** mc);
  // Collective: make an ordinary device buffer (cudaMalloc family) usable zero-copy by the
  // peer-to-peer kernels by exchanging CUDA IPC handles once; the opened mappings are cached.
  void register_buffer(void* ptr, size_t bytes);
  void deregister_buffer(void* ptr);
  void barrier();
  void abort();
  Result async_error();
  std::string stats_json();
  Algo query_algo(size_t bytes, DType t, RedOp op, bool registered);
  const CommDev& device_handle() const { return dev_; }
  bool set_knob(const char* name, long long value) {
    std::lock_guard<std::mutex> lk(call_mu_);
    return cfg_.set_knob(name ? name : "", value);
  }
  void set_tuning(int max_blocks, int unroll) {
    std::lock_guard<std::mutex> lk(call_mu_);
    cfg_.max_blocks = max_blocks;
    cfg_.unroll = unroll;
  }

 private:
  Comm() = default;
  void init(int nranks, int rank, const char* ip);
  void init_gpu_plane();
  void init_net_plane();
  void setup_shared_host_segment();
  void check_usable();
  void launch(Mode mode, const void* send, DType send_t, void* recv, DType recv_t, DType wire_t, size_t count,
              RedOp op, double scale, Algo forced, cudaStream_t stream);
  void launch_pipelined(const void* send, DType send_t, void* recv, DType recv_t, DType wire_t, size_t count, RedOp op,
                        double scale, Algo forced, cudaStream_t stream, bool host_in = false, bool host_out = false);
  void launch_solo_host(const void* send, DType send_t, void* recv, DType recv_t, size_t count, double factor,
                        cudaStream_t stream, bool host_in, bool host_out);
  void ensure_pipeline();
  void ring_all_reduce(const void* send, void* recv, size_t count, DType t, RedOp op, cudaStream_t stream);
  void init_shared_gpu_plane();
  void host_barrier();
  void shared_gpu_all_reduce(const void* send, void* recv, size_t count, DType t, RedOp op, double scale, cudaStream_t stream);
  // Segment containing [ptr, ptr+bytes) on this rank; offset returned.
  std::shared_ptr<Segment> find_segment(const void* ptr, size_t bytes, size_t* offset);
  void wait_blocking(cudaStream_t stream);

  int rank_ = 0, size_ = 1;
  int local_rank_ = 0, local_size_ = 1;
  int device_ = -1;
  bool has_gpu_ = false, gpu_plane_ = false;
  Config cfg_;
  std::string root_ip_, job_ns_;

  std::unique_ptr<hera::Worker> hera_;
  std::unique_ptr<BootstrapStore> store_;
  std::unique_ptr<FdChannel> fds_;
  std::unique_ptr<SymmetricMemory> symm_;
  std::shared_ptr<Segment> ctrl_;
  std::mutex seg_mu_;
  std::map<uintptr_t, std::shared_ptr<Segment>> user_segments_;  // keyed by local base address
  CommDev dev_{};
  CommCaps caps_{};

  // host-mapped words shared by the ranks of this host
  void* shm_map_ = nullptr;
  size_t shm_bytes_ = 0;
  bool shm_registered_ = false;
  void* private_host_ = nullptr;  // fallback when the shared mapping cannot be registered
  volatile uint32_t* abort_host_ = nullptr;
  volatile uint32_t* progress_host_ = nullptr;
  std::unique_ptr<Watchdog> watchdog_;

  // CUDA IPC mappings of peers' allocations, opened once per (peer, allocation): the handle
  // cache that plays the role of the reference's MR cache for device memory.
  struct IpcMapping {
    void* base = nullptr;
    int refs = 0;
  };
  std::map<std::string, IpcMapping> ipc_cache_;   // key: peer rank + handle bytes
  std::map<uintptr_t, std::vector<std::string>> registered_;  // local ptr -> cache keys it holds
  uint64_t ipc_hits_ = 0, ipc_misses_ = 0;

  // Lazy direct access to ordinary device buffers (kernels/comm_dev.h, AutoCtl): every rank lists the
  // allocations it has exported in the host's shared page; peers map them when they see them and note
  // the mapping in a table in device memory that the kernel reads.
  char* auto_shm_ = nullptr;                 // export tables in the shared page, one per rank (null: off)
  AutoMapEntry* auto_map_dev_ = nullptr;     // [kMaxRanks][kAutoSlots], device memory
  cudaStream_t auto_stream_ = nullptr;       // carries the table's updates
  std::vector<uint32_t> auto_seen_;          // per peer: entries of its export table already looked at
  std::vector<uint16_t> auto_mask_;          // per peer: its export slots that are mapped here
  std::vector<unsigned long long> auto_refused_;  // allocations of this rank that cannot be exported
  int auto_export(const void* ptr, size_t bytes, bool may_export);  // export slot of ptr's allocation (exported now if new), -1 if none
  void auto_import();                        // map what the peers have exported since the last look

  // chunk pipeline for large AllReduces on ordinary buffers
  struct Pipeline {
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t ev_start = nullptr, ev_in[2] = {nullptr, nullptr}, ev_comm[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
  };
  std::unique_ptr<Pipeline> pipe_;
  // single rank with pinned-host buffers: private device staging (two halves per direction)
  char* solo_stage_ = nullptr;
  size_t solo_stage_half_ = 0;

  // plane for ranks that share a GPU: host-synchronised, staging exchanged over CUDA IPC
  bool shared_plane_ = false;
  char* shared_stage_ = nullptr;        // this rank's staging (cudaMalloc)
  char* shared_out_ = nullptr;          // result staging for host-memory recv buffers
  size_t shared_stage_bytes_ = 0;
  std::vector<char*> shared_peer_stage_;  // every rank's staging as mapped here
  uint32_t shared_epoch_ = 0;

  // network plane
  std::unique_ptr<OneSidedTransport> transport_;
  std::unique_ptr<RingAllReduce> ring_;
  void* bounce_ = nullptr;
  size_t bounce_bytes_ = 0;

  std::atomic<bool> aborted_{false};
  std::atomic<bool> capture_warned_{false};
  std::mutex call_mu_;
  CommStats stats_;
};

}  // namespace mnccl
