#include "comm.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <functional>
#include <random>
#include <sstream>
#include <thread>

#include "bootstrap/fdpass.h"
#include "bootstrap/hera.h"
#include "bootstrap/store.h"
#include "core/log.h"
#include "core/nvtx.h"
#include "mem/cuda_driver.h"
#include "mem/symmetric.h"
#include "net/ring.h"
#include "net/transport.h"
#include "watchdog/watchdog.h"

namespace mnccl {
namespace {

#define RT_CHECK(call, what)                                                                   \
  do {                                                                                         \
    cudaError_t _e = (call);                                                                   \
    if (_e != cudaSuccess) {                                                                   \
      (void)cudaGetLastError();                                                                \
      fail(Result::UnhandledCudaError, std::string(what) + ": " + cudaGetErrorString(_e));     \
    }                                                                                          \
  } while (0)

struct PeerInfo {
  uint64_t host_hash;
  int32_t has_gpu;
  int32_t device;
  int32_t device_count;
  int32_t pid;
  int32_t may_pick_device;  // this rank lets the library pick its GPU (Hera mode, automatic choice on, no device forced)
  char bus_id[32];
};

uint64_t host_hash() {
  char name[256] = {0};
  if (gethostname(name, sizeof(name) - 1) != 0) strcpy(name, "unknown");
  // Containers on one machine may share a hostname but not /dev/shm or the
  // abstract socket namespace; mix in the boot id and the network namespace.
  std::string key = name;
  char buf[128];
  ssize_t n = readlink("/proc/self/ns/net", buf, sizeof(buf) - 1);
  if (n > 0) key.append(buf, static_cast<size_t>(n));
  return std::hash<std::string>{}(key);
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// One export table per rank behind the first 4 KB of the shared page (lazy direct access).
struct AutoExport {
  uint64_t id, base, size;
  cudaIpcMemHandle_t handle;
};
struct AutoExportTable {
  uint32_t count;   // entries published so far (only grows; written after the entry)
  uint32_t pad;
  AutoExport e[kAutoSlots];
};
constexpr size_t kAutoShmOffset = 4096;
constexpr int kAutoShmRanks = 8;
constexpr size_t kShmBytes = 4096 + ((kAutoShmRanks * sizeof(AutoExportTable) + 4095) / 4096) * 4096;
constexpr int kProgressWords = 16;  // per local rank, 64 bytes

enum class MemKind { Device, PinnedHost, PlainHost };

// The driver's id of the allocation `p` lies in (unique per allocation for the life of the process);
// 0 when it cannot be told.
unsigned long long allocation_id(const void* p) {
  const CudaDriver* d = CudaDriver::get();
  unsigned long long id = 0;
  if (!d || !d->PointerGetAttribute ||
      d->PointerGetAttribute(&id, CU_POINTER_ATTRIBUTE_BUFFER_ID, reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS)
    return 0;
  return id;
}

MemKind classify(const void* p, bool has_gpu) {
  if (!has_gpu) return MemKind::PlainHost;
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return MemKind::PlainHost;
  }
  switch (a.type) {
    case cudaMemoryTypeDevice: return MemKind::Device;
    case cudaMemoryTypeManaged: return MemKind::Device;
    case cudaMemoryTypeHost: return MemKind::PinnedHost;
    default: return MemKind::PlainHost;
  }
}

}  // namespace

Comm* Comm::create(int nranks, int rank, const char* ip) {
  std::unique_ptr<Comm> c(new Comm());
  c->init(nranks, rank, ip);
  return c.release();
}

void Comm::init(int nranks, int rank, const char* ip) {
  cfg_ = Config::get();
  root_ip_ = ip ? ip : "127.0.0.1";
  rank_ = rank;
  size_ = nranks;
  bool hera_mode = false;
  if (rank == -1) {
    // Hera auto-bootstrap: `ip` is the master; rank, world size and the root
    // address come back from it (reference: src/api.cpp:38-51).
    hera_mode = true;
    log_always("Mini-NCCL", "Hera Mode Activated. Connecting to Master at %s...", root_ip_.c_str());
    hera_.reset(new hera::Worker(root_ip_, cfg_.hera_port));
    hera_->connect_and_register(cfg_.connect_retries, 250, cfg_.socket_timeout_ms);
    rank_ = hera_->rank();
    size_ = hera_->size();
    root_ip_ = hera_->root_ip();
    log_always("Mini-NCCL", "Auto-Assigned Rank: %d Size: %d Root-IP: %s", rank_, size_, root_ip_.c_str());
    if (!cfg_.hera_keepalive) hera_->disconnect();  // the reference's worker lives for the registration only
  }
  if (size_ <= 0 || rank_ < 0 || rank_ >= size_) fail(Result::InvalidArgument, "rank out of range");
  if (size_ > kMaxRanks && cfg_.transport != "soft" && cfg_.transport != "verbs")
    MNCCL_INFO("Mini-NCCL", "more than %d ranks: the NVLink plane is not used", kMaxRanks);

  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess) {
    (void)cudaGetLastError();
    ndev = 0;
  }
  has_gpu_ = ndev > 0;
  if (has_gpu_) {
    if (cfg_.cuda_device >= 0) RT_CHECK(cudaSetDevice(cfg_.cuda_device), "cudaSetDevice");
    RT_CHECK(cudaGetDevice(&device_), "cudaGetDevice");
  }

  store_.reset(new BootstrapStore(rank_, size_, root_ip_, cfg_.bootstrap_port, cfg_.socket_timeout_ms,
                                  cfg_.connect_retries));
  store_->connect();

  // Measured crossovers for this machine, if a table was given (the built-in ones are the fallback).
  if (!cfg_.tuning_file.empty()) {
    std::string errors;
    const int applied = cfg_.apply_tuning_file(cfg_.tuning_file, size_, &errors);
    if (!errors.empty()) MNCCL_WARN("Mini-NCCL", "tuning file %s: %s", cfg_.tuning_file.c_str(), errors.c_str());
    MNCCL_INFO("Mini-NCCL", "rank %d: %d knob(s) from %s", rank_, applied, cfg_.tuning_file.c_str());
  }

  // Job namespace for host shared memory and unix sockets: a nonce from rank 0.
  uint64_t nonce = 0;
  if (rank_ == 0) {
    std::random_device rd;
    nonce = (static_cast<uint64_t>(rd()) << 32) ^ rd() ^ static_cast<uint64_t>(getpid());
  }
  store_->broadcast(&nonce, sizeof(nonce), 0);
  {
    char buf[64];
    snprintf(buf, sizeof(buf), "%016llx", static_cast<unsigned long long>(nonce));
    job_ns_ = cfg_.job_id.empty() ? std::string(buf) : cfg_.job_id + "-" + buf;
  }

  // Who is where.
  PeerInfo me{};
  me.host_hash = host_hash();
  me.has_gpu = has_gpu_ ? 1 : 0;
  me.device = device_;
  me.device_count = ndev;
  me.pid = static_cast<int32_t>(getpid());
  me.may_pick_device = (hera_mode && cfg_.auto_device && has_gpu_ && cfg_.cuda_device < 0) ? 1 : 0;
  if (has_gpu_) cudaDeviceGetPCIBusId(me.bus_id, sizeof(me.bus_id), device_);
  std::vector<PeerInfo> all(size_);
  store_->all_gather(&me, all.data(), sizeof(me));
  local_rank_ = 0;
  local_size_ = 0;
  bool one_host = true, all_gpu = true;
  for (int r = 0; r < size_; ++r) {
    if (all[r].host_hash == me.host_hash) {
      if (r < rank_) ++local_rank_;
      ++local_size_;
    } else {
      one_host = false;
    }
    if (!all[r].has_gpu) all_gpu = false;
  }

  // Hera mode: ranks that were all started on the same device (the reference
  // benchmark pins every rank to GPU 0, reference: tests/perf_test.cpp:46)
  // spread over the host's GPUs by local rank.
  // Whether this second exchange happens is decided from the GATHERED data only, so that every rank
  // takes the same branch even when their environments differ (one rank with MINI_NCCL_CUDA_DEVICE set
  // would otherwise skip an all_gather the others wait in).
  bool all_may_pick = true;
  for (int r = 0; r < size_; ++r) all_may_pick = all_may_pick && all[r].may_pick_device != 0;
  if (all_may_pick && one_host && all_gpu && size_ > 1) {
    bool shared = true;
    for (int r = 0; r < size_; ++r) shared = shared && all[r].device == all[0].device;
    if (shared && ndev >= local_size_) {
      RT_CHECK(cudaSetDevice(local_rank_), "cudaSetDevice(local rank)");
      device_ = local_rank_;
      log_always("Mini-NCCL", "Rank %d: selected GPU %d from the local rank", rank_, device_);
      me.device = device_;
      cudaDeviceGetPCIBusId(me.bus_id, sizeof(me.bus_id), device_);
      // fallthrough to the gather below
    }
    store_->all_gather(&me, all.data(), sizeof(me));
  }

  bool distinct = true;
  for (int a = 0; a < size_ && distinct; ++a)
    for (int b = a + 1; b < size_; ++b)
      if (all[a].host_hash == all[b].host_hash && strncmp(all[a].bus_id, all[b].bus_id, sizeof(me.bus_id)) == 0) {
        distinct = false;
        break;
      }
  bool p2p_ok = has_gpu_;
  if (has_gpu_ && one_host && all_gpu && distinct) {
    for (int r = 0; r < size_ && p2p_ok; ++r) {
      if (r == rank_) continue;
      int peer_dev = -1, can = 0;
      if (cudaDeviceGetByPCIBusId(&peer_dev, all[r].bus_id) != cudaSuccess) {
        (void)cudaGetLastError();
        continue;  // not visible in this process: the mapping step decides
      }
      if (cudaDeviceCanAccessPeer(&can, device_, peer_dev) != cudaSuccess || !can) {
        (void)cudaGetLastError();
        p2p_ok = false;
      }
    }
  }
  bool want_gpu_plane = size_ == 1 ? has_gpu_ : (one_host && all_gpu && distinct && p2p_ok && size_ <= kMaxRanks);
  // Ranks that share a GPU (the reference's benchmark pins every rank to GPU 0, reference:
  // tests/perf_test.cpp:46): kernels of different processes on one GPU cannot wait for one another, so
  // the NVLink plane is out; a host-synchronised plane over CUDA IPC staging takes its place.
  bool want_shared = size_ > 1 && has_gpu_ && one_host && all_gpu && !distinct && size_ <= kMaxRanks;
  if (cfg_.transport == "soft" || cfg_.transport == "verbs") want_gpu_plane = want_shared = false;
  // Every rank must take the same plane.
  uint8_t mine = want_gpu_plane ? 1 : (want_shared ? 2 : 0);
  std::vector<uint8_t> votes(size_);
  store_->all_gather(&mine, votes.data(), 1);
  gpu_plane_ = true;
  shared_plane_ = true;
  for (uint8_t v : votes) {
    gpu_plane_ = gpu_plane_ && v == 1;
    shared_plane_ = shared_plane_ && v == 2;
  }
  if (cfg_.transport == "nvlink" && !gpu_plane_)
    fail(Result::SystemError, "MINI_NCCL_TRANSPORT=nvlink but the ranks do not share one NVLink-connected host");

  setup_shared_host_segment();
  if (gpu_plane_) init_gpu_plane();
  else if (shared_plane_) init_shared_gpu_plane();
  else init_net_plane();

  if (hera_ && cfg_.hera_keepalive) {
    hera_->start_agent(200, [this](int origin, uint32_t reason) {
      log_always("Mini-NCCL", "rank %d: GLOBAL_ABORT received (origin %d, reason %u)", rank_, origin, reason);
      abort();
    });
  }
  store_->barrier();
  MNCCL_INFO("Mini-NCCL", "rank %d/%d ready: plane=%s device=%d local_rank=%d", rank_, size_,
             gpu_plane_ ? "nvlink" : (shared_plane_ ? "shared-gpu" : (transport_ ? transport_->name() : "none")), device_, local_rank_);
}

void Comm::setup_shared_host_segment() {
  // One page per host: word 0 is the abort word, each local rank owns 16 words
  // of progress.  Created by the host's first rank, unlinked once all mapped it.
  std::string name = "/mnccl-" + job_ns_ + "-" + std::to_string(static_cast<unsigned long long>(host_hash() & 0xffffffffull));
  int fd = -1;
  if (local_rank_ == 0) {
    fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd >= 0 && ftruncate(fd, kShmBytes) != 0) {
      close(fd);
      fd = -1;
    }
  }
  store_->barrier();
  if (local_rank_ != 0) fd = shm_open(name.c_str(), O_RDWR, 0600);
  if (fd >= 0) {
    void* m = mmap(nullptr, kShmBytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (m != MAP_FAILED) {
      shm_map_ = m;
      shm_bytes_ = kShmBytes;
    }
  }
  store_->barrier();
  if (local_rank_ == 0) shm_unlink(name.c_str());
  uint32_t* words = nullptr;
  if (shm_map_ && (1 + local_rank_ + 1) * kProgressWords * 4 <= static_cast<int>(kShmBytes)) {
    words = static_cast<uint32_t*>(shm_map_);
    if (has_gpu_) {
      if (cudaHostRegister(shm_map_, kShmBytes, cudaHostRegisterMapped | cudaHostRegisterPortable) == cudaSuccess) {
        shm_registered_ = true;
      } else {
        (void)cudaGetLastError();
        words = nullptr;
        MNCCL_WARN("Mini-NCCL", "rank %d: cannot map the shared abort page into the GPU; abort stays local to this rank", rank_);
      }
    }
  }
  if (!words) {
    if (has_gpu_) {
      RT_CHECK(cudaHostAlloc(&private_host_, kShmBytes, cudaHostAllocMapped), "cudaHostAlloc(abort page)");
    } else {
      private_host_ = calloc(1, kShmBytes);
      if (!private_host_) fail(Result::SystemError, "out of memory");
    }
    memset(private_host_, 0, kShmBytes);
    words = static_cast<uint32_t*>(private_host_);
    abort_host_ = words;
    progress_host_ = words + kProgressWords;
  } else {
    abort_host_ = words;
    progress_host_ = words + kProgressWords * (1 + local_rank_);
    for (int i = 0; i < kProgressWords; ++i) progress_host_[i] = 0;
  }
}

void Comm::init_gpu_plane() {
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_);
  caps_.nranks = size_;
  caps_.sm_count = sms;
  memset(&dev_, 0, sizeof(dev_));
  dev_.rank = rank_;
  dev_.nranks = size_;
  dev_.spin_timeout_ns = static_cast<uint64_t>(cfg_.watchdog_timeout_ms) * 1500000ull;  // 1.5x the host bound
  uint32_t* dptr = nullptr;
  void* host_base = private_host_ ? private_host_ : shm_map_;
  if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&dptr), host_base, 0) == cudaSuccess && dptr) {
    const size_t prog_off = reinterpret_cast<const char*>(const_cast<const uint32_t*>(progress_host_)) - static_cast<const char*>(host_base);
    dev_.abort_word = dptr;
    dev_.host_progress = cfg_.watchdog_enable ? reinterpret_cast<volatile uint32_t*>(reinterpret_cast<char*>(dptr) + prog_off) : nullptr;
  } else {
    (void)cudaGetLastError();
    dev_.abort_word = nullptr;
    dev_.host_progress = nullptr;
  }
  if (size_ == 1) return;  // a single rank needs no symmetric memory

  fds_.reset(new FdChannel(job_ns_, rank_));
  fds_->open();
  store_->barrier();
  symm_.reset(new SymmetricMemory(rank_, size_, device_, store_.get(), fds_.get(), cfg_));

  // Control segment layout.
  caps_.ll_slot_bytes = align_up(default_ll_slot_bytes(size_, cfg_), 4096);
  caps_.inbox_slot_bytes = align_up(default_inbox_slot_bytes(size_, cfg_), 4096);
  caps_.stage_bytes = align_up(cfg_.staging_bytes, 4096);
  size_t off = 0;
  dev_.off_sig = off;
  off += align_up(sizeof(uint32_t) * kMaxBlocks * kMaxRanks, 4096);
  dev_.off_local = off;
  off += align_up(sizeof(LocalState), 4096);
  dev_.off_pipe = off;
  off += align_up(sizeof(PipeCtl), 4096);
  dev_.off_auto = off;
  off += align_up(sizeof(AutoCtl), 4096);
  dev_.off_ll = off;
  off += 2 * size_t(size_) * caps_.ll_slot_bytes;
  dev_.off_inbox = off;
  off += 2 * size_t(size_) * caps_.inbox_slot_bytes;
  off = align_up(off, 1 << 16);
  dev_.off_stage_a = off;
  off += caps_.stage_bytes;
  dev_.off_stage_b = off;
  off += caps_.stage_bytes;
  dev_.ll_slot_bytes = caps_.ll_slot_bytes;
  dev_.inbox_slot_bytes = caps_.inbox_slot_bytes;
  dev_.stage_bytes = caps_.stage_bytes;

  ctrl_ = symm_->allocate(off, true);
  for (int r = 0; r < size_; ++r) dev_.ctrl[r] = static_cast<char*>(ctrl_->peer[r]);
  dev_.ctrl_mc = static_cast<char*>(ctrl_->mc);
  caps_.nvls = ctrl_->mc != nullptr;

  // lazy direct access: needs the page shared by the host's ranks and a table the kernels can read.
  // The table lives in DEVICE memory: reads of host-mapped memory from many blocks at once take
  // about a microsecond each, one after the other (measured: 96 blocks x 8 reads = 750 us per call).
  if (cfg_.auto_map && shm_map_ && shm_registered_ && size_ <= kAutoShmRanks && local_size_ == size_) {
    void* tab = nullptr;
    const size_t tab_bytes = sizeof(AutoMapEntry) * kMaxRanks * kAutoSlots;
    if (cudaMalloc(&tab, tab_bytes) == cudaSuccess && cudaMemset(tab, 0, tab_bytes) == cudaSuccess &&
        cudaStreamCreateWithFlags(&auto_stream_, cudaStreamNonBlocking) == cudaSuccess) {
      auto_map_dev_ = static_cast<AutoMapEntry*>(tab);
      dev_.auto_map = auto_map_dev_;
      auto_shm_ = static_cast<char*>(shm_map_) + kAutoShmOffset;
      memset(auto_shm_ + rank_ * sizeof(AutoExportTable), 0, sizeof(AutoExportTable));
      auto_seen_.assign(size_, 0);
      auto_mask_.assign(size_, 0);
    } else {
      (void)cudaGetLastError();
      if (tab) cudaFree(tab);
    }
  }

  if (cfg_.watchdog_enable && dev_.host_progress) {
    watchdog_.reset(new Watchdog(progress_host_, abort_host_, cfg_.watchdog_timeout_ms, rank_));
    watchdog_->set_on_trip([this](uint32_t reason) {
      if (hera_ && cfg_.hera_keepalive) {
        try { hera_->send_global_abort(reason); } catch (...) {}
      }
    });
    watchdog_->start();
  }
}

// ---------------------------------------------------------------------------------------------
// Plane for ranks that share a GPU.  Every rank owns a staging buffer in device memory that all
// ranks map over CUDA IPC.  An AllReduce is, per piece of at most one staging buffer:
//   copy the input into my staging  ->  host barrier  ->  ONE kernel per rank that adds all ranks'
//   staging in rank order into my result  ->  host barrier (staging may be overwritten again).
// No kernel ever waits for another process's kernel; the ranks meet on the HOST, on per-rank epoch
// words in the shared page (bounded by the watchdog timeout, ended by the abort word).  The call is
// host-synchronous, like the reference's (reference: src/mini_nccl.cu:200-214).  This is what the
// reference's CUDA-IPC branch (reference: src/mini_nccl.cu:128-133,171-176) is meant to be.
void Comm::init_shared_gpu_plane() {
  if (!shm_map_ || private_host_)
    fail(Result::SystemError, "ranks that share a GPU need the host's shared page for their barrier (shm_open failed)");
  shared_stage_bytes_ = std::min<size_t>(cfg_.staging_bytes, size_t(64) << 20);
  RT_CHECK(cudaMalloc(reinterpret_cast<void**>(&shared_stage_), shared_stage_bytes_), "cudaMalloc(shared staging)");
  RT_CHECK(cudaMalloc(reinterpret_cast<void**>(&shared_out_), shared_stage_bytes_), "cudaMalloc(shared result staging)");
  struct Wire {
    cudaIpcMemHandle_t handle;
    int32_t ok;
  } mine{};
  mine.ok = cudaIpcGetMemHandle(&mine.handle, shared_stage_) == cudaSuccess ? 1 : 0;
  if (!mine.ok) (void)cudaGetLastError();
  std::vector<Wire> all(size_);
  store_->all_gather(&mine, all.data(), sizeof(mine));
  shared_peer_stage_.assign(size_, nullptr);
  bool ok = true;
  for (int r = 0; r < size_ && ok; ++r) {
    if (!all[r].ok) { ok = false; break; }
    if (r == rank_) { shared_peer_stage_[r] = shared_stage_; continue; }
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, all[r].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      (void)cudaGetLastError();
      ok = false;
      break;
    }
    shared_peer_stage_[r] = static_cast<char*>(p);
  }
  uint8_t mine_ok = ok ? 1 : 0;
  std::vector<uint8_t> oks(size_);
  store_->all_gather(&mine_ok, oks.data(), 1);
  for (uint8_t v : oks) ok = ok && v;
  if (!ok) fail(Result::SystemError, "cannot map the peers' staging over CUDA IPC");
  memset(&dev_, 0, sizeof(dev_));
  dev_.rank = rank_;
  dev_.nranks = size_;
}

// All ranks of the host meet: each publishes its epoch in its own words of the shared page and waits
// until every rank's epoch has caught up.  Bounded; the abort word ends it.
void Comm::host_barrier() {
  volatile uint32_t* words = static_cast<volatile uint32_t*>(shm_map_);
  const uint32_t e = ++shared_epoch_;
  __atomic_store_n(const_cast<uint32_t*>(progress_host_ + 8), e, __ATOMIC_RELEASE);
  const auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; r < size_; ++r) {
    volatile uint32_t* w = words + kProgressWords * (1 + r) + 8;
    uint32_t spins = 0;
    while (static_cast<int32_t>(__atomic_load_n(const_cast<uint32_t*>(w), __ATOMIC_ACQUIRE) - e) < 0) {
      if ((++spins & 1023u) != 0) continue;
      if (*abort_host_ != 0) {
        aborted_.store(true);
        fail(Result::InternalError, "NCCL Watchdog Timeout: Communication hang detected.");
      }
      const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
      if (ms > cfg_.watchdog_timeout_ms) {
        log_always("Watchdog", "TIMEOUT DETECTED! rank %d waited %lld ms for rank %d at a host barrier", rank_, static_cast<long long>(ms), r);
        __atomic_store_n(const_cast<uint32_t*>(abort_host_), 1u, __ATOMIC_RELEASE);
        aborted_.store(true);
        fail(Result::InternalError, "NCCL Watchdog Timeout: Communication hang detected.");
      }
      if (spins > (1u << 16)) std::this_thread::yield();
    }
  }
}

void Comm::shared_gpu_all_reduce(const void* send, void* recv, size_t count, DType t, RedOp op, double scale,
                                 cudaStream_t stream) {
  const size_t esz = dtype_size(t);
  const bool is_float = t == DType::Float16 || t == DType::Bfloat16 || t == DType::Float32 || t == DType::Float64;
  if (!is_float && scale != 1.0) fail(Result::InvalidArgument, "a scale factor needs a floating-point type");
  const MemKind sk = classify(send, true), rk = classify(recv, true);
  if (sk == MemKind::PlainHost || rk == MemKind::PlainHost)
    fail(Result::InvalidArgument, "buffers must be device memory or pinned host memory");
  LaunchSpec spec;
  spec.algo = Algo::HostSync;
  spec.mode = Mode::AllReduce;
  spec.in = spec.wire = spec.out = t;
  spec.op = op;
  spec.nthreads = 512;
  if (!kernel_exists(spec)) fail(Result::InvalidArgument, "no kernel for this type / operator combination");
  const size_t cap = (shared_stage_bytes_ / esz) & ~size_t(15);
  const double factor = scale * (op == RedOp::Avg ? 1.0 / static_cast<double>(size_) : 1.0);
  for (size_t off = 0; off < count; off += cap) {
    const size_t n = std::min(cap, count - off);
    RT_CHECK(cudaMemcpyAsync(shared_stage_, static_cast<const char*>(send) + off * esz, n * esz, cudaMemcpyDefault, stream),
             "cudaMemcpyAsync(stage)");
    RT_CHECK(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    host_barrier();  // every rank's piece is staged
    KParams kp;
    memset(&kp, 0, sizeof(kp));
    kp.comm = dev_;
    CollArgs& a = kp.args;
    for (int r = 0; r < size_; ++r) a.in_peer[r] = shared_peer_stage_[r];
    char* dst = static_cast<char*>(recv) + off * esz;
    const bool to_host = rk != MemKind::Device;
    a.recv = to_host ? static_cast<void*>(shared_out_) : static_cast<void*>(dst);
    a.count = n;
    a.scale_f = static_cast<float>(factor);
    a.scale_d = factor;
    a.int_div = (op == RedOp::Avg && !is_float) ? size_ : 0;
    const size_t vecs = (n * esz + 15) / 16;
    spec.nblocks = static_cast<int>(std::min<size_t>(std::max<size_t>(vecs / 2048, 1), 592));
    RT_CHECK(launch_collective(spec, kp, stream), "kernel launch");
    if (to_host) RT_CHECK(cudaMemcpyAsync(dst, shared_out_, n * esz, cudaMemcpyDeviceToHost, stream), "cudaMemcpyAsync(result)");
    RT_CHECK(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    host_barrier();  // every rank has read every staging: it may be overwritten
  }
}

void Comm::init_net_plane() {
  std::string kind = cfg_.transport;
  if (kind == "nvlink" || kind.empty()) kind = "auto";
  transport_ = make_transport(kind, rank_, size_);
  transport_->connect(*store_);
  ring_.reset(new RingAllReduce(rank_, size_, transport_.get(), store_.get(), cfg_, abort_host_));
}

Comm::~Comm() {
  if (hera_) hera_->stop_agent();
  if (watchdog_) watchdog_->stop();
  if (has_gpu_ && device_ >= 0) {
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    (void)cudaGetLastError();
  }
  // Goodbye barrier, so that nobody unmaps memory a peer's kernel still uses.
  // A dead peer must not hold destroy up for long: errors are swallowed.
  if (store_ && !aborted_.load()) {
    try { store_->barrier(); } catch (...) {}
  }
  if (pipe_) {
    cudaStreamDestroy(pipe_->s_in);
    cudaStreamDestroy(pipe_->s_out);
    cudaEventDestroy(pipe_->ev_start);
    for (int h = 0; h < 2; ++h) {
      cudaEventDestroy(pipe_->ev_in[h]);
      cudaEventDestroy(pipe_->ev_comm[h]);
      cudaEventDestroy(pipe_->ev_out[h]);
    }
    pipe_.reset();
  }
  if (solo_stage_) {
    cudaFree(solo_stage_);
    solo_stage_ = nullptr;
  }
  for (int r = 0; r < static_cast<int>(shared_peer_stage_.size()); ++r)
    if (r != rank_ && shared_peer_stage_[r]) cudaIpcCloseMemHandle(shared_peer_stage_[r]);
  shared_peer_stage_.clear();
  if (shared_stage_) cudaFree(shared_stage_);
  if (shared_out_) cudaFree(shared_out_);
  shared_stage_ = shared_out_ = nullptr;
  ring_.reset();
  transport_.reset();
  {
    std::lock_guard<std::mutex> lk(seg_mu_);
    user_segments_.clear();
  }
  for (auto& kv : ipc_cache_) cudaIpcCloseMemHandle(kv.second.base);
  ipc_cache_.clear();
  if (auto_map_dev_) cudaFree(auto_map_dev_);
  if (auto_stream_) cudaStreamDestroy(auto_stream_);
  auto_map_dev_ = nullptr;
  auto_stream_ = nullptr;
  ctrl_.reset();
  symm_.reset();
  fds_.reset();
  if (bounce_) {
    if (has_gpu_) cudaFreeHost(bounce_); else free(bounce_);
  }
  if (shm_registered_) cudaHostUnregister(shm_map_);
  if (shm_map_) munmap(shm_map_, shm_bytes_);
  if (private_host_) {
    if (has_gpu_) cudaFreeHost(private_host_); else free(private_host_);
  }
  (void)cudaGetLastError();
}

void Comm::check_usable() {
  if (aborted_.load()) fail(Result::InternalError, "communicator was aborted");
  if (abort_host_ && *abort_host_ != 0) {
    aborted_.store(true);
    fail(Result::InternalError, "NCCL Watchdog Timeout: Communication hang detected.");
  }
  if (progress_host_ && progress_host_[2] != 0) {
    aborted_.store(true);
    fail(Result::InternalError, "a collective kernel reported a failed wait (status " + std::to_string(progress_host_[2]) + ")");
  }
}

std::shared_ptr<Segment> Comm::find_segment(const void* ptr, size_t bytes, size_t* offset) {
  std::lock_guard<std::mutex> lk(seg_mu_);
  const uintptr_t p = reinterpret_cast<uintptr_t>(ptr);
  auto it = user_segments_.upper_bound(p);
  if (it == user_segments_.begin()) return nullptr;
  --it;
  const uintptr_t base = it->first;
  if (p >= base && p + bytes <= base + it->second->mapped_bytes) {
    if (offset) *offset = p - base;
    return it->second;
  }
  return nullptr;
}

void Comm::launch(Mode mode, const void* send, DType send_t, void* recv, DType recv_t, DType wire_t, size_t count,
                  RedOp op, double scale, Algo forced, cudaStream_t stream) {
  const bool is_float = send_t == DType::Float16 || send_t == DType::Bfloat16 || send_t == DType::Float32 ||
                        send_t == DType::Float64;
  if (!is_float && scale != 1.0) fail(Result::InvalidArgument, "a scale factor needs a floating-point type");
  const size_t in_elems = mode == Mode::ReduceScatter ? count * size_ : count;
  const size_t out_elems = mode == Mode::AllGather ? count * size_ : count;
  const size_t in_bytes = in_elems * dtype_size(send_t), out_bytes = out_elems * dtype_size(recv_t);
  PlanInput pi;
  pi.mode = mode;
  pi.count = count;
  pi.in = send_t;
  pi.wire = wire_t;
  pi.out = recv_t;
  pi.op = op;
  pi.forced = forced;
  size_t in_off = 0, out_off = 0;
  std::shared_ptr<Segment> in_seg, out_seg;
  if (size_ > 1) {
    in_seg = find_segment(send, in_bytes, &in_off);
    out_seg = find_segment(recv, out_bytes, &out_off);
    // A registered buffer that was freed and whose address range now belongs to another allocation: the
    // peers' mappings point at the old memory.  Nothing can be reduced into the right place any more
    // (and the ranks could disagree on whether the buffer still counts as registered), so the call is
    // refused: buffers are deregistered before they are freed.
    for (const auto* sp : {&in_seg, &out_seg}) {
      if (*sp && (*sp)->buffer_id != 0) {
        const void* p = sp == &in_seg ? send : recv;
        const unsigned long long now = allocation_id(p);
        if (now != 0 && now != (*sp)->buffer_id) {
          stats_.stale_registrations++;
          fail(Result::InvalidUsage, "a buffer registered with mncclCommRegister was freed and its address range allocated "
                                     "again; call mncclCommDeregister before freeing a registered buffer");
        }
      }
    }

    pi.in_symmetric = in_seg && (reinterpret_cast<uintptr_t>(send) & 15u) == 0;
    pi.out_symmetric = out_seg && (reinterpret_cast<uintptr_t>(recv) & 15u) == 0;
    pi.in_has_mc = in_seg && in_seg->mc;
    pi.out_has_mc = out_seg && out_seg->mc;
    // Buffers registered through CUDA IPC have no multicast mapping.  Where the switch is
    // available and the message is large, the pipelined NVLS path (measured 716 GB/s at 1 GiB on
    // 8 GPUs) beats the zero-copy peer-to-peer two-shot (624 GB/s): treat them as ordinary there.
    const bool switch_sum = (op == RedOp::Sum || op == RedOp::Avg) &&
                            (wire_t == DType::Float32 || wire_t == DType::Float16 || wire_t == DType::Bfloat16);
    const size_t demote_from = cfg_.pipe_min_bytes ? cfg_.pipe_min_bytes : cfg_.pipeline_min_bytes;
    if (mode == Mode::AllReduce && caps_.nvls && size_ > 2 && switch_sum && demote_from != 0 &&
        count * dtype_size(wire_t) >= demote_from) {
      if (in_seg && !in_seg->mc) pi.in_symmetric = false;
      if (out_seg && !out_seg->mc) pi.out_symmetric = false;
    }
  }
  // Kernels dereference these pointers: pageable host memory would fault.  (One driver query per
  // buffer that is not in symmetric memory; the result also decides on the host pipeline below.)
  const MemKind send_kind = in_seg ? MemKind::Device : classify(send, true);
  const MemKind recv_kind = out_seg ? MemKind::Device : (recv == send ? send_kind : classify(recv, true));
  if (send_kind == MemKind::PlainHost || recv_kind == MemKind::PlainHost)
    fail(Result::InvalidArgument, "buffers must be device memory or pinned host memory on the GPU data plane");
  pi.host_memory = send_kind == MemKind::PinnedHost || recv_kind == MemKind::PinnedHost;
  pi.auto_eligible = auto_shm_ != nullptr && cfg_.auto_map && mode == Mode::AllReduce && size_ > 1 && !in_seg && !out_seg &&
                     send_t == wire_t && recv_t == wire_t && send_kind == MemKind::Device && recv_kind == MemKind::Device;
  Plan plan = make_plan(pi, caps_, cfg_);
  if (!plan.valid) fail(Result::InvalidArgument, std::string("no kernel for this request: ") + plan.reason);
  if (!kernel_exists(plan.spec)) fail(Result::InvalidArgument, "no kernel for this type / operator combination");
  // range in the library's NVTX domain: "<collective>/<algorithm>", payload = bytes
  static const char* const kModeNames[] = {"allreduce", "reducescatter", "allgather"};
  char range_name[48];
  snprintf(range_name, sizeof(range_name), "%s/%s", kModeNames[static_cast<int>(mode) % 3], algo_name(plan.spec.algo));
  NvtxDomainRange nvtx_range(range_name, in_bytes);
  // Pinned host buffers: the copy engines move them (both directions at once over PCIe) in chunks
  // that overlap the collective, instead of kernels reading and writing host memory word by word.
  const bool host_in = send_kind == MemKind::PinnedHost;
  const bool host_out = recv_kind == MemKind::PinnedHost;
  bool host_pipe = mode == Mode::AllReduce && (host_in || host_out) && cfg_.host_pipeline_min_bytes != 0 &&
                   std::max(in_bytes, out_bytes) >= cfg_.host_pipeline_min_bytes;
  if (host_pipe && (!pipe_ || (size_ == 1 && solo_stage_ == nullptr))) {
    // The first pipelined call creates streams, events and (one rank) device staging: not while a
    // graph is being captured.  Such a call takes the direct kernel instead.
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) (void)cudaGetLastError();
    if (cs == cudaStreamCaptureStatusActive) host_pipe = false;
  }
  if (host_pipe && size_ == 1) {
    launch_solo_host(send, send_t, recv, recv_t, count, scale, stream, host_in, host_out);  // one rank: Avg == Sum
    stats_.calls++;
    stats_.bytes += in_bytes;
    stats_.pipelined++;
    return;
  }
  // Ordinary device buffers of the peer-to-peer two-shot AllReduce: export what is new, map what the
  // peers have exported, and let the kernel go direct as soon as every rank can (twoshot_auto_body).
  // The choice of this kernel depends on the request only, never on what has been mapped so far, so
  // every rank launches the same kernel.
  AutoDesc auto_desc{};
  bool auto_direct = false;
  if (auto_shm_ && cfg_.auto_map && mode == Mode::AllReduce && size_ > 1 && plan.spec.algo == Algo::TwoShot && plan.copy_in &&
      plan.copy_out && !in_seg && !out_seg && send_t == wire_t && recv_t == wire_t && send_kind == MemKind::Device &&
      recv_kind == MemKind::Device && !host_pipe) {
    LaunchSpec probe = plan.spec;
    probe.auto_direct = true;
    if (kernel_exists(probe)) {
      auto_direct = true;
      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) (void)cudaGetLastError();
      const bool live = cs != cudaStreamCaptureStatusActive;   // nothing is exported or mapped while a graph is being captured
      const int s_slot = auto_export(send, in_bytes, live);
      const int r_slot = recv == send ? s_slot : auto_export(recv, out_bytes, live);
      if (live) auto_import();
      const bool usable = s_slot >= 0 && r_slot >= 0 &&
                          ((reinterpret_cast<uintptr_t>(send) | reinterpret_cast<uintptr_t>(recv)) & 15u) == 0;
      auto_desc.send_addr = reinterpret_cast<uint64_t>(send);
      auto_desc.recv_addr = reinterpret_cast<uint64_t>(recv);
      auto_desc.slots = usable ? (static_cast<uint32_t>(s_slot) | (static_cast<uint32_t>(r_slot) << 8) | (1u << 16)) : 0u;
      for (int r = 0; r < size_ && r < kAutoRanks; ++r) auto_desc.mask[r] = auto_mask_[r];
    }
  }
  if (!auto_direct && mode == Mode::AllReduce && size_ > 1 && (plan.copy_in || plan.copy_out) &&
      (plan.spec.algo == Algo::TwoShot || plan.spec.algo == Algo::Nvls || host_pipe) &&
      ((cfg_.pipeline_min_bytes != 0 && count * dtype_size(wire_t) >= cfg_.pipeline_min_bytes) || host_pipe)) {
    launch_pipelined(send, send_t, recv, recv_t, wire_t, count, op, scale, forced, stream, host_pipe && host_in,
                     host_pipe && host_out);
    stats_.calls++;
    stats_.bytes += in_bytes;
    stats_.pipelined++;
    return;
  }

  KParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.comm = dev_;
  CollArgs& a = kp.args;
  a.send = send;
  a.recv = recv;
  a.count = count;
  a.shard_elems = plan.shard_elems;
  a.chunk_shard_vecs = plan.chunk_shard_vecs;
  const double factor = scale * (op == RedOp::Avg ? 1.0 / static_cast<double>(size_) : 1.0);
  a.scale_f = static_cast<float>(factor);
  a.scale_d = factor;
  a.int_div = (op == RedOp::Avg && !is_float) ? size_ : 0;
  a.copy_in = plan.copy_in ? 1 : 0;
  a.copy_out = plan.copy_out ? 1 : 0;
  a.pipe_ramp = plan.pipe_ramp;
  a.auto_desc = auto_desc;
  if (auto_direct) {
    plan.spec.auto_direct = true;
    if (plan.spec.nblocks > kAutoBlocks) plan.spec.nblocks = kAutoBlocks;
  }
  if (size_ > 1 && (plan.spec.algo == Algo::TwoShot || plan.spec.algo == Algo::Nvls)) {
    const bool zc_in = !plan.copy_in && mode != Mode::AllGather;
    const bool zc_out = !plan.copy_out && mode != Mode::ReduceScatter;
    for (int r = 0; r < size_; ++r) {
      a.in_peer[r] = zc_in ? static_cast<char*>(in_seg->peer[r]) + in_off : dev_.ctrl[r] + dev_.off_stage_a;
      a.out_peer[r] = zc_out ? static_cast<char*>(out_seg->peer[r]) + out_off : dev_.ctrl[r] + dev_.off_stage_b;
    }
    a.in_mc = zc_in ? (in_seg->mc ? static_cast<char*>(in_seg->mc) + in_off : nullptr)
                    : (dev_.ctrl_mc ? dev_.ctrl_mc + dev_.off_stage_a : nullptr);
    a.out_mc = zc_out ? (out_seg->mc ? static_cast<char*>(out_seg->mc) + out_off : nullptr)
                      : (dev_.ctrl_mc ? dev_.ctrl_mc + dev_.off_stage_b : nullptr);
    if (zc_in) stats_.zero_copy_in++;
    if (zc_out) stats_.zero_copy_out++;
    if (plan.copy_in || plan.copy_out) stats_.staged_passes++;
  }
  if (plan.spec.algo == Algo::Pipe) stats_.staged_passes++;
  if (size_ == 1 && mode == Mode::AllReduce && send == recv && send_t == recv_t && factor == 1.0) {
    // Nothing to do; keep stream order semantics without a launch.
  } else {
    RT_CHECK(launch_collective(plan.spec, kp, stream), "kernel launch");
  }
  stats_.calls++;
  stats_.bytes += in_bytes;
  stats_.by_algo[static_cast<int>(plan.spec.algo)]++;
}

// Large AllReduce on ordinary buffers.  The two-phase kernels need their operands in symmetric
// memory; instead of staging inside one kernel (copy, barrier, reduce, barrier, copy: the
// link idles during the copies) the message is cut into chunks that flow through two halves of
// the staging areas: a copy-in kernel on one side stream, the zero-copy collective on the
// caller's stream, a copy-out kernel on another side stream, tied together with events.  The
// collective of chunk i overlaps the copy-in of chunk i+1 and the copy-out of chunk i-1.
// Slot reuse is safe across ranks because every collective kernel starts and ends with a
// cross-rank barrier: a peer touches this rank's half only between those two barriers, and this
// rank enters the barrier of chunk i+2 only after its own copy-out of chunk i.
void Comm::ensure_pipeline() {
  if (pipe_) return;
  {
    pipe_.reset(new Pipeline());
    RT_CHECK(cudaStreamCreateWithFlags(&pipe_->s_in, cudaStreamNonBlocking), "cudaStreamCreate");
    RT_CHECK(cudaStreamCreateWithFlags(&pipe_->s_out, cudaStreamNonBlocking), "cudaStreamCreate");
    RT_CHECK(cudaEventCreateWithFlags(&pipe_->ev_start, cudaEventDisableTiming), "cudaEventCreate");
    for (int h = 0; h < 2; ++h) {
      RT_CHECK(cudaEventCreateWithFlags(&pipe_->ev_in[h], cudaEventDisableTiming), "cudaEventCreate");
      RT_CHECK(cudaEventCreateWithFlags(&pipe_->ev_comm[h], cudaEventDisableTiming), "cudaEventCreate");
      RT_CHECK(cudaEventCreateWithFlags(&pipe_->ev_out[h], cudaEventDisableTiming), "cudaEventCreate");
    }
  }
}

void Comm::launch_pipelined(const void* send, DType send_t, void* recv, DType recv_t, DType wire_t, size_t count,
                            RedOp op, double scale, Algo forced, cudaStream_t stream, bool host_in, bool host_out) {
  ensure_pipeline();
  const size_t wsz = dtype_size(wire_t), osz = dtype_size(recv_t), isz = dtype_size(send_t);
  const size_t half = (caps_.stage_bytes / 2) & ~size_t(4095);
  // Chunks: a quarter of the message, at least 32 MB (the collective kernel needs size to be
  // efficient: measured 620 GB/s bus bandwidth at 32 MB, 770 at 128 MB on 8 GPUs), at most what
  // one half of the staging holds.
  size_t chunk_bytes = std::max<size_t>(count * wsz / 4, size_t(32) << 20);
  // Host buffers: PCIe (not NVLink) sets the pace, so chunks are small: the exposed head (first
  // copy-in) and tail (last collective and copy-out) shrink with them.
  if (host_in || host_out) chunk_bytes = cfg_.host_chunk_bytes;
  size_t chunk = chunk_bytes / wsz;
  chunk = std::min(chunk, half / std::max(wsz, osz));
  chunk &= ~size_t(4095);
  if (chunk == 0) fail(Result::InternalError, "staging too small for the chunk pipeline");
  const std::vector<size_t> chunks = pipeline_chunks(count, wsz, chunk, (half / std::max(wsz, osz)) & ~size_t(4095),
                                                     cfg_.pipeline_taper && !host_in && !host_out);
  const bool is_float = send_t != DType::Int8 && send_t != DType::Uint8 && send_t != DType::Int32 &&
                        send_t != DType::Uint32 && send_t != DType::Int64 && send_t != DType::Uint64;
  const double factor = scale * (op == RedOp::Avg ? 1.0 / static_cast<double>(size_) : 1.0);

  auto local_copy = [&](const void* src, DType st, void* dst, DType dt, size_t n, cudaStream_t s) {
    LaunchSpec ls;
    ls.algo = Algo::Local;
    ls.in = st;
    ls.wire = (st == dt) ? st : DType::Bfloat16;  // the mixed triples all travel as bf16
    ls.out = dt;
    ls.op = RedOp::Sum;
    ls.nthreads = 512;
    const size_t vecs = (n * std::max(dtype_size(st), dtype_size(dt)) + 15) / 16;
    ls.nblocks = static_cast<int>(std::min<size_t>(std::max<size_t>(vecs / 2048, 1), 48));
    KParams kp;
    memset(&kp, 0, sizeof(kp));
    kp.comm = dev_;
    kp.args.send = src;
    kp.args.recv = dst;
    kp.args.count = n;
    kp.args.scale_f = 1.0f;
    kp.args.scale_d = 1.0;
    if (!kernel_exists(ls)) fail(Result::InvalidArgument, "no copy kernel for this type combination");
    RT_CHECK(launch_collective(ls, kp, s), "copy kernel launch");
  };

  RT_CHECK(cudaEventRecord(pipe_->ev_start, stream), "cudaEventRecord");
  RT_CHECK(cudaStreamWaitEvent(pipe_->s_in, pipe_->ev_start, 0), "cudaStreamWaitEvent");
  RT_CHECK(cudaStreamWaitEvent(pipe_->s_out, pipe_->ev_start, 0), "cudaStreamWaitEvent");
  size_t i = 0;
  for (size_t off = 0; i < chunks.size(); off += chunks[i], ++i) {
    const int h = static_cast<int>(i & 1);
    const size_t n = chunks[i];
    char* a_h = dev_.ctrl[rank_] + dev_.off_stage_a + h * half;
    char* b_h = dev_.ctrl[rank_] + dev_.off_stage_b + h * half;
    // copy-in (after the collective that last read this half)
    if (i >= 2) RT_CHECK(cudaStreamWaitEvent(pipe_->s_in, pipe_->ev_comm[h], 0), "cudaStreamWaitEvent");
    if ((host_in || cfg_.pipeline_copy_engine) && send_t == wire_t)
      RT_CHECK(cudaMemcpyAsync(a_h, static_cast<const char*>(send) + off * isz, n * isz, cudaMemcpyDefault, pipe_->s_in), "cudaMemcpyAsync");
    else
      local_copy(static_cast<const char*>(send) + off * isz, send_t, a_h, wire_t, n, pipe_->s_in);
    RT_CHECK(cudaEventRecord(pipe_->ev_in[h], pipe_->s_in), "cudaEventRecord");
    // collective on the staging halves, zero-copy (after the copy-out that last read B_h)
    RT_CHECK(cudaStreamWaitEvent(stream, pipe_->ev_in[h], 0), "cudaStreamWaitEvent");
    if (i >= 2) RT_CHECK(cudaStreamWaitEvent(stream, pipe_->ev_out[h], 0), "cudaStreamWaitEvent");
    PlanInput pi;
    pi.mode = Mode::AllReduce;
    pi.count = n;
    pi.in = wire_t;
    pi.wire = wire_t;
    pi.out = recv_t;
    pi.op = op;
    pi.forced = forced;
    pi.in_symmetric = pi.out_symmetric = true;
    pi.in_has_mc = pi.out_has_mc = caps_.nvls;
    Plan plan = make_plan(pi, caps_, cfg_);
    if (!plan.valid || plan.copy_in || plan.copy_out || !kernel_exists(plan.spec))
      fail(Result::InternalError, "chunk pipeline: no zero-copy plan for a chunk");
    if (plan.spec.algo != Algo::TwoShot && plan.spec.algo != Algo::Nvls) {
      plan.spec.algo = Algo::TwoShot;  // small tail chunk: stay on a kernel that uses the staging views
      if (!kernel_exists(plan.spec)) fail(Result::InternalError, "chunk pipeline: no kernel");
      const uint64_t VW = 16 / wsz;
      plan.shard_elems = ((n + VW - 1) / VW + size_ - 1) / size_ * VW;
      plan.chunk_shard_vecs = (plan.shard_elems + VW - 1) / VW;
      plan.spec.nthreads = 512;
      plan.spec.nblocks = static_cast<int>(std::min<uint64_t>(std::max<uint64_t>(plan.chunk_shard_vecs / 2048, 1), 96));
    }
    KParams kp;
    memset(&kp, 0, sizeof(kp));
    kp.comm = dev_;
    CollArgs& a = kp.args;
    a.send = a_h;
    a.recv = b_h;
    a.count = n;
    a.shard_elems = plan.shard_elems;
    a.chunk_shard_vecs = plan.chunk_shard_vecs;
    a.scale_f = static_cast<float>(factor);
    a.scale_d = factor;
    a.int_div = (op == RedOp::Avg && !is_float) ? size_ : 0;
    for (int r = 0; r < size_; ++r) {
      a.in_peer[r] = dev_.ctrl[r] + dev_.off_stage_a + h * half;
      a.out_peer[r] = dev_.ctrl[r] + dev_.off_stage_b + h * half;
    }
    a.in_mc = dev_.ctrl_mc ? dev_.ctrl_mc + dev_.off_stage_a + h * half : nullptr;
    a.out_mc = dev_.ctrl_mc ? dev_.ctrl_mc + dev_.off_stage_b + h * half : nullptr;
    RT_CHECK(launch_collective(plan.spec, kp, stream), "kernel launch");
    RT_CHECK(cudaEventRecord(pipe_->ev_comm[h], stream), "cudaEventRecord");
    stats_.by_algo[static_cast<int>(plan.spec.algo)]++;
    // copy-out
    RT_CHECK(cudaStreamWaitEvent(pipe_->s_out, pipe_->ev_comm[h], 0), "cudaStreamWaitEvent");
    if (host_out || cfg_.pipeline_copy_engine)
      RT_CHECK(cudaMemcpyAsync(static_cast<char*>(recv) + off * osz, b_h, n * osz, cudaMemcpyDefault, pipe_->s_out), "cudaMemcpyAsync");
    else
      local_copy(b_h, recv_t, static_cast<char*>(recv) + off * osz, recv_t, n, pipe_->s_out);
    RT_CHECK(cudaEventRecord(pipe_->ev_out[h], pipe_->s_out), "cudaEventRecord");
  }
  RT_CHECK(cudaStreamWaitEvent(stream, pipe_->ev_out[0], 0), "cudaStreamWaitEvent");
  if (i >= 2) RT_CHECK(cudaStreamWaitEvent(stream, pipe_->ev_out[1], 0), "cudaStreamWaitEvent");
}

// One rank, pinned host buffers: out = factor * in with the types converted, as a three-stage
// pipeline through private device staging: copy engine in, kernel, copy engine out.  Host -> device
// and device -> host run at the same time (PCIe is full duplex).
void Comm::launch_solo_host(const void* send, DType send_t, void* recv, DType recv_t, size_t count, double factor,
                            cudaStream_t stream, bool host_in, bool host_out) {
  ensure_pipeline();
  const size_t isz = dtype_size(send_t), osz = dtype_size(recv_t);
  size_t chunk = cfg_.host_chunk_bytes / std::max(isz, osz);
  chunk &= ~size_t(4095);
  if (chunk == 0) chunk = 4096;
  const size_t half = (std::max(cfg_.host_chunk_bytes, chunk * std::max(isz, osz)) + 255) & ~size_t(255);  // the same for every type
  if (solo_stage_ == nullptr || solo_stage_half_ < half) {
    if (solo_stage_) {
      RT_CHECK(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
      cudaFree(solo_stage_);
      solo_stage_ = nullptr;
    }
    RT_CHECK(cudaMalloc(reinterpret_cast<void**>(&solo_stage_), 4 * half), "cudaMalloc (host staging)");
    solo_stage_half_ = half;
  }
  LaunchSpec ls;
  ls.algo = Algo::Local;
  ls.in = send_t;
  ls.wire = (send_t == recv_t) ? send_t : DType::Bfloat16;
  ls.out = recv_t;
  ls.op = RedOp::Sum;
  ls.nthreads = 512;
  if (!kernel_exists(ls)) fail(Result::InvalidArgument, "no kernel for this type combination");
  // only the side streams that get work are forked (a forked stream must be joined under capture)
  RT_CHECK(cudaEventRecord(pipe_->ev_start, stream), "cudaEventRecord");
  if (host_in) RT_CHECK(cudaStreamWaitEvent(pipe_->s_in, pipe_->ev_start, 0), "cudaStreamWaitEvent");
  if (host_out) RT_CHECK(cudaStreamWaitEvent(pipe_->s_out, pipe_->ev_start, 0), "cudaStreamWaitEvent");
  size_t i = 0;
  for (size_t off = 0; off < count; off += chunk, ++i) {
    const int h = static_cast<int>(i & 1);
    const size_t n = std::min(chunk, count - off);
    char* a_h = solo_stage_ + h * half;
    char* b_h = solo_stage_ + (2 + h) * half;
    const char* src = static_cast<const char*>(send) + off * isz;
    char* dst = static_cast<char*>(recv) + off * osz;
    const void* k_in = src;
    if (host_in) {
      if (i >= 2) RT_CHECK(cudaStreamWaitEvent(pipe_->s_in, pipe_->ev_comm[h], 0), "cudaStreamWaitEvent");
      RT_CHECK(cudaMemcpyAsync(a_h, src, n * isz, cudaMemcpyHostToDevice, pipe_->s_in), "cudaMemcpyAsync");
      RT_CHECK(cudaEventRecord(pipe_->ev_in[h], pipe_->s_in), "cudaEventRecord");
      RT_CHECK(cudaStreamWaitEvent(stream, pipe_->ev_in[h], 0), "cudaStreamWaitEvent");
      k_in = a_h;
    }
    if (host_out && i >= 2) RT_CHECK(cudaStreamWaitEvent(stream, pipe_->ev_out[h], 0), "cudaStreamWaitEvent");
    KParams kp;
    memset(&kp, 0, sizeof(kp));
    kp.comm = dev_;
    kp.args.send = k_in;
    kp.args.recv = host_out ? static_cast<void*>(b_h) : static_cast<void*>(dst);
    kp.args.count = n;
    kp.args.scale_f = static_cast<float>(factor);
    kp.args.scale_d = factor;
    const size_t vecs = (n * std::max(isz, osz) + 15) / 16;
    ls.nblocks = static_cast<int>(std::min<size_t>(std::max<size_t>(vecs / 2048, 1), 96));
    RT_CHECK(launch_collective(ls, kp, stream), "kernel launch");
    RT_CHECK(cudaEventRecord(pipe_->ev_comm[h], stream), "cudaEventRecord");
    if (host_out) {
      RT_CHECK(cudaStreamWaitEvent(pipe_->s_out, pipe_->ev_comm[h], 0), "cudaStreamWaitEvent");
      RT_CHECK(cudaMemcpyAsync(dst, b_h, n * osz, cudaMemcpyDeviceToHost, pipe_->s_out), "cudaMemcpyAsync");
      RT_CHECK(cudaEventRecord(pipe_->ev_out[h], pipe_->s_out), "cudaEventRecord");
    }
  }
  stats_.by_algo[static_cast<int>(Algo::Local)]++;
  if (host_out) {
    RT_CHECK(cudaStreamWaitEvent(stream, pipe_->ev_out[0], 0), "cudaStreamWaitEvent");
    if (i >= 2) RT_CHECK(cudaStreamWaitEvent(stream, pipe_->ev_out[1], 0), "cudaStreamWaitEvent");
  }
}

void Comm::wait_blocking(cudaStream_t stream) {
  // Reference behaviour on request (MINI_NCCL_BLOCKING=1): return only when
  // the stream has drained, report a watchdog trip as an error.
  for (;;) {
    cudaError_t q = cudaStreamQuery(stream);
    if (q == cudaSuccess) break;
    if (q != cudaErrorNotReady) {
      (void)cudaGetLastError();
      fail(Result::UnhandledCudaError, std::string("stream error: ") + cudaGetErrorString(q));
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
  check_usable();
}

void Comm::all_reduce(const void* send, DType send_t, void* recv, DType recv_t, DType wire_t, size_t count, RedOp op,
                      double scale, Algo forced, cudaStream_t stream) {
  std::lock_guard<std::mutex> lk(call_mu_);
  check_usable();
  bool capturing = false;
  if (has_gpu_) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cs) == cudaSuccess) capturing = cs == cudaStreamCaptureStatusActive;
    else (void)cudaGetLastError();
  }
  if (capturing) {
    stats_.graph_captures_seen++;
    if (!capture_warned_.exchange(true)) {
      if (gpu_plane_)
        MNCCL_INFO("Mini-NCCL", "CUDA Graph capture detected: the collective is captured as one kernel node; flags and epochs are device-resident, so replays are safe.");
      else
        log_always("Mini-NCCL", "[Warning] CUDA Graph capture detected, but this data plane is driven by the host and cannot be captured.");
    }
    if (!gpu_plane_) fail(Result::InvalidUsage, "the network data plane cannot run under CUDA Graph capture");
  }
  if (shared_plane_) {
    if (send_t != recv_t || send_t != wire_t) fail(Result::InvalidArgument, "ranks that share a GPU reduce homogeneous types");
    shared_gpu_all_reduce(send, recv, count, send_t, op, scale, stream);
    stats_.calls++;
    stats_.bytes += count * dtype_size(send_t);
    stats_.by_algo[static_cast<int>(Algo::HostSync)]++;
    return;
  }
  if (!gpu_plane_) {
    if (send_t != recv_t || send_t != wire_t || scale != 1.0)
      fail(Result::InvalidArgument, "the network data plane supports homogeneous types without a scale");
    ring_all_reduce(send, recv, count, send_t, op, stream);
    stats_.calls++;
    stats_.bytes += count * dtype_size(send_t);
    stats_.by_algo[static_cast<int>(Algo::Ring)]++;
    return;
  }
  if (forced == Algo::Auto) forced = parse_algo(cfg_.algo);
  if (forced == Algo::Ring) forced = Algo::Auto;
  launch(Mode::AllReduce, send, send_t, recv, recv_t, wire_t, count, op, scale, forced, stream);
  if (cfg_.blocking && !capturing) wait_blocking(stream);
}

void Comm::reduce_scatter(const void* send, void* recv, size_t recvcount, DType t, RedOp op, cudaStream_t stream) {
  std::lock_guard<std::mutex> lk(call_mu_);
  check_usable();
  if (!gpu_plane_) fail(Result::InvalidUsage, "ReduceScatter needs the GPU data plane");
  if (size_ == 1) {
    launch(Mode::AllReduce, send, t, recv, t, t, recvcount, op, 1.0, Algo::Auto, stream);
    return;
  }
  launch(Mode::ReduceScatter, send, t, recv, t, t, recvcount, op, 1.0, parse_algo(cfg_.algo), stream);
}

void Comm::all_gather(const void* send, void* recv, size_t sendcount, DType t, cudaStream_t stream) {
  std::lock_guard<std::mutex> lk(call_mu_);
  check_usable();
  if (!gpu_plane_) fail(Result::InvalidUsage, "AllGather needs the GPU data plane");
  if (size_ == 1) {
    if (send != recv) RT_CHECK(cudaMemcpyAsync(recv, send, sendcount * dtype_size(t), cudaMemcpyDefault, stream), "cudaMemcpyAsync");
    return;
  }
  launch(Mode::AllGather, send, t, recv, t, t, sendcount, RedOp::Sum, 1.0, Algo::TwoShot, stream);
}

void Comm::ring_all_reduce(const void* send, void* recv, size_t count, DType t, RedOp op, cudaStream_t stream) {
  const size_t bytes = count * dtype_size(t);
  if (has_gpu_) RT_CHECK(cudaStreamSynchronize(stream), "cudaStreamSynchronize");  // order after the caller's GPU work
  const MemKind sk = classify(send, has_gpu_), rk = classify(recv, has_gpu_);
  if (rk != MemKind::Device && sk != MemKind::Device) {
    if (send != recv) memmove(recv, send, bytes);
    ring_->run(recv, count, t, op);
    return;
  }
  // Device memory: bounce through pinned host memory.
  if (bounce_bytes_ < bytes) {
    if (bounce_) cudaFreeHost(bounce_);
    bounce_ = nullptr;
    bounce_bytes_ = 0;
    RT_CHECK(cudaHostAlloc(&bounce_, bytes, cudaHostAllocDefault), "cudaHostAlloc(bounce)");
    bounce_bytes_ = bytes;
  }
  RT_CHECK(cudaMemcpy(bounce_, send, bytes, cudaMemcpyDefault), "cudaMemcpy(D2H)");
  ring_->run(bounce_, count, t, op);
  RT_CHECK(cudaMemcpy(recv, bounce_, bytes, cudaMemcpyDefault), "cudaMemcpy(H2D)");
}

void* Comm::mem_alloc(size_t bytes) {
  if (!gpu_plane_) fail(Result::InvalidUsage, "symmetric allocations need the GPU data plane");
  if (size_ == 1) {
    void* p = nullptr;
    RT_CHECK(cudaMalloc(&p, bytes), "cudaMalloc");
    auto seg = std::make_shared<Segment>();
    seg->bytes = bytes;
    seg->mapped_bytes = bytes;
    seg->local = p;
    seg->peer.assign(1, p);
    std::lock_guard<std::mutex> lk(seg_mu_);
    user_segments_[reinterpret_cast<uintptr_t>(p)] = seg;
    return p;
  }
  std::shared_ptr<Segment> seg = symm_->allocate(bytes, true);
  std::lock_guard<std::mutex> lk(seg_mu_);
  user_segments_[reinterpret_cast<uintptr_t>(seg->local)] = seg;
  return seg->local;
}

void Comm::mem_free(void* ptr) {
  std::shared_ptr<Segment> seg;
  {
    std::lock_guard<std::mutex> lk(seg_mu_);
    auto it = user_segments_.find(reinterpret_cast<uintptr_t>(ptr));
    if (it == user_segments_.end()) fail(Result::InvalidArgument, "pointer was not returned by mncclMemAlloc");
    seg = it->second;
    user_segments_.erase(it);
  }
  if (size_ == 1) {
    cudaFree(ptr);
    return;
  }
  symm_->release(seg);
}

// Lazy direct access, host side.  Exporting and importing are one-sided and never wait for a peer:
// the kernel finds out per call whether every rank can reach every buffer (twoshot_auto_body).
int Comm::auto_export(const void* ptr, size_t bytes, bool may_export) {
  const unsigned long long id = allocation_id(ptr);
  if (id == 0 || !auto_shm_) return -1;
  AutoExportTable* mine = reinterpret_cast<AutoExportTable*>(auto_shm_) + rank_;
  const uint64_t addr = reinterpret_cast<uint64_t>(ptr);
  for (uint32_t i = 0; i < mine->count; ++i)
    if (mine->e[i].id == id) return (addr >= mine->e[i].base && addr + bytes <= mine->e[i].base + mine->e[i].size) ? static_cast<int>(i) : -1;
  if (!may_export) return -1;
  for (unsigned long long r : auto_refused_)
    if (r == id) return -1;
  if (mine->count >= static_cast<uint32_t>(kAutoSlots)) return -1;   // slots are never reused: later allocations stay staged
  const CudaDriver* d = CudaDriver::get();
  CUdeviceptr base = 0;
  size_t alloc_size = 0;
  AutoExport e{};
  if (!d || !d->MemGetAddressRange ||
      d->MemGetAddressRange(&base, &alloc_size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS ||
      cudaIpcGetMemHandle(&e.handle, reinterpret_cast<void*>(base)) != cudaSuccess) {
    (void)cudaGetLastError();
    if (auto_refused_.size() < 64) auto_refused_.push_back(id);
    return -1;
  }
  e.id = id;
  e.base = static_cast<uint64_t>(base);
  e.size = alloc_size;
  const uint32_t slot = mine->count;
  mine->e[slot] = e;
  __atomic_store_n(&mine->count, slot + 1, __ATOMIC_RELEASE);
  stats_.auto_exports++;
  return (addr + bytes <= e.base + e.size) ? static_cast<int>(slot) : -1;
}

void Comm::auto_import() {
  if (!auto_shm_) return;
  for (int r = 0; r < size_; ++r) {
    if (r == rank_) continue;
    AutoExportTable* t = reinterpret_cast<AutoExportTable*>(auto_shm_) + r;
    const uint32_t n = std::min<uint32_t>(__atomic_load_n(&t->count, __ATOMIC_ACQUIRE), kAutoSlots);
    for (uint32_t i = auto_seen_[r]; i < n; ++i) {
      const AutoExport e = t->e[i];
      std::string key(reinterpret_cast<const char*>(&e.handle), sizeof(cudaIpcMemHandle_t));
      key.push_back(static_cast<char>(r));
      auto it = ipc_cache_.find(key);
      if (it == ipc_cache_.end()) {
        void* opened = nullptr;
        if (cudaIpcOpenMemHandle(&opened, e.handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
          (void)cudaGetLastError();
          continue;   // stays unmapped: calls on that buffer keep staging
        }
        ++ipc_misses_;
        it = ipc_cache_.emplace(key, IpcMapping{opened, 0}).first;
      }
      it->second.refs++;   // held until the communicator goes
      // Row [peer][its slot] of the device table, on a stream of its own so that nothing queued on the
      // caller's streams is waited for.  Kernels only look at rows whose bit their launch carried, and
      // the bit is set after the copy has completed.
      const AutoMapEntry row{e.id, e.base, e.size, reinterpret_cast<uint64_t>(it->second.base)};
      if (cudaMemcpyAsync(auto_map_dev_ + r * kAutoSlots + i, &row, sizeof(row), cudaMemcpyHostToDevice, auto_stream_) != cudaSuccess ||
          cudaStreamSynchronize(auto_stream_) != cudaSuccess) {
        (void)cudaGetLastError();
        continue;
      }
      auto_mask_[r] = static_cast<uint16_t>(auto_mask_[r] | (1u << i));
      stats_.auto_imports++;
    }
    auto_seen_[r] = n;
  }
}

void Comm::register_buffer(void* ptr, size_t bytes) {
  std::lock_guard<std::mutex> lk(call_mu_);
  if (!gpu_plane_) fail(Result::InvalidUsage, "buffer registration needs the GPU data plane");
  if (!ptr || bytes == 0) fail(Result::InvalidArgument, "bad buffer");
  if (size_ == 1) return;
  if (find_segment(ptr, bytes, nullptr)) return;  // already symmetric or registered
  struct Wire {
    cudaIpcMemHandle_t handle;
    uint64_t offset;
    uint64_t bytes;
    int32_t ok;
    int32_t pad;
  } mine{};
  const CudaDriver* d = CudaDriver::get();
  CUdeviceptr base = 0;
  size_t alloc_size = 0;
  mine.ok = 0;
  if (d && d->MemGetAddressRange && classify(ptr, true) == MemKind::Device &&
      d->MemGetAddressRange(&base, &alloc_size, reinterpret_cast<CUdeviceptr>(ptr)) == CUDA_SUCCESS &&
      cudaIpcGetMemHandle(&mine.handle, reinterpret_cast<void*>(base)) == cudaSuccess) {
    mine.ok = 1;
    mine.offset = reinterpret_cast<uintptr_t>(ptr) - static_cast<uintptr_t>(base);
  } else {
    (void)cudaGetLastError();
  }
  mine.bytes = bytes;
  std::vector<Wire> all(size_);
  store_->all_gather(&mine, all.data(), sizeof(mine));
  for (int r = 0; r < size_; ++r) {
    if (!all[r].ok) fail(Result::InvalidUsage, "rank " + std::to_string(r) + " cannot export this buffer over CUDA IPC "
                                               "(only cudaMalloc-family device memory can be registered)");
    if (all[r].bytes != bytes) fail(Result::InvalidUsage, "registered sizes differ between ranks");
  }
  auto seg = std::make_shared<Segment>();
  seg->bytes = bytes;
  seg->mapped_bytes = bytes;
  seg->local = ptr;
  seg->peer.assign(size_, nullptr);
  seg->buffer_id = allocation_id(ptr);
  std::vector<std::string> keys;
  bool ok = true;
  for (int r = 0; r < size_; ++r) {
    if (r == rank_) {
      seg->peer[r] = ptr;
      continue;
    }
    std::string key(reinterpret_cast<const char*>(&all[r].handle), sizeof(cudaIpcMemHandle_t));
    key.push_back(static_cast<char>(r));
    auto it = ipc_cache_.find(key);
    if (it == ipc_cache_.end()) {
      void* opened = nullptr;
      if (cudaIpcOpenMemHandle(&opened, all[r].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        (void)cudaGetLastError();
        ok = false;
        break;
      }
      ++ipc_misses_;
      it = ipc_cache_.emplace(key, IpcMapping{opened, 0}).first;
    } else {
      ++ipc_hits_;
    }
    it->second.refs++;
    keys.push_back(key);
    seg->peer[r] = static_cast<char*>(it->second.base) + all[r].offset;
  }
  // every rank must end up in the same state
  uint8_t mine_ok = ok ? 1 : 0;
  std::vector<uint8_t> oks(size_);
  store_->all_gather(&mine_ok, oks.data(), 1);
  for (uint8_t v : oks) ok = ok && v;
  if (!ok) {
    for (const std::string& k : keys) {
      auto it = ipc_cache_.find(k);
      if (it != ipc_cache_.end() && --it->second.refs == 0) {
        cudaIpcCloseMemHandle(it->second.base);
        ipc_cache_.erase(it);
      }
    }
    fail(Result::UnhandledCudaError, "cudaIpcOpenMemHandle failed on at least one rank");
  }
  std::lock_guard<std::mutex> lk2(seg_mu_);
  user_segments_[reinterpret_cast<uintptr_t>(ptr)] = seg;
  registered_[reinterpret_cast<uintptr_t>(ptr)] = keys;
}

void Comm::deregister_buffer(void* ptr) {
  std::lock_guard<std::mutex> lk(call_mu_);
  if (size_ == 1) return;
  auto it = registered_.find(reinterpret_cast<uintptr_t>(ptr));
  if (it == registered_.end()) fail(Result::InvalidArgument, "buffer was not registered");
  if (has_gpu_) cudaDeviceSynchronize();
  store_->barrier();  // no peer kernel still reads this buffer
  for (const std::string& k : it->second) {
    auto c = ipc_cache_.find(k);
    if (c != ipc_cache_.end() && --c->second.refs == 0) {
      cudaIpcCloseMemHandle(c->second.base);
      ipc_cache_.erase(c);
    }
  }
  registered_.erase(it);
  std::lock_guard<std::mutex> lk2(seg_mu_);
  user_segments_.erase(reinterpret_cast<uintptr_t>(ptr));
}

void Comm::peer_pointers(void* ptr, void** peers, void** mc) {
  size_t off = 0;
  std::shared_ptr<Segment> seg = find_segment(ptr, 1, &off);
  if (!seg) fail(Result::InvalidArgument, "pointer is not inside a symmetric allocation");
  for (int r = 0; r < size_; ++r) peers[r] = static_cast<char*>(seg->peer[r]) + off;
  if (mc) *mc = seg->mc ? static_cast<char*>(seg->mc) + off : nullptr;
}

void Comm::barrier() { store_->barrier(); }

void Comm::abort() {
  aborted_.store(true);
  if (abort_host_) __atomic_store_n(const_cast<uint32_t*>(abort_host_), 1u, __ATOMIC_RELEASE);
  if (transport_) transport_->abort();
}

Result Comm::async_error() {
  if (aborted_.load()) return Result::InternalError;
  if (abort_host_ && *abort_host_ != 0) return Result::InternalError;
  if (progress_host_ && progress_host_[2] != 0) return Result::InternalError;
  if (watchdog_ && watchdog_->tripped()) return Result::InternalError;
  if (progress_host_ && progress_host_[0] != progress_host_[1]) return Result::InProgress;
  return Result::Success;
}

Algo Comm::query_algo(size_t bytes, DType t, RedOp op, bool registered) {
  if (!gpu_plane_) return Algo::Ring;
  PlanInput pi;
  pi.count = bytes / dtype_size(t);
  pi.in = pi.wire = pi.out = t;
  pi.op = op;
  pi.in_symmetric = pi.out_symmetric = registered;
  pi.in_has_mc = pi.out_has_mc = registered && caps_.nvls;
  pi.auto_eligible = !registered && auto_shm_ != nullptr && cfg_.auto_map;   // as for ordinary device buffers
  pi.forced = parse_algo(cfg_.algo);
  if (pi.forced == Algo::Ring) pi.forced = Algo::Auto;
  Plan p = make_plan(pi, caps_, cfg_);
  return p.valid ? p.spec.algo : Algo::Auto;
}

std::string Comm::stats_json() {
  std::ostringstream o;
  o << "{\"rank\":" << rank_ << ",\"size\":" << size_ << ",\"plane\":\"" << (gpu_plane_ ? "nvlink" : (shared_plane_ ? "shared-gpu" : (transport_ ? transport_->name() : "none")))
    << "\",\"device\":" << device_ << ",\"symmetric_provider\":\"" << (symm_ ? symm_->provider() : "none") << "\",\"nvls\":"
    << (caps_.nvls ? "true" : "false") << ",\"calls\":" << stats_.calls << ",\"bytes\":" << stats_.bytes << ",\"algo\":{";
  const Algo algos[] = {Algo::LL, Algo::OneShot, Algo::TwoShot, Algo::Nvls, Algo::Ring, Algo::Local, Algo::Pipe, Algo::HostSync};
  bool first = true;
  for (Algo a : algos) {
    if (!first) o << ",";
    first = false;
    o << "\"" << algo_name(a) << "\":" << stats_.by_algo[static_cast<int>(a)];
  }
  o << "},\"zero_copy_in\":" << stats_.zero_copy_in << ",\"zero_copy_out\":" << stats_.zero_copy_out
    << ",\"ipc_cache\":{\"hits\":" << ipc_hits_ << ",\"misses\":" << ipc_misses_ << ",\"open\":" << ipc_cache_.size() << "}"
    << ",\"stale_registrations\":" << stats_.stale_registrations << ",\"staged_calls\":" << stats_.staged_passes << ",\"pipelined_calls\":" << stats_.pipelined
    << ",\"auto_map\":{\"exports\":" << stats_.auto_exports << ",\"imports\":" << stats_.auto_imports << ",\"direct_calls\":"
    << (auto_shm_ && progress_host_ ? progress_host_[6] : 0u) << "}" << ",\"graph_captures_seen\":" << stats_.graph_captures_seen;
  if (watchdog_) {
    o << ",\"watchdog\":{\"polls\":" << watchdog_->stats().polls.load() << ",\"trips\":" << watchdog_->stats().trips.load()
      << ",\"device_failures\":" << watchdog_->stats().device_failures.load() << ",\"remote_aborts\":"
      << watchdog_->stats().remote_aborts.load() << "}";
  }
  if (progress_host_) o << ",\"progress\":{\"started\":" << progress_host_[0] << ",\"done\":" << progress_host_[1] << ",\"status\":" << progress_host_[2] << "}";
  if (transport_) {
    TransportStats& t = transport_->stats();
    o << ",\"transport\":{\"writes\":" << t.writes.load() << ",\"flag_writes\":" << t.flag_writes.load() << ",\"bytes\":"
      << t.bytes_written.load() << ",\"signaled\":" << t.signaled.load() << ",\"direct_writes\":" << t.direct_writes.load() << ",\"direct_flags\":" << t.direct_flags.load() << ",\"reg_hits\":" << t.reg_hits.load()
      << ",\"reg_misses\":" << t.reg_misses.load() << ",\"completion_errors\":" << t.completion_errors.load() << "}";
  }
  if (ring_) {
    const RingStats& r = ring_->stats();
    o << ",\"ring\":{\"calls\":" << r.calls << ",\"slices_sent\":" << r.slices_sent << ",\"credit_stalls\":" << r.credit_stalls
      << ",\"window_stalls\":" << r.window_stalls << ",\"threaded_calls\":" << r.threaded_calls << ",\"slice_bytes\":" << ring_->slice_bytes() << ",\"slots\":" << ring_->slots() << "}";
  }
  o << ",\"aborted\":" << (aborted_.load() ? "true" : "false") << "}";
  return o.str();
}

}  // namespace mnccl
