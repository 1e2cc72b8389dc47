// Environment knobs.  The three reference knobs keep their names, defaults and
// clamps (reference: include/Config.h:29-51): MINI_NCCL_SLICE_SIZE (bytes,
// default 131072, 0 -> 1024), MINI_NCCL_WINDOW_SIZE (default 64, <=0 -> 1),
// MINI_NCCL_SIGNAL_BATCH (default 16).  Unlike the reference, SIGNAL_BATCH is
// validated (<=0 -> 1; the reference would compute `s % 0`) and malformed
// numbers raise InvalidArgument instead of an uncaught std::invalid_argument.
// The banner "[Config] Loaded: SLICE_SIZE=... B, WINDOW=..., BATCH=..." is
// printed once per process.
// Two switches of the GEMM kernels are read where they are used (csrc/kernels):
// MINI_NCCL_GEMM_PAIR = -1|0|1 (automatic / single-CTA tiles / CTA pairs) and
// MINI_NCCL_RS_TILED = 0|1 (staging layout of GEMM -> reduce-scatter).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace mnccl {

struct Config {
  // --- reference knobs ---
  size_t slice_size = 128 * 1024;
  int window_size = 64;
  int signal_batch = 16;
  bool gdr_enable = false;  // reserved in the reference; MINI_NCCL_GDR_ENABLE here
  std::string net_device;   // MINI_NCCL_NET_DEVICE (exact NIC name override)

  // --- new knobs ---
  int bootstrap_port = 8888;          // MINI_NCCL_BOOTSTRAP_PORT (reference: fixed 8888)
  int hera_port = 9999;               // MINI_NCCL_HERA_PORT      (reference: fixed 9999)
  int watchdog_timeout_ms = 10000;    // MINI_NCCL_WATCHDOG_TIMEOUT_MS (reference: fixed 10 s)
  bool watchdog_enable = true;        // MINI_NCCL_WATCHDOG
  int socket_timeout_ms = 30000;      // MINI_NCCL_SOCKET_TIMEOUT_MS (reference: unbounded)
  int connect_retries = 20;           // MINI_NCCL_CONNECT_RETRIES (reference: 20 x 1 s)
  std::string transport = "auto";     // MINI_NCCL_TRANSPORT = auto|nvlink|soft|verbs
  std::string symm_mode = "auto";     // MINI_NCCL_SYMM = auto|vmm|ipc
  bool nvls_enable = true;            // MINI_NCCL_NVLS_ENABLE
  std::string algo = "auto";          // MINI_NCCL_ALGO = auto|ll|oneshot|twoshot|nvls|ring
  size_t ll_max_bytes = 0;            // MINI_NCCL_LL_MAX_BYTES      (0 = built-in table)
  size_t oneshot_max_bytes = 0;       // MINI_NCCL_ONESHOT_MAX_BYTES (0 = built-in table)
  size_t nvls_min_bytes = 0;          // MINI_NCCL_NVLS_MIN_BYTES    (0 = built-in table)
  size_t staging_bytes = 256u << 20;  // MINI_NCCL_STAGING_BYTES (per direction, per rank)
  size_t host_pipeline_min_bytes = 4u << 20;  // MINI_NCCL_HOST_PIPELINE_MIN_BYTES: pinned-host buffers of at least this size are moved by the copy engines in chunks that overlap the collective (0 = never)
  size_t host_chunk_bytes = 8u << 20;  // MINI_NCCL_HOST_CHUNK_BYTES: chunk of that pipeline
  bool auto_map = true;         // MINI_NCCL_AUTO_MAP: ordinary device buffers of the peer-to-peer two-shot AllReduce are exported over CUDA IPC when first seen and used directly once every rank has mapped them
  bool ring_sender_thread = true;  // MINI_NCCL_RING_SENDER_THREAD: the host ring sends from a second thread while the caller's thread receives and reduces (messages of 4 MB and more, providers that allow it)
  bool pipeline_taper = false;  // MINI_NCCL_PIPELINE_TAPER: small first and last chunk, large chunks between (device buffers of 128 MB and more)
  bool pipeline_copy_engine = false;  // MINI_NCCL_PIPELINE_COPY_ENGINE: the chunk pipeline moves ordinary DEVICE buffers with the copy engines too (off: copy kernels)
  size_t pipeline_min_bytes = 48u << 20;  // MINI_NCCL_PIPELINE_MIN_BYTES: ordinary buffers of at least this size go through the chunk pipeline (0 = never)
  size_t pipe_min_bytes = 24u << 20;  // MINI_NCCL_PIPE_MIN_BYTES: ordinary DEVICE buffers of at least this size take the pipelined kernel (copy-in, reduce, copy-out blocks in one launch); 0 = never (then MINI_NCCL_PIPELINE_MIN_BYTES decides on the stream pipeline)
  size_t pipe_chunk_bytes = 0;        // MINI_NCCL_PIPE_CHUNK_BYTES: chunk of that kernel (0 = 512 KB)
  int max_blocks = 0;                 // MINI_NCCL_MAX_BLOCKS (0 = built-in)
  int unroll = 0;                     // MINI_NCCL_UNROLL (NVLS vectors in flight per thread: 4 or 8; 0 = built-in)
  bool numa_bind = true;              // MINI_NCCL_NUMA_BIND (verbs path only, calling thread)
  int cuda_device = -1;               // MINI_NCCL_CUDA_DEVICE (-1 = current device)
  bool hera_keepalive = false;        // MINI_NCCL_HERA_KEEPALIVE (heartbeat + global abort)
  std::string job_id;                 // MINI_NCCL_JOB_ID (namespace for shm / unix sockets)
  bool blocking = false;              // MINI_NCCL_BLOCKING: AllReduce returns only when the stream work is done (reference behaviour)
  bool auto_device = true;            // MINI_NCCL_AUTO_DEVICE: in Hera mode pick GPU = local rank when ranks share a device

  // Parse from the process environment.  Throws Error(InvalidArgument) on
  // malformed numbers.  Does not print.
  static Config from_env();
  // Parse from an explicit lookup function (unit tests).
  using Getter = const char* (*)(const char* name, void* ctx);
  static Config from_getter(Getter get, void* ctx);

  // Process-wide instance: parsed on first use, banner printed once.
  static const Config& get();
  // Re-read the environment (tests); prints no banner.
  static const Config& reload();

  // Sets one numeric tuning knob by the name of its environment variable without the MINI_NCCL_
  // or a value out of range.  Only launch-tuning knobs can be set this way (not ports or timeouts).
  bool set_knob(const std::string& name, long long value);
  // Applies a tuning table (MINI_NCCL_TUNING_FILE; written by benchmarks/tune.py) for `nranks`:
  // text lines "<nranks> <KNOB> <value>", '#' starts a comment, nranks 0 matches every size.
  // Returns the number of knobs applied; malformed lines and unknown knobs are reported in *errors.
  int apply_tuning_text(const std::string& text, int nranks, std::string* errors = nullptr);
  int apply_tuning_file(const std::string& path, int nranks, std::string* errors = nullptr);
  std::string tuning_file;            // MINI_NCCL_TUNING_FILE

  std::string banner() const;
};

}  // namespace mnccl
