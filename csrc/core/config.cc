#include "core/config.h"

#include <cerrno>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <strings.h>

#include "core/error.h"
#include "core/log.h"

namespace mnccl {
namespace {

const char* env_getter(const char* name, void*) { return std::getenv(name); }

long long parse_ll(const char* name, const char* s) {
  errno = 0;
  char* end = nullptr;
  long long v = std::strtoll(s, &end, 10);
  while (end && (*end == ' ' || *end == '\t' || *end == '\n')) ++end;
  // Accept K/M/G suffixes (powers of two) as a convenience.
  if (end && *end && !end[1]) {
    if (*end == 'k' || *end == 'K') { v <<= 10; ++end; }
    else if (*end == 'm' || *end == 'M') { v <<= 20; ++end; }
    else if (*end == 'g' || *end == 'G') { v <<= 30; ++end; }
  }
  if (errno != 0 || end == s || (end && *end)) {
    fail(Result::InvalidArgument, std::string("malformed value for ") + name + ": '" + s + "'");
  }
  return v;
}

bool parse_bool(const char* name, const char* s) {
  if (!strcasecmp(s, "1") || !strcasecmp(s, "true") || !strcasecmp(s, "on") || !strcasecmp(s, "yes")) return true;
  if (!strcasecmp(s, "0") || !strcasecmp(s, "false") || !strcasecmp(s, "off") || !strcasecmp(s, "no")) return false;
  fail(Result::InvalidArgument, std::string("malformed boolean for ") + name + ": '" + s + "'");
}

struct Reader {
  Config::Getter get;
  void* ctx;
  const char* raw(const char* n) const {
    const char* v = get(n, ctx);
    return (v && *v) ? v : nullptr;
  }
  template <typename T>
  void num(const char* n, T& out) const {
    if (const char* v = raw(n)) out = static_cast<T>(parse_ll(n, v));
  }
  void boolean(const char* n, bool& out) const {
    if (const char* v = raw(n)) out = parse_bool(n, v);
  }
  void str(const char* n, std::string& out) const {
    if (const char* v = raw(n)) out = v;
  }
};

std::mutex g_mu;
Config* g_cfg = nullptr;
bool g_banner_printed = false;

}  // namespace

Config Config::from_getter(Getter get, void* ctx) {
  Config c;
  Reader r{get, ctx};
  if (const char* v = r.raw("MINI_NCCL_SLICE_SIZE")) {
    long long x = parse_ll("MINI_NCCL_SLICE_SIZE", v);
    if (x < 0) fail(Result::InvalidArgument, "MINI_NCCL_SLICE_SIZE must be >= 0");
    c.slice_size = static_cast<size_t>(x);
  }
  r.num("MINI_NCCL_WINDOW_SIZE", c.window_size);
  r.num("MINI_NCCL_SIGNAL_BATCH", c.signal_batch);
  if (c.slice_size == 0) c.slice_size = 1024;
  if (c.window_size <= 0) c.window_size = 1;
  if (c.signal_batch <= 0) c.signal_batch = 1;
  r.boolean("MINI_NCCL_GDR_ENABLE", c.gdr_enable);
  r.str("MINI_NCCL_NET_DEVICE", c.net_device);

  r.num("MINI_NCCL_BOOTSTRAP_PORT", c.bootstrap_port);
  r.num("MINI_NCCL_HERA_PORT", c.hera_port);
  r.num("MINI_NCCL_WATCHDOG_TIMEOUT_MS", c.watchdog_timeout_ms);
  r.boolean("MINI_NCCL_WATCHDOG", c.watchdog_enable);
  r.num("MINI_NCCL_SOCKET_TIMEOUT_MS", c.socket_timeout_ms);
  r.num("MINI_NCCL_CONNECT_RETRIES", c.connect_retries);
  r.str("MINI_NCCL_TRANSPORT", c.transport);
  r.str("MINI_NCCL_SYMM", c.symm_mode);
  r.boolean("MINI_NCCL_NVLS_ENABLE", c.nvls_enable);
  r.str("MINI_NCCL_ALGO", c.algo);
  r.num("MINI_NCCL_LL_MAX_BYTES", c.ll_max_bytes);
  r.num("MINI_NCCL_ONESHOT_MAX_BYTES", c.oneshot_max_bytes);
  r.num("MINI_NCCL_NVLS_MIN_BYTES", c.nvls_min_bytes);
  r.num("MINI_NCCL_STAGING_BYTES", c.staging_bytes);
  r.num("MINI_NCCL_PIPELINE_MIN_BYTES", c.pipeline_min_bytes);
  r.num("MINI_NCCL_HOST_PIPELINE_MIN_BYTES", c.host_pipeline_min_bytes);
  r.num("MINI_NCCL_HOST_CHUNK_BYTES", c.host_chunk_bytes);
  r.num("MINI_NCCL_PIPE_MIN_BYTES", c.pipe_min_bytes);
  r.num("MINI_NCCL_PIPE_CHUNK_BYTES", c.pipe_chunk_bytes);
  r.num("MINI_NCCL_MAX_BLOCKS", c.max_blocks);
  r.num("MINI_NCCL_UNROLL", c.unroll);
  r.boolean("MINI_NCCL_NUMA_BIND", c.numa_bind);
  r.num("MINI_NCCL_CUDA_DEVICE", c.cuda_device);
  r.boolean("MINI_NCCL_HERA_KEEPALIVE", c.hera_keepalive);
  r.str("MINI_NCCL_JOB_ID", c.job_id);
  r.boolean("MINI_NCCL_BLOCKING", c.blocking);
  r.boolean("MINI_NCCL_PIPELINE_COPY_ENGINE", c.pipeline_copy_engine);
  r.boolean("MINI_NCCL_PIPELINE_TAPER", c.pipeline_taper);
  r.boolean("MINI_NCCL_AUTO_MAP", c.auto_map);
  r.boolean("MINI_NCCL_RING_SENDER_THREAD", c.ring_sender_thread);
  r.boolean("MINI_NCCL_AUTO_DEVICE", c.auto_device);
  r.str("MINI_NCCL_TUNING_FILE", c.tuning_file);

  if (c.bootstrap_port <= 0 || c.bootstrap_port > 65535) fail(Result::InvalidArgument, "MINI_NCCL_BOOTSTRAP_PORT out of range");
  if (c.hera_port <= 0 || c.hera_port > 65535) fail(Result::InvalidArgument, "MINI_NCCL_HERA_PORT out of range");
  if (c.watchdog_timeout_ms <= 0) c.watchdog_timeout_ms = 1;
  if (c.socket_timeout_ms <= 0) c.socket_timeout_ms = 1;
  if (c.connect_retries <= 0) c.connect_retries = 1;
  if (c.host_chunk_bytes < (64u << 10)) c.host_chunk_bytes = 64u << 10;
  if (c.staging_bytes < (1u << 20)) c.staging_bytes = 1u << 20;
  c.staging_bytes = (c.staging_bytes + 4095) & ~size_t(4095);
  return c;
}

bool Config::set_knob(const std::string& name, long long v) {
  if (v < 0) return false;
  struct SizeKnob { const char* name; size_t Config::*field; };
  struct IntKnob { const char* name; int Config::*field; int lo, hi; };
  static const SizeKnob sizes[] = {
      {"LL_MAX_BYTES", &Config::ll_max_bytes}, {"ONESHOT_MAX_BYTES", &Config::oneshot_max_bytes},
      {"NVLS_MIN_BYTES", &Config::nvls_min_bytes}, {"PIPELINE_MIN_BYTES", &Config::pipeline_min_bytes},
      {"PIPE_MIN_BYTES", &Config::pipe_min_bytes}, {"PIPE_CHUNK_BYTES", &Config::pipe_chunk_bytes},
      {"HOST_PIPELINE_MIN_BYTES", &Config::host_pipeline_min_bytes}, {"HOST_CHUNK_BYTES", &Config::host_chunk_bytes},
  };
  static const IntKnob ints[] = {
      {"MAX_BLOCKS", &Config::max_blocks, 0, 512}, {"UNROLL", &Config::unroll, 0, 8},
  };
  for (const auto& k : sizes)
    if (name == k.name) {
      if (name == "HOST_CHUNK_BYTES" && v < (64 << 10)) return false;
      this->*(k.field) = static_cast<size_t>(v);
      return true;
    }
  for (const auto& k : ints)
    if (name == k.name) {
      if (v < k.lo || v > k.hi || (name == "UNROLL" && v != 0 && v != 4 && v != 8)) return false;
      this->*(k.field) = static_cast<int>(v);
      return true;
    }
  return false;
}

int Config::apply_tuning_text(const std::string& text, int nranks, std::string* errors) {
  int applied = 0, lineno = 0;
  size_t pos = 0;
  while (pos <= text.size()) {
    size_t nl = text.find('\n', pos);
    if (nl == std::string::npos) nl = text.size();
    std::string line = text.substr(pos, nl - pos);
    pos = nl + 1;
    ++lineno;
    const size_t hash = line.find('#');
    if (hash != std::string::npos) line.erase(hash);
    char knob[64];
    long long n = 0, v = 0;
    char extra = 0;
    const int got = sscanf(line.c_str(), " %lld %63s %lld %c", &n, knob, &v, &extra);
    if (line.find_first_not_of(" \t\r") == std::string::npos) continue;  // blank
    if (got != 3) {
      if (errors) *errors += "line " + std::to_string(lineno) + ": expected '<nranks> <KNOB> <value>'; ";
      continue;
    }
    if (n != 0 && n != nranks) continue;
    std::string name = knob;
    if (name.rfind("MINI_NCCL_", 0) == 0) name.erase(0, 10);
    if (set_knob(name, v)) ++applied;
    else if (errors) *errors += "line " + std::to_string(lineno) + ": unknown knob or bad value '" + name + "'; ";
  }
  return applied;
}

// Environment variables win over the tuning table: applied again after it.
static void reapply_env_knobs(Config& c) {
  static const char* const names[] = {"LL_MAX_BYTES", "ONESHOT_MAX_BYTES", "NVLS_MIN_BYTES", "PIPELINE_MIN_BYTES",
                                      "PIPE_MIN_BYTES", "PIPE_CHUNK_BYTES", "HOST_PIPELINE_MIN_BYTES", "HOST_CHUNK_BYTES",
                                      "MAX_BLOCKS", "UNROLL"};
  for (const char* n : names) {
    const std::string var = std::string("MINI_NCCL_") + n;
    if (const char* v = getenv(var.c_str())) {
      char* end = nullptr;
      const long long x = strtoll(v, &end, 10);
      if (end != v) c.set_knob(n, x);
    }
  }
}

int Config::apply_tuning_file(const std::string& path, int nranks, std::string* errors) {
  FILE* f = fopen(path.c_str(), "r");
  if (!f) {
    if (errors) *errors += "cannot open " + path + "; ";
    return 0;
  }
  std::string text;
  char buf[4096];
  size_t n;
  while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
  fclose(f);
  const int applied = apply_tuning_text(text, nranks, errors);
  reapply_env_knobs(*this);
  return applied;
}

Config Config::from_env() { return from_getter(env_getter, nullptr); }

const Config& Config::get() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_cfg) g_cfg = new Config(from_env());
  if (!g_banner_printed) {
    g_banner_printed = true;
    log_always("Config", "%s", g_cfg->banner().c_str());
  }
  return *g_cfg;
}

const Config& Config::reload() {
  std::lock_guard<std::mutex> lk(g_mu);
  Config fresh = from_env();
  if (!g_cfg) g_cfg = new Config(fresh);
  else *g_cfg = fresh;
  return *g_cfg;
}

std::string Config::banner() const {
  char buf[160];
  snprintf(buf, sizeof(buf), "Loaded: SLICE_SIZE=%zu B, WINDOW=%d, BATCH=%d", slice_size,
           window_size, signal_batch);
  return buf;
}

}  // namespace mnccl
