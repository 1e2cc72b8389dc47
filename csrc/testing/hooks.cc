// C entry points that expose internal components to the Python test-suite
// (ctypes).  They are thin: each one drives a component the way its users do
// and reports what happened.  Built into libmini_nccl_testhooks.so only: the
// product library exports the API and the host oracle, nothing of this file.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <sstream>
#include <unistd.h>
#include <string>
#include <thread>
#include <vector>

#include "algo/select.h"
#include "bootstrap/fdpass.h"
#include "bootstrap/hera.h"
#include "bootstrap/store.h"
#include "comm.h"
#include "core/config.h"
#include "core/error.h"
#include "core/log.h"
#include "net/nic_select.h"
#include "net/reg_cache.h"
#include "net/request_pool.h"
#include "net/ring.h"
#include "net/soft_transport.h"
#include "net/spsc_queue.h"
#include "ref/oracle.h"
#include "watchdog/watchdog.h"

namespace mnccl {
int noalloc_dirty_control(int byte);  // csrc/kernels/noalloc.cu
}

using namespace mnccl;

namespace {
template <typename Fn>
int guarded(Fn&& fn) {
  try {
    return fn();
  } catch (const Error& e) {
    return 100 + static_cast<int>(e.code());
  } catch (const std::exception&) {
    return 99;
  }
}
void copy_out(const std::string& s, char* out, size_t len) {
  if (!out || !len) return;
  size_t n = s.size() < len - 1 ? s.size() : len - 1;
  memcpy(out, s.data(), n);
  out[n] = 0;
}
}  // namespace

extern "C" {
#define MNCCL_EXPORT __attribute__((visibility("default")))

// ---- config ---------------------------------------------------------------
// env: "NAME=value;NAME=value".  out: JSON of the parsed knobs.
MNCCL_EXPORT int mnccl_test_config(const char* env, char* out, size_t len) {
  return guarded([&] {
    std::map<std::string, std::string> kv;
    std::stringstream ss(env ? env : "");
    std::string item;
    while (std::getline(ss, item, ';')) {
      size_t eq = item.find('=');
      if (eq != std::string::npos) kv[item.substr(0, eq)] = item.substr(eq + 1);
    }
    Config c = Config::from_getter(
        [](const char* name, void* ctx) -> const char* {
          auto* m = static_cast<std::map<std::string, std::string>*>(ctx);
          auto it = m->find(name);
          return it == m->end() ? nullptr : it->second.c_str();
        },
        &kv);
    std::ostringstream o;
    o << "{\"slice_size\":" << c.slice_size << ",\"window_size\":" << c.window_size << ",\"signal_batch\":" << c.signal_batch
      << ",\"net_device\":\"" << c.net_device << "\",\"watchdog_timeout_ms\":" << c.watchdog_timeout_ms
      << ",\"bootstrap_port\":" << c.bootstrap_port << ",\"hera_port\":" << c.hera_port << ",\"staging_bytes\":" << c.staging_bytes
      << ",\"pipeline_min_bytes\":" << c.pipeline_min_bytes << ",\"host_pipeline_min_bytes\":" << c.host_pipeline_min_bytes
      << ",\"host_chunk_bytes\":" << c.host_chunk_bytes
      << ",\"algo\":\"" << c.algo << "\",\"nvls_enable\":" << (c.nvls_enable ? "true" : "false") << ",\"banner\":\"" << c.banner() << "\"}";
    copy_out(o.str(), out, len);
    return 0;
  });
}

// Applies a tuning table given as text for `nranks`; out: JSON of the tunable knobs and the loader's complaints.
MNCCL_EXPORT int mnccl_test_tuning_text(const char* text, int nranks, char* out, size_t len) {
  return guarded([&] {
    Config c;
    std::string errors;
    const int applied = c.apply_tuning_text(text ? text : "", nranks, &errors);
    for (char& ch : errors)
      if (ch == '"' || ch == '\\') ch = '\'';
    std::ostringstream o;
    o << "{\"applied\":" << applied << ",\"ll_max_bytes\":" << c.ll_max_bytes << ",\"oneshot_max_bytes\":" << c.oneshot_max_bytes
      << ",\"nvls_min_bytes\":" << c.nvls_min_bytes << ",\"pipe_min_bytes\":" << c.pipe_min_bytes << ",\"pipe_chunk_bytes\":"
      << c.pipe_chunk_bytes << ",\"max_blocks\":" << c.max_blocks
      << ",\"errors\":\"" << errors << "\"}";
    copy_out(o.str(), out, len);
    return 0;
  });
}

// Dirties the control words of the allocation-free entry point's static scratch (of THIS library's copy).
#ifndef MNCCL_HOST_ONLY_SELFTEST  // the sanitizer self-test links no CUDA code
MNCCL_EXPORT int mnccl_test_noalloc_dirty(int byte) { return noalloc_dirty_control(byte); }
#endif

// ---- chunk schedule of the pipeline -------------------------------------------
// Writes up to `max` chunk sizes (elements) to `out`; returns the number of chunks or a negative code.
MNCCL_EXPORT int mnccl_test_pipeline_chunks(size_t count, size_t elem_bytes, size_t uniform_elems, size_t cap_elems, int taper,
                                            size_t* out, int max) {
  int n = -1;
  int rc = guarded([&] {
    std::vector<size_t> c = pipeline_chunks(count, elem_bytes, uniform_elems, cap_elems, taper != 0);
    n = static_cast<int>(c.size());
    for (int i = 0; i < n && i < max; ++i) out[i] = c[i];
    return 0;
  });
  return rc == 0 ? n : -rc;
}

// ---- soft provider: key and range checks ------------------------------------------
// Two ranks as threads.  Rank 0 posts a write with a wrong key, a write that runs past the region,
// then a good write and a flag; rank 1 must end up with exactly the good payload and the two bad
// writes must be counted as remote access errors (by the receiver over sockets, by the poster on
// the cross-memory-attach path, where a signalled request also completes with an error status).
// Returns 0 when all of that holds, otherwise a code that names the first failed check.
MNCCL_EXPORT int mnccl_test_soft_reject(int port, int cma) {
  const char* old_env = getenv("MINI_NCCL_SOFT_CMA");
  const std::string saved = old_env ? old_env : "";
  const bool had = old_env != nullptr;
  setenv("MINI_NCCL_SOFT_CMA", cma ? "1" : "0", 1);
  std::atomic<int> verdict{0};
  std::atomic<uint64_t> errors_seen{0};
  std::atomic<int> used_cma{0};
  auto set = [&](int code) { int zero = 0; verdict.compare_exchange_strong(zero, code); };
  std::vector<std::thread> th;
  for (int r = 0; r < 2; ++r) {
    th.emplace_back([&, r] {
      try {
        BootstrapStore store(r, 2, "127.0.0.1", port, 10000, 50);
        store.connect();
        SoftTransport t(r, 2);
        t.connect(store);
        std::vector<uint32_t> region(1024, 0xAAAAAAAAu);   // 4 KB target on rank 1, source on rank 0
        auto mr = t.register_memory(region.data(), region.size() * 4);
        RemoteBuffer mine;
        mine.addr = reinterpret_cast<uint64_t>(region.data());
        mine.rkey = mr->rkey;
        RemoteBuffer all[2], flags[2];
        store.all_gather(&mine, all, sizeof(mine));
        RemoteBuffer myflags = t.flags_remote();
        store.all_gather(&myflags, flags, sizeof(myflags));
        if (r == 0) {
          for (auto& w : region) w = 0x12345678u;
          if (t.cma_enabled(1)) used_cma.store(1);
          RemoteBuffer bad = all[1];
          bad.rkey ^= 0x5a5a;
          Request* a = t.write(1, region.data(), *mr, bad, 0, 256, true);            // wrong key
          Request* b = t.write(1, region.data(), *mr, all[1], 4096 - 128, 256, true);  // runs past the end
          Request* c = t.write(1, region.data(), *mr, all[1], 1024, 512, true);        // fine: words 256..383
          if (!a || !b || !c) set(1);
          if (t.cma_enabled(1) && a && b && (a->status() == 0 || b->status() == 0)) set(2);
          if (c && c->status() != 0) set(3);
          for (Request* q : {a, b, c}) if (q) t.release(q);
          t.write_flag(1, flags[1], 5, 1, false);
        } else {
          auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(5);
          while (__atomic_load_n(t.flags() + 5, __ATOMIC_ACQUIRE) < 1) {
            if (std::chrono::steady_clock::now() > deadline) { set(4); break; }
            std::this_thread::yield();
          }
          for (size_t i = 0; i < region.size(); ++i) {
            const uint32_t want = (i >= 256 && i < 384) ? 0x12345678u : 0xAAAAAAAAu;
            if (region[i] != want) { set(5); break; }
          }
        }
        store.barrier();
        errors_seen += t.remote_access_errors();
        store.barrier();
        mr.reset();
      } catch (const std::exception& e) {
        fprintf(stderr, "soft reject rank %d: %s\n", r, e.what());
        set(6);
      }
    });
  }
  for (auto& t : th) t.join();
  if (had) setenv("MINI_NCCL_SOFT_CMA", saved.c_str(), 1);
  else unsetenv("MINI_NCCL_SOFT_CMA");
  if (verdict.load() == 0 && errors_seen.load() != 2) return 7;
  if (verdict.load() == 0 && cma && !used_cma.load()) return -1;  // fast path not permitted here: nothing was tested
  return verdict.load();
}

// ---- SPSC queue -----------------------------------------------------------
// One producer thread, one consumer thread, n items; checks order and loss.
MNCCL_EXPORT int mnccl_test_spsc(int capacity, int n_items) {
  SpscQueue<int> q(static_cast<size_t>(capacity));
  if (!q.empty()) return 1;
  // full / empty behaviour, single-threaded
  int filled = 0;
  while (q.push(filled)) ++filled;
  if (filled < capacity) return 2;
  int v = -1;
  for (int i = 0; i < filled; ++i) {
    if (!q.pop(&v) || v != i) return 3;
  }
  if (q.pop(&v)) return 4;
  std::atomic<int> bad{0};
  std::thread prod([&] {
    for (int i = 0; i < n_items; ++i)
      while (!q.push(i)) std::this_thread::yield();
  });
  std::thread cons([&] {
    int x;
    for (int i = 0; i < n_items; ++i) {
      while (!q.pop(&x)) std::this_thread::yield();
      if (x != i) bad++;
    }
  });
  prod.join();
  cons.join();
  return bad.load() ? 5 : 0;
}

// ---- request pool ---------------------------------------------------------
MNCCL_EXPORT int mnccl_test_request_pool(int n) {
  RequestPool pool(static_cast<size_t>(n));
  std::vector<Request*> held;
  for (int i = 0; i < n; ++i) {
    Request* r = pool.acquire(static_cast<uint64_t>(i));
    if (!r || r->wr_id() != static_cast<uint64_t>(i) || r->completed()) return 1;
    held.push_back(r);
  }
  if (pool.acquire(0) != nullptr) return 2;  // exhaustion is reported, not hidden
  held[0]->complete(7);
  if (!held[0]->completed() || held[0]->status() != 7) return 3;
  pool.release(held[0]);
  Request* again = pool.acquire(42);
  if (!again || again->completed() || again->status() != 0 || again->wr_id() != 42) return 4;
  pool.release(again);
  for (size_t i = 1; i < held.size(); ++i) pool.release(held[i]);
  return pool.available() == static_cast<size_t>(n) ? 0 : 5;
}

// ---- registration cache ---------------------------------------------------
MNCCL_EXPORT int mnccl_test_reg_cache() {
  struct H { int id; };
  int made = 0;
  RegistrationCache<H> cache(3);
  auto make = [&](void*, size_t) { auto h = std::make_shared<H>(); h->id = ++made; return h; };
  char* base = reinterpret_cast<char*>(0x100000);
  auto a = cache.get(base, 4096, make);
  if (made != 1) return 1;
  if (cache.get(base, 1024, make)->id != a->id || made != 1) return 2;           // smaller request hits
  if (cache.get(base + 512, 1024, make)->id != a->id || made != 1) return 3;     // interior pointer hits
  if (cache.get(base, 8192, make)->id == a->id || made != 2) return 4;           // larger request re-registers
  cache.get(base + 0x10000, 64, make);
  cache.get(base + 0x20000, 64, make);
  if (cache.size() != 3) return 5;
  cache.get(base, 64, make);                 // touch: base is most recently used
  cache.get(base + 0x30000, 64, make);       // evicts the least recently used (0x10000)
  if (cache.size() != 3 || cache.evictions() != 1) return 6;
  int before = made;
  cache.get(base + 0x10000, 64, make);
  if (made != before + 1) return 7;          // it was evicted, so this is a miss
  if (cache.invalidate(base, 0) != 1) return 8;
  before = made;
  cache.get(base, 64, make);
  if (made != before + 1) return 9;          // invalidated entries miss
  if (cache.hits() < 3 || cache.misses() < 5) return 10;
  return 0;
}

// ---- NIC / NUMA -----------------------------------------------------------
MNCCL_EXPORT int mnccl_test_select_nic(const char* csv, const char* override_name, int* index) {
  return guarded([&] {
    std::vector<std::string> names;
    std::stringstream ss(csv ? csv : "");
    std::string n;
    while (std::getline(ss, n, ',')) if (!n.empty()) names.push_back(n);
    *index = select_nic(names, override_name ? override_name : "");
    return 0;
  });
}
MNCCL_EXPORT int mnccl_test_parse_cpu_list(const char* list, int* out, int max) {
  std::vector<int> c = parse_cpu_list(list ? list : "");
  for (int i = 0; i < static_cast<int>(c.size()) && i < max; ++i) out[i] = c[i];
  return static_cast<int>(c.size());
}
MNCCL_EXPORT int mnccl_test_numa(const char* sysfs_root, const char* device, int* node, int* ncpus) {
  *node = read_nic_numa_node(sysfs_root, device);
  *ncpus = static_cast<int>(read_numa_cpus(sysfs_root, *node).size());
  return 0;
}

// ---- planner --------------------------------------------------------------
MNCCL_EXPORT int mnccl_test_plan(int nranks, int mode, uint64_t count, int in_t, int wire_t, int out_t, int op, int in_sym,
                                 int out_sym, int nvls, int forced, uint64_t stage_bytes, int* algo, int* nblocks,
                                 uint64_t* shard_elems, uint64_t* chunk_vecs, int* copy_in, int* copy_out) {
  Config cfg;  // defaults, independent of the environment
  CommCaps caps;
  caps.nranks = nranks;
  caps.nvls = nvls != 0;
  caps.ll_slot_bytes = default_ll_slot_bytes(nranks, cfg);
  caps.inbox_slot_bytes = default_inbox_slot_bytes(nranks, cfg);
  caps.stage_bytes = stage_bytes ? stage_bytes : cfg.staging_bytes;
  PlanInput pi;
  pi.mode = static_cast<Mode>(mode);
  pi.count = count;
  pi.in = static_cast<DType>(in_t);
  pi.wire = static_cast<DType>(wire_t);
  pi.out = static_cast<DType>(out_t);
  pi.op = static_cast<RedOp>(op);
  pi.in_symmetric = (in_sym & 1) != 0;
  pi.out_symmetric = (out_sym & 1) != 0;
  pi.auto_eligible = (in_sym & 2) != 0;   // bit 1 of in_sym: ordinary device buffers with lazy direct access on
  pi.in_has_mc = pi.in_symmetric && nvls;
  pi.out_has_mc = pi.out_symmetric && nvls;
  pi.forced = static_cast<Algo>(forced);
  Plan p = make_plan(pi, caps, cfg);
  if (!p.valid) return 1;
  *algo = static_cast<int>(p.spec.algo);
  *nblocks = p.spec.nblocks;
  *shard_elems = p.shard_elems;
  *chunk_vecs = p.chunk_shard_vecs;
  *copy_in = p.copy_in;
  *copy_out = p.copy_out;
  return 0;
}

// ---- watchdog -------------------------------------------------------------
// Scenario 0: a collective that finishes in time; 1: one that never finishes;
// 2: a kernel-reported failure.  Returns the abort word at the end (expected
// 0, 1, 1) or a negative number on a logic error.
MNCCL_EXPORT int mnccl_test_watchdog(int scenario, int timeout_ms) {
  alignas(64) uint32_t words[32] = {0};
  volatile uint32_t* abort_word = words;
  volatile uint32_t* progress = words + 16;
  Watchdog wd(progress, abort_word, timeout_ms, 0);
  int trips = 0;
  wd.set_on_trip([&](uint32_t) { ++trips; });
  auto t0 = std::chrono::steady_clock::now();
  auto at = [&](int ms) { return t0 + std::chrono::milliseconds(ms); };
  wd.step(at(0));
  progress[0] = 1;  // a collective started
  wd.step(at(1));
  if (scenario == 0) {
    wd.step(at(timeout_ms / 2));
    progress[1] = 1;  // ... and finished
    wd.step(at(timeout_ms * 3));
    progress[0] = 2;
    wd.step(at(timeout_ms * 3 + 1));
    progress[1] = 2;
    wd.step(at(timeout_ms * 10));
    if (wd.tripped() || trips) return -1;
  } else if (scenario == 1) {
    wd.step(at(timeout_ms / 2));
    if (wd.tripped()) return -2;  // too early
    wd.step(at(timeout_ms + 5));
    if (!wd.tripped() || trips != 1) return -3;
    wd.step(at(timeout_ms * 4));
    if (trips != 1) return -4;  // trips once
  } else {
    progress[3] = 0x10002;
    progress[2] = 1;
    wd.step(at(2));
    if (!wd.tripped() || trips != 1) return -5;
  }
  return static_cast<int>(*abort_word);
}

// ---- Hera -----------------------------------------------------------------
MNCCL_EXPORT void* mnccl_hera_master_start(int world_size, int port, int heartbeat_timeout_ms) {
  try {
    auto* m = new hera::Master(world_size, port);
    m->set_heartbeat_timeout_ms(heartbeat_timeout_ms);
    m->start_background();
    return m;
  } catch (const std::exception& e) {
    log_always("Hera-Master", "start failed: %s", e.what());
    return nullptr;
  }
}
MNCCL_EXPORT int mnccl_hera_master_port(void* m) { return static_cast<hera::Master*>(m)->port(); }
MNCCL_EXPORT int mnccl_hera_master_registered(void* m) { return static_cast<int>(static_cast<hera::Master*>(m)->workers().size()); }
MNCCL_EXPORT int mnccl_hera_master_abort_sent(void* m) { return static_cast<hera::Master*>(m)->abort_broadcast() ? 1 : 0; }
MNCCL_EXPORT int mnccl_hera_master_worker(void* m, int idx, int* rank, int* pid, char* host, char* ip, int* alive) {
  auto ws = static_cast<hera::Master*>(m)->workers();
  if (idx < 0 || idx >= static_cast<int>(ws.size())) return 1;
  *rank = ws[idx].rank;
  *pid = ws[idx].pid;
  copy_out(ws[idx].hostname, host, 64);
  copy_out(ws[idx].ip, ip, 64);
  *alive = ws[idx].alive ? 1 : 0;
  return 0;
}
MNCCL_EXPORT void mnccl_hera_master_stop(void* m) {
  auto* mm = static_cast<hera::Master*>(m);
  mm->stop();
  delete mm;
}

MNCCL_EXPORT void* mnccl_hera_worker_register(const char* ip, int port, int* rank, int* size, char* root_ip) {
  try {
    auto* w = new hera::Worker(ip, port);
    w->connect_and_register(20, 100, 5000);
    *rank = w->rank();
    *size = w->size();
    copy_out(w->root_ip(), root_ip, 64);
    return w;
  } catch (const std::exception& e) {
    log_always("Hera-Worker", "register failed: %s", e.what());
    return nullptr;
  }
}
MNCCL_EXPORT int mnccl_hera_worker_topology(void* w, int* prev, int* next, char* next_ip) {
  return guarded([&] {
    hera::TopologyInfo t = static_cast<hera::Worker*>(w)->query_topology(3000);
    *prev = t.prev_rank;
    *next = t.next_rank;
    copy_out(t.next_ip, next_ip, 64);
    return 0;
  });
}
static std::atomic<int> g_abort_seen[64];
MNCCL_EXPORT int mnccl_hera_worker_start_agent(void* w, int period_ms, int slot) {
  if (slot < 0 || slot >= 64) return 1;
  g_abort_seen[slot].store(0);
  static_cast<hera::Worker*>(w)->start_agent(period_ms, [slot](int origin, uint32_t reason) {
    g_abort_seen[slot].store(1000 + (origin + 1) * 10 + static_cast<int>(reason));
  });
  return 0;
}
MNCCL_EXPORT int mnccl_hera_worker_abort_seen(int slot) { return g_abort_seen[slot].load(); }
MNCCL_EXPORT int mnccl_hera_worker_send_abort(void* w, unsigned reason) {
  return guarded([&] { static_cast<hera::Worker*>(w)->send_global_abort(reason); return 0; });
}
MNCCL_EXPORT void mnccl_hera_worker_set_state(void* w, unsigned s) { static_cast<hera::Worker*>(w)->set_local_state(s); }
MNCCL_EXPORT void mnccl_hera_worker_free(void* w) { delete static_cast<hera::Worker*>(w); }

// ---- fd passing -----------------------------------------------------------
// Two channels in one process pass a pipe's write end; the receiver writes
// through it and the sender reads the byte back.
MNCCL_EXPORT int mnccl_test_fdpass(const char* ns) {
  return guarded([&] {
    FdChannel a(ns, 0), b(ns, 1);
    a.open();
    b.open();
    int p[2];
    if (pipe(p) != 0) return 1;
    a.send_fd(1, p[1], 77, 2000);
    int src = -1;
    uint32_t tag = 0;
    int got = b.recv_fd(&src, &tag, 2000);
    if (src != 0 || tag != 77) return 2;
    char c = 'x';
    if (write(got, &c, 1) != 1) return 3;
    char d = 0;
    if (read(p[0], &d, 1) != 1 || d != 'x') return 4;
    close(got);
    close(p[0]);
    close(p[1]);
    return 0;
  });
}

}  // extern "C"
