// Host self-test meant to be built with sanitizers (address + undefined, or thread): it drives
// the host components through the same hooks the Python tests use, plus a three-rank ring
// AllReduce whose ranks are threads of this process (so the thread sanitizer sees the transport's
// receiver threads, the request pool and the flag protocol together).  The reference has no
// sanitizer or race-detection support of any kind.
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include "bootstrap/store.h"
#include "core/config.h"
#include "net/ring.h"
#include "net/soft_transport.h"

extern "C" {
int mnccl_test_spsc(int, int);
int mnccl_test_request_pool(int);
int mnccl_test_reg_cache();
int mnccl_test_watchdog(int, int);
int mnccl_test_fdpass(const char*);
int mnccl_test_config(const char*, char*, size_t);
void* mnccl_hera_master_start(int, int, int);
int mnccl_hera_master_port(void*);
int mnccl_hera_master_registered(void*);
void mnccl_hera_master_stop(void*);
void* mnccl_hera_worker_register(const char*, int, int*, int*, char*);
void mnccl_hera_worker_free(void*);
}

using namespace mnccl;

static int g_fail = 0;
#define CHECK(cond)                                                  \
  do {                                                               \
    if (!(cond)) {                                                   \
      fprintf(stderr, "[FAIL] %s:%d %s\n", __FILE__, __LINE__, #cond); \
      ++g_fail;                                                      \
    }                                                                \
  } while (0)

// count: 200003 elements run in one thread per rank; 1100003 (4.4 MB) take the ring's second thread,
// so that the thread sanitizer sees the sender, the receiver and the provider's threads together.
static void ring_threads(int port, size_t count, int iters) {
  const int n = 3;
  std::vector<std::vector<float>> data(n, std::vector<float>(count));
  for (int r = 0; r < n; ++r)
    for (size_t i = 0; i < count; ++i) data[r][i] = static_cast<float>((i * 7 + r * 13) % 101) * 0.25f;
  std::vector<float> want(count);
  for (size_t i = 0; i < count; ++i) want[i] = data[0][i] + data[1][i] + data[2][i];
  std::atomic<int> errors{0};
  std::vector<std::thread> th;
  for (int r = 0; r < n; ++r) {
    th.emplace_back([&, r] {
      try {
        Config cfg = Config::get();
        cfg.slice_size = 4096;
        cfg.window_size = 4;
        cfg.signal_batch = 3;
        BootstrapStore store(r, n, "127.0.0.1", port, 10000, 50);
        store.connect();
        SoftTransport t(r, n);
        t.connect(store);
        RingAllReduce ring(r, n, &t, &store, cfg, nullptr);
        for (int it = 0; it < iters; ++it) {
          std::vector<float> buf = data[r];
          ring.run(buf.data(), count, DType::Float32, RedOp::Sum);
          for (size_t i = 0; i < count; ++i)
            if (std::fabs(buf[i] - want[i]) > 1e-3f) { errors++; break; }
        }
        if (count * sizeof(float) >= (size_t(4) << 20) && ring.stats().threaded_calls != static_cast<uint64_t>(iters)) errors++;
        store.barrier();
      } catch (const std::exception& e) {
        fprintf(stderr, "rank %d: %s\n", r, e.what());
        errors++;
      }
    });
  }
  for (auto& t : th) t.join();
  CHECK(errors.load() == 0);
}

int main(int argc, char** argv) {
  const int port = argc > 1 ? atoi(argv[1]) : 23456;
  CHECK(mnccl_test_spsc(7, 200000) == 0);
  CHECK(mnccl_test_request_pool(64) == 0);
  CHECK(mnccl_test_reg_cache() == 0);
  for (int s = 0; s < 3; ++s) CHECK(mnccl_test_watchdog(s, 50) == (s == 0 ? 0 : 1));
  CHECK(mnccl_test_fdpass("selftest") == 0);
  char buf[1024];
  CHECK(mnccl_test_config("MINI_NCCL_SIGNAL_BATCH=0", buf, sizeof(buf)) == 0);
  void* m = mnccl_hera_master_start(4, port + 1, 0);
  CHECK(m != nullptr);
  if (m) {
    std::vector<std::thread> ws;
    std::atomic<int> sum{0};
    for (int i = 0; i < 4; ++i)
      ws.emplace_back([&] {
        int rank = -1, size = 0;
        char root[64];
        void* w = mnccl_hera_worker_register("127.0.0.1", mnccl_hera_master_port(m), &rank, &size, root);
        if (w && size == 4) sum += rank + 1;
        if (w) mnccl_hera_worker_free(w);
      });
    for (auto& t : ws) t.join();
    CHECK(sum.load() == 10);  // ranks 0..3, each once
    CHECK(mnccl_hera_master_registered(m) == 4);
    mnccl_hera_master_stop(m);
  }
  ring_threads(port, 200003, 3);
  ring_threads(port + 7, 1100003, 2);
  printf(g_fail ? "[FAIL] host self-test: %d check(s) failed\n" : "[PASS] host self-test\n", g_fail);
  return g_fail ? 1 : 0;
}
