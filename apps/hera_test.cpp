// In-process integration test of the control plane: one master thread and
// four workers that register 100 ms apart on 127.0.0.1.  The reference's test
// of the same shape only checks that the workers return (reference:
// tests/hera_test.cpp:9-47); this one also checks the assignment: ranks are
// 0..3 in arrival order, every worker learns the world size and the same root
// address, and a frame with a bad magic number is rejected.
#include <arpa/inet.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "bootstrap/hera.h"
#include "bootstrap/socket.h"

using namespace mnccl;

int main(int argc, char** argv) {
  const int kWorkers = 4;
  int port = argc > 1 ? atoi(argv[1]) : hera::kDefaultPort;
  hera::Master master(kWorkers, port);
  master.start_background();
  port = master.port();

  // A stranger speaking another protocol must not disturb registration.
  try {
    TcpSocket bad = TcpSocket::connect_to("127.0.0.1", port, 5, 100);
    hera::Header h{0xdeadbeefu, 1, 1, 0, 0};
    bad.send_all(&h, sizeof(h), 1000);
  } catch (const std::exception& e) {
    fprintf(stderr, "[FAIL] could not reach the master: %s\n", e.what());
    return 1;
  }
  std::this_thread::sleep_for(std::chrono::milliseconds(150));

  std::vector<int> ranks(kWorkers, -1), sizes(kWorkers, 0);
  std::vector<std::string> roots(kWorkers);
  std::atomic<int> failures{0};
  std::vector<std::thread> threads;
  for (int i = 0; i < kWorkers; ++i) {
    threads.emplace_back([&, i] {
      std::this_thread::sleep_for(std::chrono::milliseconds(100 * i));
      try {
        hera::Worker w("127.0.0.1", port);
        w.connect_and_register(20, 100, 5000);
        ranks[i] = w.rank();
        sizes[i] = w.size();
        roots[i] = w.root_ip();
      } catch (const std::exception& e) {
        fprintf(stderr, "[Worker %d] %s\n", i, e.what());
        failures++;
      }
    });
  }
  for (auto& t : threads) t.join();
  bool ok = failures.load() == 0;
  for (int i = 0; i < kWorkers; ++i) {
    if (ranks[i] != i) { fprintf(stderr, "[FAIL] worker %d got rank %d (arrival order expected)\n", i, ranks[i]); ok = false; }
    if (sizes[i] != kWorkers) { fprintf(stderr, "[FAIL] worker %d got world size %d\n", i, sizes[i]); ok = false; }
    if (roots[i] != "127.0.0.1") { fprintf(stderr, "[FAIL] worker %d got root '%s'\n", i, roots[i].c_str()); ok = false; }
  }
  if (!master.all_registered()) { fprintf(stderr, "[FAIL] master does not report a full world\n"); ok = false; }
  master.stop();
  printf(ok ? "[PASS] Hera-Core: 4 workers registered, ranks 0..3, root 127.0.0.1\n" : "[FAIL] Hera-Core test\n");
  return ok ? 0 : 1;
}
