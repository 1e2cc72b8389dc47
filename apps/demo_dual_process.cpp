// demo_dual_process server|client [ip] [port]
// Transport bring-up demo in the spirit of the reference's "01_dual_process_rdma" (reference:
// demos/01_dual_process_rdma/src/main.cu:26-193): two processes shake hands over TCP, register a
// 1 KiB buffer each and exchange a greeting.  The reference does it with two-sided SEND / RECV on a
// hard-wired rxe0 device; here the greeting travels the way the library's data plane works: a
// one-sided write into the peer's registered buffer followed by a flag write on the same ordered
// connection, through whichever provider is available (libibverbs when compiled in, else the TCP
// emulation), and the completion status is checked.  No GPU kernel is involved, as in the
// reference's demo.
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "bootstrap/store.h"
#include "core/config.h"
#include "core/error.h"
#include "net/transport.h"

using namespace mnccl;

int main(int argc, char** argv) {
  if (argc < 2 || (strcmp(argv[1], "server") != 0 && strcmp(argv[1], "client") != 0)) {
    fprintf(stderr, "Usage: %s server|client [ip] [port]\n", argv[0]);
    return 1;
  }
  const int rank = strcmp(argv[1], "server") == 0 ? 0 : 1;
  const char* ip = argc > 2 ? argv[2] : "127.0.0.1";
  const int port = argc > 3 ? atoi(argv[3]) : 8888;
  try {
    const Config& cfg = Config::get();
    BootstrapStore store(rank, 2, ip, port, cfg.socket_timeout_ms, cfg.connect_retries);
    store.connect();
    std::unique_ptr<OneSidedTransport> t = make_transport(cfg.transport == "verbs" ? "verbs" : "auto", rank, 2);
    t->connect(store);
    printf("[%s] transport: %s\n", argv[1], t->name());

    alignas(64) static char inbox[1024];
    alignas(64) static char outbox[1024];
    memset(inbox, 0, sizeof(inbox));
    snprintf(outbox, sizeof(outbox), "Hello from the %s (pid %d)", argv[1], static_cast<int>(getpid()));
    auto in_mr = t->register_memory(inbox, sizeof(inbox));
    auto out_mr = t->register_memory(outbox, sizeof(outbox));
    struct Peer { RemoteBuffer inbox, flags; } me{{reinterpret_cast<uint64_t>(inbox), in_mr->rkey, 0}, t->flags_remote()}, all[2];
    store.all_gather(&me, all, sizeof(me));
    const int peer = 1 - rank;

    Request* data = t->write(peer, outbox, *out_mr, all[peer].inbox, 0, sizeof(outbox), true);
    Request* flag = t->write_flag(peer, all[peer].flags, 0, 1, true);
    if (!t->wait(data, 5000) || !t->wait(flag, 5000)) fail(Result::InternalError, "send completion timed out");
    t->release(data);
    t->release(flag);

    auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(10);
    while (__atomic_load_n(t->flags(), __ATOMIC_ACQUIRE) == 0) {
      t->poll();
      if (std::chrono::steady_clock::now() > deadline) fail(Result::InternalError, "no greeting arrived");
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    printf("[%s] received: \"%s\"\n", argv[1], inbox);
    store.barrier();
    const bool ok = strncmp(inbox, "Hello from the ", 15) == 0;
    printf("[%s] %s\n", argv[1], ok ? "[PASS]" : "[FAIL]");
    return ok ? 0 : 1;
  } catch (const std::exception& e) {
    fprintf(stderr, "[%s] error: %s\n", argv[1], e.what());
    return 2;
  }
}
