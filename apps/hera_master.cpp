// hera_master <world_size> [port]
// Stand-alone Hera-Core master: hands out ranks in arrival order and the root
// address, then stays up serving heartbeats / aborts until killed.  Same
// command line as the reference's program (reference:
// tests/hera_master_main.cpp:5-13) plus an optional port.
#include <csignal>
#include <cstdio>
#include <cstdlib>

#include "bootstrap/hera.h"

static mnccl::hera::Master* g_master = nullptr;
static void on_signal(int) {
  if (g_master) g_master->stop();
}

int main(int argc, char** argv) {
  if (argc < 2) {
    fprintf(stderr, "Usage: %s <world_size> [port]\n", argv[0]);
    return 1;
  }
  int world = atoi(argv[1]);
  int port = argc > 2 ? atoi(argv[2]) : mnccl::hera::kDefaultPort;
  if (world <= 0 || port <= 0 || port > 65535) {
    fprintf(stderr, "invalid world size or port\n");
    return 1;
  }
  try {
    mnccl::hera::Master master(world, port);
    g_master = &master;
    signal(SIGINT, on_signal);
    signal(SIGTERM, on_signal);
    master.run();
  } catch (const std::exception& e) {
    fprintf(stderr, "[Hera-Master] %s\n", e.what());
    return 2;
  }
  return 0;
}
