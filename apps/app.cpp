// app <rank> [root_ip] [n_ranks]
// Minimal example in the shape of the reference's (reference: src/main.cpp:16-70):
// every rank fills 1 Mi floats with (rank + 1), one in-place ncclAllReduce(sum),
// every element must equal n(n+1)/2 exactly.  Defaults to 2 ranks (1.0 + 2.0 = 3.0).
// Buffers are pinned host memory when a GPU exists (each rank uses GPU
// rank % device_count), ordinary host memory otherwise (network data plane).
// Exit code 0 on PASS, 1 on FAIL.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "mini_nccl_api.h"

#define NCCL_OK(call)                                                              \
  do {                                                                             \
    ncclResult_t _r = (call);                                                      \
    if (_r != ncclSuccess) {                                                       \
      fprintf(stderr, "%s failed: %s\n", #call, ncclGetErrorString(_r));           \
      return 1;                                                                    \
    }                                                                              \
  } while (0)

int main(int argc, char** argv) {
  if (argc < 2) {
    fprintf(stderr, "Usage: %s <rank> [root_ip] [n_ranks]\n", argv[0]);
    return 1;
  }
  const int rank = atoi(argv[1]);
  const char* ip = argc > 2 ? argv[2] : "127.0.0.1";
  const int n = argc > 3 ? atoi(argv[3]) : 2;
  const size_t count = 1024 * 1024;

  int ndev = 0;
  bool gpu = cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0;
  if (!gpu) (void)cudaGetLastError();
  if (gpu && cudaSetDevice(rank >= 0 ? rank % ndev : 0) != cudaSuccess) gpu = false;

  ncclComm_t comm;
  NCCL_OK(ncclCommInitRank(&comm, n, rank, ip));
  int my_rank = rank, world = n;
  NCCL_OK(ncclCommUserRank(comm, &my_rank));
  NCCL_OK(ncclCommCount(comm, &world));

  float* data = nullptr;
  std::vector<float> plain;
  cudaStream_t stream = nullptr;
  if (gpu) {
    if (cudaHostAlloc(reinterpret_cast<void**>(&data), count * sizeof(float), cudaHostAllocDefault) != cudaSuccess) return 1;
    cudaStreamCreate(&stream);
  } else {
    plain.resize(count);
    data = plain.data();
  }
  for (size_t i = 0; i < count; ++i) data[i] = static_cast<float>(my_rank + 1);

  NCCL_OK(ncclAllReduce(data, data, count, ncclFloat, ncclSum, comm, stream));
  if (gpu) cudaStreamSynchronize(stream);

  const float expect = static_cast<float>(world * (world + 1) / 2);
  bool pass = true;
  for (size_t i = 0; i < count; ++i) {
    if (data[i] != expect) {
      printf("[Rank %d] mismatch at %zu: expected %.1f, got %.1f\n", my_rank, i, expect, data[i]);
      pass = false;
      break;
    }
  }
  printf("[Rank %d] %s AllReduce of %zu floats = %.1f\n", my_rank, pass ? "[PASS]" : "[FAIL]", count, data[0]);
  NCCL_OK(ncclCommDestroy(comm));
  if (gpu) {
    cudaStreamDestroy(stream);
    cudaFreeHost(data);
  }
  return pass ? 0 : 1;
}
