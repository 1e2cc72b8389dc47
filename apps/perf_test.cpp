// perf_test <rank> <n_ranks> [master_ip]      (rank = -1: Hera auto-bootstrap)
// The reference's benchmark, same command line and table (reference:
// tests/perf_test.cpp:34-158): fp32 sum, out of place, 1 / 16 / 64 / 128 MiB,
// 5 warm-up + 20 timed iterations, algBW = bytes / time, busBW = algBW * 2(n-1)/n,
// AVX2 verification against n * 1.0.  Differences: each rank uses GPU
// rank % device_count instead of GPU 0 for everyone, a verification failure makes
// the exit code non-zero, and a column with the device-side time (CUDA events)
// is printed next to the host-clock time the reference measures.
// Environment: PERF_TEST_DEVICE_BUFFERS=1 uses device memory instead of pinned
// host memory; PERF_TEST_MAX_MIB caps the sizes (useful without a GPU).
#include <immintrin.h>
#include <time.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "mini_nccl_api.h"

#define NCCL_OK(call)                                                              \
  do {                                                                             \
    ncclResult_t _r = (call);                                                      \
    if (_r != ncclSuccess) {                                                       \
      fprintf(stderr, "%s failed: %s\n", #call, ncclGetErrorString(_r));           \
      return 2;                                                                    \
    }                                                                              \
  } while (0)

static double now_us() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec * 1e6 + ts.tv_nsec * 1e-3;
}

// 8-wide compare against a constant, scalar tail at 1e-5.
static bool verify(const float* p, size_t n, float want, size_t* bad) {
  const __m256 w = _mm256_set1_ps(want);
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    __m256 v = _mm256_loadu_ps(p + i);
    int mask = _mm256_movemask_ps(_mm256_cmp_ps(v, w, _CMP_NEQ_UQ));
    if (mask) {
      *bad = i + static_cast<size_t>(__builtin_ctz(static_cast<unsigned>(mask)));
      return false;
    }
  }
  for (; i < n; ++i)
    if (!(std::fabs(p[i] - want) <= 1e-5f)) {
      *bad = i;
      return false;
    }
  return true;
}

int main(int argc, char** argv) {
  if (argc < 3) {
    fprintf(stderr, "Usage: %s <rank> <n_ranks> [master_ip]\n", argv[0]);
    fprintf(stderr, "       Pass rank = -1 to enable Hera Auto-Networking\n");
    return 1;
  }
  const int rank_arg = atoi(argv[1]);
  int n = atoi(argv[2]);
  const char* ip = argc > 3 ? argv[3] : "127.0.0.1";

  int ndev = 0;
  bool gpu = cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0;
  if (!gpu) (void)cudaGetLastError();
  // PERF_TEST_SHARE_GPU=1: every rank on GPU 0, the reference benchmark's layout (reference:
  // tests/perf_test.cpp:46); the library then runs its host-synchronised plane for ranks that share a GPU.
  const bool share_gpu = getenv("PERF_TEST_SHARE_GPU") && atoi(getenv("PERF_TEST_SHARE_GPU")) != 0;
  if (gpu && share_gpu) cudaSetDevice(0);
  else if (gpu && rank_arg >= 0) cudaSetDevice(rank_arg % ndev);  // Hera mode: the library picks the GPU from the local rank

  ncclComm_t comm;
  NCCL_OK(ncclCommInitRank(&comm, n, rank_arg, ip));
  int rank = rank_arg;
  NCCL_OK(ncclCommUserRank(comm, &rank));
  NCCL_OK(ncclCommCount(comm, &n));

  cudaStream_t stream = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (gpu) {
    cudaStreamCreate(&stream);
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
  }
  const bool device_buffers = gpu && getenv("PERF_TEST_DEVICE_BUFFERS") && atoi(getenv("PERF_TEST_DEVICE_BUFFERS")) != 0;
  const size_t max_mib = getenv("PERF_TEST_MAX_MIB") ? strtoul(getenv("PERF_TEST_MAX_MIB"), nullptr, 10) : 128;
  const size_t all_sizes[] = {1ul << 20, 16ul << 20, 64ul << 20, 128ul << 20};

  if (rank == 0) {
    printf("\n=== Mini-NCCL Performance Benchmark (Rank %d) ===\n", rank);
    printf("%15s %15s %15s %15s %15s\n", "Size(B)", "Time(us)", "AlgBW(GB/s)", "BusBW(GB/s)", "DevTime(us)");
  }
  int failures = 0;
  for (size_t size : all_sizes) {
    if (size > (max_mib << 20)) continue;
    const size_t count = size / sizeof(float);
    float *send = nullptr, *recv = nullptr, *h_send = nullptr, *h_recv = nullptr;
    std::vector<float> plain_send, plain_recv;
    if (gpu) {
      cudaHostAlloc(reinterpret_cast<void**>(&h_send), size, cudaHostAllocDefault);
      cudaHostAlloc(reinterpret_cast<void**>(&h_recv), size, cudaHostAllocDefault);
    } else {
      plain_send.resize(count);
      plain_recv.resize(count);
      h_send = plain_send.data();
      h_recv = plain_recv.data();
    }
    for (size_t i = 0; i < count; ++i) h_send[i] = 1.0f;
    memset(h_recv, 0, size);
    if (device_buffers) {
      cudaMalloc(reinterpret_cast<void**>(&send), size);
      cudaMalloc(reinterpret_cast<void**>(&recv), size);
      cudaMemcpy(send, h_send, size, cudaMemcpyHostToDevice);
      cudaMemset(recv, 0, size);
    } else {
      send = h_send;
      recv = h_recv;
    }
    for (int i = 0; i < 5; ++i) NCCL_OK(ncclAllReduce(send, recv, count, ncclFloat, ncclSum, comm, stream));
    if (gpu) cudaStreamSynchronize(stream);
    const int iterations = 20;
    if (gpu) cudaEventRecord(e0, stream);
    const double t0 = now_us();
    for (int i = 0; i < iterations; ++i) NCCL_OK(ncclAllReduce(send, recv, count, ncclFloat, ncclSum, comm, stream));
    if (gpu) {
      cudaEventRecord(e1, stream);
      cudaStreamSynchronize(stream);
    }
    const double t1 = now_us();
    float dev_ms = 0.f;
    if (gpu) cudaEventElapsedTime(&dev_ms, e0, e1);
    if (device_buffers) cudaMemcpy(h_recv, recv, size, cudaMemcpyDeviceToHost);

    size_t bad = 0;
    const bool pass = verify(h_recv, count, static_cast<float>(n), &bad);
    if (!pass) {
      printf("[Rank %d] Verification FAILED for size %zu at index %zu: expected %.1f, got %.1f\n", rank, size, bad,
             static_cast<float>(n), h_recv[bad]);
      ++failures;
    }
    const double avg_us = (t1 - t0) / iterations;
    const double alg = static_cast<double>(size) / avg_us / 1e3;
    const double bus = alg * 2.0 * (n - 1) / static_cast<double>(n);
    if (rank == 0)
      printf("%15zu %15.2f %15.2f %15.2f %15.2f %s\n", size, avg_us, alg, bus, dev_ms * 1e3 / iterations, pass ? "" : "(FAIL)");
    if (device_buffers) {
      cudaFree(send);
      cudaFree(recv);
    }
    if (gpu) {
      cudaFreeHost(h_send);
      cudaFreeHost(h_recv);
    }
    usleep(10000);
  }
  if (gpu) {
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaStreamDestroy(stream);
  }
  NCCL_OK(ncclCommDestroy(comm));
  return failures ? 3 : 0;
}
