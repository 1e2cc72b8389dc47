// Single-GPU emulation of a multi-rank communicator, for tests and debugging.
// All "ranks" live in one process on one device: each gets its own control
// segment and the peer pointers are ordinary device pointers.  A collective is
// ONE cooperative launch that covers the blocks of every virtual rank, so the
// ranks' blocks are co-resident and may wait on one another.  (Ranks emulated
// as separate launches, streams or processes on one GPU could never be
// guaranteed to run concurrently.)  NVLS needs a real multicast object and is
// not emulated.
#include <cuda_runtime.h>

#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "algo/select.h"
#include "core/config.h"
#include "core/error.h"
#include "core/log.h"
#include "kernels/dev_prims.cuh"
#include "kernels/launch.h"

namespace mnccl {
namespace {

struct EmuWorld {
  int n = 0;
  CommCaps caps;
  std::vector<CommDev> dev;
  std::vector<char*> ctrl;
  KParams* table = nullptr;  // device
  std::vector<std::vector<std::pair<char*, size_t>>> segs;  // symmetric allocations: [alloc][rank] -> (ptr, bytes)
  std::vector<int> deaf;
  uint64_t timeout_ns = 2000000000ull;
  size_t ctrl_bytes = 0;
  int last_algo = 0, last_blocks = 0;
  Config cfg;
  // lazy direct access: which virtual rank has which rank's buffers "mapped" (row q, column r), and the
  // tables the kernel reads (device memory here; every buffer lives in the one address space)
  std::vector<int> auto_mapped;
  AutoMapEntry* auto_tab = nullptr;  // [n][kMaxRanks * kAutoSlots]
};

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

#define EMU_RT(call)                                   \
  do {                                                 \
    cudaError_t _e = (call);                           \
    if (_e != cudaSuccess) {                           \
      (void)cudaGetLastError();                        \
      return static_cast<int>(_e) + 1000;              \
    }                                                  \
  } while (0)

__global__ void bounded_wait_probe(CommDev c, uint32_t* flag, uint32_t target, uint32_t* out) {
  // One thread waits for a flag that nothing sets; the wait must give up.
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const uint64_t t0 = dev::globaltimer_ns();
    uint32_t r = dev::wait_ge(flag, target, c);
    const uint64_t t1 = dev::globaltimer_ns();
    out[0] = r;
    out[1] = static_cast<uint32_t>((t1 - t0) / 1000ull);  // microseconds waited
  }
}

}  // namespace
}  // namespace mnccl

using namespace mnccl;

extern "C" {
#define MNCCL_EXPORT __attribute__((visibility("default")))

MNCCL_EXPORT int mncclEmuCreate(int nranks, size_t staging_bytes, void** world) {
  if (!world || nranks < 2 || nranks > kMaxRanks) return 4;
  auto* w = new EmuWorld();
  w->n = nranks;
  w->cfg = Config::get();
  if (staging_bytes) w->cfg.staging_bytes = staging_bytes;
  w->caps.nranks = nranks;
  w->caps.nvls = false;
  int devid = 0, sms = 0;
  EMU_RT(cudaGetDevice(&devid));
  EMU_RT(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, devid));
  w->caps.sm_count = sms;
  w->caps.ll_slot_bytes = align_up(default_ll_slot_bytes(nranks, w->cfg), 4096);
  w->caps.inbox_slot_bytes = align_up(default_inbox_slot_bytes(nranks, w->cfg), 4096);
  w->caps.stage_bytes = align_up(w->cfg.staging_bytes, 4096);
  CommDev proto;
  memset(&proto, 0, sizeof(proto));
  size_t off = 0;
  proto.off_sig = off;
  off += align_up(sizeof(uint32_t) * kMaxBlocks * kMaxRanks, 4096);
  proto.off_local = off;
  off += align_up(sizeof(LocalState), 4096);
  proto.off_pipe = off;
  off += align_up(sizeof(PipeCtl), 4096);
  proto.off_auto = off;
  off += align_up(sizeof(AutoCtl), 4096);
  proto.off_ll = off;
  off += 2 * size_t(nranks) * w->caps.ll_slot_bytes;
  proto.off_inbox = off;
  off += 2 * size_t(nranks) * w->caps.inbox_slot_bytes;
  off = align_up(off, 1 << 16);
  proto.off_stage_a = off;
  off += w->caps.stage_bytes;
  proto.off_stage_b = off;
  off += w->caps.stage_bytes;
  proto.ll_slot_bytes = w->caps.ll_slot_bytes;
  proto.inbox_slot_bytes = w->caps.inbox_slot_bytes;
  proto.stage_bytes = w->caps.stage_bytes;
  proto.nranks = nranks;
  proto.spin_timeout_ns = w->timeout_ns;
  w->ctrl_bytes = off;
  w->ctrl.assign(nranks, nullptr);
  for (int r = 0; r < nranks; ++r) {
    EMU_RT(cudaMalloc(&w->ctrl[r], off));
    EMU_RT(cudaMemset(w->ctrl[r], 0, off));
  }
  for (int r = 0; r < nranks; ++r) proto.ctrl[r] = w->ctrl[r];
  w->dev.assign(nranks, proto);
  for (int r = 0; r < nranks; ++r) w->dev[r].rank = r;
  w->deaf.assign(nranks, 0);
  EMU_RT(cudaMalloc(&w->table, sizeof(KParams) * nranks));
  EMU_RT(cudaDeviceSynchronize());
  *world = w;
  return 0;
}

MNCCL_EXPORT int mncclEmuDestroy(void* world) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w) return 4;
  cudaDeviceSynchronize();
  for (char* p : w->ctrl) cudaFree(p);
  if (w->auto_tab) cudaFree(w->auto_tab);
  for (auto& a : w->segs)
    for (auto& pr : a) cudaFree(pr.first);
  cudaFree(w->table);
  delete w;
  (void)cudaGetLastError();
  return 0;
}

// "Symmetric" allocation: one buffer per virtual rank; ptrs[nranks] receives them.
MNCCL_EXPORT int mncclEmuAlloc(void* world, size_t bytes, void** ptrs) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w || !ptrs || !bytes) return 4;
  std::vector<std::pair<char*, size_t>> a(w->n);
  for (int r = 0; r < w->n; ++r) {
    EMU_RT(cudaMalloc(&a[r].first, align_up(bytes, 256)));
    a[r].second = bytes;
    ptrs[r] = a[r].first;
  }
  w->segs.push_back(a);
  return 0;
}

MNCCL_EXPORT int mncclEmuSetTimeoutNs(void* world, uint64_t ns) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w) return 4;
  w->timeout_ns = ns;
  for (auto& d : w->dev) d.spin_timeout_ns = ns;
  return 0;
}

// Chunk size of the pipelined kernel for the calls that follow (0 = built-in choice).  Small chunks
// make a small message wrap the ring of staging slots, which is what the tests want to see.
MNCCL_EXPORT int mncclEmuSetPipeChunk(void* world, size_t bytes) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w) return 4;
  w->cfg.pipe_chunk_bytes = bytes;
  return 0;
}

// The size of the staging areas as the KERNELS are told it, without changing the allocation or the
// planning: a smaller claim makes staged accesses cross the claimed end while they stay inside memory
// the world owns.  For the checked build (MNCCL_DEVICE_CHECKS), whose kernels must record and skip such
// accesses; 0 restores the true size.
MNCCL_EXPORT int mncclEmuClaimStageBytes(void* world, size_t bytes) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w || bytes > w->caps.stage_bytes) return 4;
  for (auto& d : w->dev) d.stage_bytes = bytes ? bytes : w->caps.stage_bytes;
  return 0;
}

// 1 when this library was compiled with the device-side checks.
MNCCL_EXPORT int mncclBuiltWithDeviceChecks(void) {
#ifdef MNCCL_DEVICE_CHECKS
  return 1;
#else
  return 0;
#endif
}

// A deaf rank takes no part in the collective (its kernel sees zero ranks and
// zero elements): it neither signals nor waits, so its peers' bounded waits
// run out.  Host-made failure for tests.
MNCCL_EXPORT int mncclEmuSetDeaf(void* world, int rank, int on) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w || rank < 0 || rank >= w->n) return 4;
  w->deaf[rank] = on;
  return 0;
}

// mode: 0 AllReduce, 1 ReduceScatter, 2 AllGather.  send / recv: nranks device
// pointers each.  algo: mncclAlgo_t (0 = auto).  nblocks 0 = planned value.
MNCCL_EXPORT int mncclEmuCollective(void* world, int mode, const void* const* send, void* const* recv, size_t count,
                                    int in_type, int wire_type, int out_type, int op, double scale, int algo,
                                    int nblocks, cudaStream_t stream) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w || !send || !recv) return 4;
  if (!valid_dtype(in_type) || !valid_dtype(wire_type) || !valid_dtype(out_type) || !valid_op(op)) return 4;
  if (count == 0) return 0;
  const int N = w->n;
  PlanInput pi;
  pi.mode = static_cast<Mode>(mode);
  pi.count = count;
  pi.in = static_cast<DType>(in_type);
  pi.wire = static_cast<DType>(wire_type);
  pi.out = static_cast<DType>(out_type);
  pi.op = static_cast<RedOp>(op);
  pi.forced = static_cast<Algo>(algo);
  // Zero-copy when every rank's buffer comes from the same emulated symmetric allocation.
  auto find = [&](const void* const* ptrs, size_t bytes, size_t* off) -> int {
    for (size_t a = 0; a < w->segs.size(); ++a) {
      const char* p0 = static_cast<const char*>(ptrs[0]);
      if (p0 < w->segs[a][0].first || p0 + bytes > w->segs[a][0].first + w->segs[a][0].second) continue;
      size_t o = p0 - w->segs[a][0].first;
      bool all = true;
      for (int r = 1; r < N; ++r) all = all && static_cast<const char*>(ptrs[r]) == w->segs[a][r].first + o;
      if (all) { *off = o; return static_cast<int>(a); }
    }
    return -1;
  };
  const size_t in_elems = pi.mode == Mode::ReduceScatter ? count * N : count;
  const size_t out_elems = pi.mode == Mode::AllGather ? count * N : count;
  size_t in_off = 0, out_off = 0;
  int in_seg = find(send, in_elems * dtype_size(pi.in), &in_off);
  int out_seg = find(const_cast<const void* const*>(recv), out_elems * dtype_size(pi.out), &out_off);
  pi.in_symmetric = in_seg >= 0 && (reinterpret_cast<uintptr_t>(send[0]) & 15u) == 0;
  pi.out_symmetric = out_seg >= 0 && (reinterpret_cast<uintptr_t>(recv[0]) & 15u) == 0;
  Plan plan = make_plan(pi, w->caps, w->cfg);
  if (!plan.valid) return 4;
  if (plan.spec.algo == Algo::Nvls) return 5;
  if (nblocks > 0) plan.spec.nblocks = nblocks;
  int cap = max_emulated_blocks(plan.spec, N);
  if (cap <= 0) return 4;
  if (plan.spec.nblocks > cap) plan.spec.nblocks = cap;
  w->last_algo = static_cast<int>(plan.spec.algo);
  w->last_blocks = plan.spec.nblocks;

  // Lazy direct access (mncclEmuSetAutoMap): the staged two-shot kernel that goes direct when every
  // virtual rank has every rank's buffers in its table.
  bool auto_direct = false;
  if (!w->auto_mapped.empty() && pi.mode == Mode::AllReduce && plan.spec.algo == Algo::TwoShot && plan.copy_in && plan.copy_out &&
      pi.in == pi.wire && pi.in == pi.out) {
    LaunchSpec probe = plan.spec;
    probe.auto_direct = true;
    if (kernel_exists(probe)) {
      auto_direct = true;
      plan.spec.auto_direct = true;
      if (plan.spec.nblocks > kAutoBlocks) plan.spec.nblocks = kAutoBlocks;
      const int cap2 = max_emulated_blocks(plan.spec, N);
      if (cap2 <= 0) return 4;
      if (plan.spec.nblocks > cap2) plan.spec.nblocks = cap2;
      w->last_blocks = plan.spec.nblocks;
      std::vector<AutoMapEntry> tab(static_cast<size_t>(N) * kMaxRanks * kAutoSlots);
      memset(tab.data(), 0, tab.size() * sizeof(AutoMapEntry));
      const uint64_t bytes = count * dtype_size(pi.in);
      for (int q = 0; q < N; ++q)
        for (int r = 0; r < N; ++r) {
          if (q == r || !w->auto_mapped[q * N + r]) continue;
          AutoMapEntry* row = tab.data() + (static_cast<size_t>(q) * kMaxRanks + r) * kAutoSlots;
          row[0] = AutoMapEntry{uint64_t(2 * r + 1), reinterpret_cast<uint64_t>(send[r]), bytes, reinterpret_cast<uint64_t>(send[r])};
          if (recv[r] != send[r])
            row[1] = AutoMapEntry{uint64_t(2 * r + 2), reinterpret_cast<uint64_t>(recv[r]), bytes, reinterpret_cast<uint64_t>(recv[r])};
        }
      if (!w->auto_tab) EMU_RT(cudaMalloc(&w->auto_tab, tab.size() * sizeof(AutoMapEntry)));
      EMU_RT(cudaMemcpyAsync(w->auto_tab, tab.data(), tab.size() * sizeof(AutoMapEntry), cudaMemcpyHostToDevice, stream));
      EMU_RT(cudaStreamSynchronize(stream));
    }
  }

  const bool is_float = pi.in == DType::Float16 || pi.in == DType::Bfloat16 || pi.in == DType::Float32 || pi.in == DType::Float64;
  std::vector<KParams> host(N);
  for (int r = 0; r < N; ++r) {
    KParams& kp = host[r];
    memset(&kp, 0, sizeof(kp));
    kp.comm = w->dev[r];
    CollArgs& a = kp.args;
    a.send = send[r];
    a.recv = recv[r];
    a.count = count;
    a.shard_elems = plan.shard_elems;
    a.chunk_shard_vecs = plan.chunk_shard_vecs;
    const double factor = scale * (pi.op == RedOp::Avg ? 1.0 / N : 1.0);
    a.scale_f = static_cast<float>(factor);
    a.scale_d = factor;
    a.int_div = (pi.op == RedOp::Avg && !is_float) ? N : 0;
    a.copy_in = plan.copy_in;
    a.copy_out = plan.copy_out;
    a.pipe_ramp = plan.pipe_ramp;
    if (w->deaf[r]) {  // takes no part: moves nothing, signals nobody
      kp.comm.nranks = 0;
      a.count = 0;
      a.shard_elems = 0;
    }
    if (auto_direct) {
      // slot 0 of every rank is its send buffer, slot 1 its recv buffer
      const bool usable = ((reinterpret_cast<uintptr_t>(send[r]) | reinterpret_cast<uintptr_t>(recv[r])) & 15u) == 0;
      a.auto_desc.send_addr = reinterpret_cast<uint64_t>(send[r]);
      a.auto_desc.recv_addr = reinterpret_cast<uint64_t>(recv[r]);
      a.auto_desc.slots = usable ? (0u | ((recv[r] == send[r] ? 0u : 1u) << 8) | (1u << 16)) : 0u;
      for (int q = 0; q < N && q < kAutoRanks; ++q) a.auto_desc.mask[q] = (q != r && w->auto_mapped[r * N + q]) ? 3u : 0u;
      kp.comm.auto_map = w->auto_tab + static_cast<size_t>(r) * kMaxRanks * kAutoSlots;
    }
    const bool zc_in = !plan.copy_in && pi.mode != Mode::AllGather;
    const bool zc_out = !plan.copy_out && pi.mode != Mode::ReduceScatter;
    const bool staged_algo = plan.spec.algo == Algo::TwoShot;
    for (int q = 0; staged_algo && q < N; ++q) {
      a.in_peer[q] = zc_in ? w->segs[in_seg][q].first + in_off : w->ctrl[q] + w->dev[q].off_stage_a;
      a.out_peer[q] = zc_out ? w->segs[out_seg][q].first + out_off : w->ctrl[q] + w->dev[q].off_stage_b;
    }
  }
  EMU_RT(cudaMemcpyAsync(w->table, host.data(), sizeof(KParams) * N, cudaMemcpyHostToDevice, stream));
  EMU_RT(cudaStreamSynchronize(stream));  // `host` goes out of scope; keep it simple
  EMU_RT(launch_collective_emulated(plan.spec, w->table, N, stream));
  return 0;
}

// Lazy direct access in the emulated world.  mapped[q * nranks + r] != 0: virtual rank q has rank r's
// buffers in its table; null switches the feature off again.  While set, AllReduce calls that plan as
// the staged two-shot kernel (ordinary buffers, one type) run the kernel that goes direct when every
// rank can reach every buffer.
MNCCL_EXPORT int mncclEmuSetAutoMap(void* world, const int* mapped) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w) return 4;
  if (!mapped) w->auto_mapped.clear();
  else w->auto_mapped.assign(mapped, mapped + w->n * w->n);
  return 0;
}

// direct[nranks]: how many calls of every virtual rank ran on the user buffers directly.
MNCCL_EXPORT int mncclEmuDirectCalls(void* world, uint32_t* direct) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w || !direct) return 4;
  EMU_RT(cudaDeviceSynchronize());
  for (int r = 0; r < w->n; ++r) {
    LocalState ls;
    EMU_RT(cudaMemcpy(&ls, w->ctrl[r] + w->dev[r].off_local, sizeof(ls), cudaMemcpyDeviceToHost));
    direct[r] = ls.pad[0];
  }
  return 0;
}

// status[nranks]: LocalState::status of every virtual rank (0 = fine).
MNCCL_EXPORT int mncclEmuStatus(void* world, uint32_t* status, uint32_t* detail) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w || !status) return 4;
  EMU_RT(cudaDeviceSynchronize());
  for (int r = 0; r < w->n; ++r) {
    LocalState ls;
    EMU_RT(cudaMemcpy(&ls, w->ctrl[r] + w->dev[r].off_local, sizeof(ls), cudaMemcpyDeviceToHost));
    status[r] = ls.status;
    if (detail) detail[r] = ls.detail;
  }
  return 0;
}

MNCCL_EXPORT int mncclEmuLastPlan(void* world, int* algo, int* nblocks) {
  auto* w = static_cast<EmuWorld*>(world);
  if (!w) return 4;
  if (algo) *algo = w->last_algo;
  if (nblocks) *nblocks = w->last_blocks;
  return 0;
}

// Runs the device-side bounded wait on a flag that nothing sets.  Writes the
// status the wait returned (kDevTimeout expected) and the microseconds it
// spent.  abort_first != 0: an abort word (device memory here) is pre-set, so
// the wait must return kDevAborted at once.
MNCCL_EXPORT int mncclProbeBoundedWait(uint64_t timeout_ns, int abort_first, uint32_t* status, uint32_t* waited_us) {
  uint32_t* buf = nullptr;  // [0] flag, [1] abort, [2..3] out
  EMU_RT(cudaMalloc(&buf, 16));
  EMU_RT(cudaMemset(buf, 0, 16));
  if (abort_first) {
    uint32_t one = 1;
    EMU_RT(cudaMemcpy(buf + 1, &one, 4, cudaMemcpyHostToDevice));
  }
  CommDev c;
  memset(&c, 0, sizeof(c));
  c.spin_timeout_ns = timeout_ns;
  c.abort_word = buf + 1;
  bounded_wait_probe<<<1, 32>>>(c, buf, 1u, buf + 2);
  cudaError_t e = cudaDeviceSynchronize();
  uint32_t out[2] = {0, 0};
  if (e == cudaSuccess) e = cudaMemcpy(out, buf + 2, 8, cudaMemcpyDeviceToHost);
  cudaFree(buf);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return static_cast<int>(e) + 1000;
  }
  if (status) *status = out[0];
  if (waited_us) *waited_us = out[1];
  return 0;
}

}  // extern "C"
