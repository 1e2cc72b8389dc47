#include "algo/select.h"

#include <algorithm>
#include <strings.h>

namespace mnccl {
namespace {

bool nvls_type_ok(DType in, DType wire, DType out, RedOp op) {
  if (op != RedOp::Sum && op != RedOp::Avg) return false;
  auto f = [](DType t) { return t == DType::Float32 || t == DType::Float16 || t == DType::Bfloat16; };
  if (in == wire && wire == out) return f(wire);
  return wire == DType::Bfloat16 && ((in == DType::Float32 && (out == DType::Float32 || out == DType::Bfloat16)) ||
                                    (in == DType::Bfloat16 && out == DType::Float32));
}

bool triple_ok(DType in, DType wire, DType out, RedOp op) {
  if (in == wire && wire == out) return true;
  return nvls_type_ok(in, wire, out, op);  // the mixed triples are the same set
}

uint64_t ceil_div(uint64_t a, uint64_t b) { return (a + b - 1) / b; }

}  // namespace

Algo parse_algo(const std::string& s) {
  const char* c = s.c_str();
  if (!strcasecmp(c, "ll")) return Algo::LL;
  if (!strcasecmp(c, "oneshot")) return Algo::OneShot;
  if (!strcasecmp(c, "twoshot")) return Algo::TwoShot;
  if (!strcasecmp(c, "nvls")) return Algo::Nvls;
  if (!strcasecmp(c, "ring")) return Algo::Ring;
  if (!strcasecmp(c, "pipe")) return Algo::Pipe;
  return Algo::Auto;
}

Thresholds thresholds_for(int nranks, const Config& cfg, bool symmetric) {
  Thresholds t;
  // Crossovers from the device-timed sweep on 8xB200 (benchmarks/tune.py, fp32
  // sum, symmetric buffers).  N=2: one-shot moves no more bytes than two-shot
  // and wins up to 4 MB.  N=4: one-shot wins up to 512 KB.  N=8: LL and
  // one-shot tie up to 64 KB, NVLS wins from 256 KB on.
  if (nranks <= 2) {
    t.ll_max = 64u << 10;
    t.oneshot_max = 4u << 20;
  } else if (nranks <= 4) {
    t.ll_max = 64u << 10;
    t.oneshot_max = 512u << 10;
  } else {
    t.ll_max = 64u << 10;
    t.oneshot_max = 192u << 10;
  }
  // Ordinary (not symmetric) buffers have to be staged by the two-phase kernels, which costs
  // two extra passes over the data; one-shot reads the user buffer directly, so it stays ahead
  // up to 2 MB.
  if (!symmetric && nranks > 2) t.oneshot_max = 2u << 20;
  t.nvls_min = t.oneshot_max + 1;
  if (cfg.ll_max_bytes) t.ll_max = cfg.ll_max_bytes;
  if (cfg.oneshot_max_bytes) t.oneshot_max = cfg.oneshot_max_bytes;
  if (cfg.nvls_min_bytes) t.nvls_min = cfg.nvls_min_bytes;
  return t;
}

size_t default_ll_slot_bytes(int nranks, const Config& cfg) {
  size_t payload = std::max<size_t>(thresholds_for(nranks, cfg, true).ll_max, 64u << 10);
  return 2 * payload;
}

size_t default_inbox_slot_bytes(int nranks, const Config& cfg) {
  size_t cap = nranks <= 2 ? (4u << 20) : (2u << 20);
  return std::max<size_t>(cap, thresholds_for(nranks, cfg, false).oneshot_max);
}

Plan make_plan(const PlanInput& in, const CommCaps& caps, const Config& cfg) {
  Plan p;
  const int N = caps.nranks;
  const size_t wsz = dtype_size(in.wire), osz = dtype_size(in.out);
  const uint64_t VW = 16 / wsz;
  p.spec.mode = in.mode;
  p.spec.in = in.in;
  p.spec.wire = in.wire;
  p.spec.out = in.out;
  p.spec.op = in.op;
  p.spec.nthreads = 512;
  if (!triple_ok(in.in, in.wire, in.out, in.op)) {
    p.reason = "unsupported (send, wire, recv) type combination for this operator";
    return p;
  }
  const int max_blocks = cfg.max_blocks > 0 ? std::min(cfg.max_blocks, kMaxBlocks) : 0;

  if (N == 1) {
    if (in.mode != Mode::AllReduce && in.in != in.out) { p.reason = "type conversion needs AllReduce"; return p; }
    p.spec.algo = Algo::Local;
    const uint64_t vecs = ceil_div(in.count, std::min<uint64_t>(16 / dtype_size(in.in), 16 / osz));
    p.spec.nblocks = static_cast<int>(std::clamp<uint64_t>(ceil_div(vecs, 512 * 4), 1, caps.sm_count * 4));
    p.valid = true;
    return p;
  }

  const uint64_t total_elems = in.mode == Mode::AllReduce ? in.count : in.count * uint64_t(N);
  const uint64_t wire_bytes = total_elems * wsz;
  const Thresholds th = thresholds_for(N, cfg, in.in_symmetric && in.out_symmetric);
  Algo algo = in.forced;
  const bool nvls_types = nvls_type_ok(in.in, in.wire, in.out, in.op);
  // NVLS needs multicast views of whatever it touches: staging always has one
  // when caps.nvls; symmetric user buffers only if their segment does.
  // With two ranks the switch cannot win: both phases move S bytes per link
  // direction one after the other, while P2P moves S/2 each way at once.
  const bool nvls_usable = caps.nvls && N > 2 && nvls_types && in.mode != Mode::AllGather &&
                           (!in.in_symmetric || in.in_has_mc) && (!in.out_symmetric || in.out_has_mc);
  if (in.mode != Mode::AllReduce) {
    if (algo != Algo::TwoShot && algo != Algo::Nvls) algo = nvls_usable && in.mode == Mode::ReduceScatter && wire_bytes >= th.nvls_min ? Algo::Nvls : Algo::TwoShot;
    if (algo == Algo::Nvls && !(nvls_usable && in.mode == Mode::ReduceScatter)) algo = Algo::TwoShot;
  } else if (algo == Algo::Auto) {
    const bool ordinary = !(in.in_symmetric && in.out_symmetric);
    // The pipelined kernel is the automatic choice where the switch reduces (more than two ranks, a type
    // and operator it can add): measured 632 us for 256 MiB on 8 GPUs against 772 us for copy kernels on
    // side streams and 717 us for NCCL.  Its peer-to-peer form (forced with algo = pipe) measured slower
    // than the stream pipeline on two GPUs (800 against 605 us), so two ranks and the other operators
    // keep that one.
    const bool pipe_auto = caps.nvls && N > 2 && nvls_types;
    // Four GPUs, ordinary device buffers: the peer-to-peer two-shot kernel running on the user buffers
    // directly (lazy direct access) measured ahead of the staged switch kernel and of the pipelined
    // kernel from 4 MB to 128 MB (4 MB: 36.7 against 40.6 us; 16 MB: 67 against 81; 32 MB: 104 against
    // 146; 128 MB: 349 against 367; NCCL 35.2 / 70.6 / 119 / 354) and behind the pipelined kernel at
    // 256 MB (663 against 655); at 2 MB the one-shot kernel is faster (25.9 against 32.7).
    const bool direct_auto = ordinary && in.auto_eligible && !in.host_memory && N > 2 && N <= 4 &&
                             wire_bytes >= (4u << 20) && wire_bytes < (192u << 20);
    if (direct_auto) algo = Algo::TwoShot;
    else if (ordinary && pipe_auto && !in.host_memory && cfg.pipe_min_bytes != 0 && wire_bytes >= cfg.pipe_min_bytes) algo = Algo::Pipe;
    else if (wire_bytes <= th.ll_max && wire_bytes * 2 <= caps.ll_slot_bytes) algo = Algo::LL;
    else if (wire_bytes <= th.oneshot_max && wire_bytes <= caps.inbox_slot_bytes) algo = Algo::OneShot;
    else if (nvls_usable && wire_bytes >= th.nvls_min) algo = Algo::Nvls;
    else algo = Algo::TwoShot;
  }
  // Forced choices that cannot be honoured degrade to the next general one.
  if (algo == Algo::LL && ceil_div(wire_bytes, 8) * 16 > caps.ll_slot_bytes) algo = Algo::OneShot;
  if (algo == Algo::OneShot && ceil_div(wire_bytes, 16) * 16 > caps.inbox_slot_bytes) algo = Algo::TwoShot;
  if (algo == Algo::Nvls && !nvls_usable) algo = Algo::TwoShot;
  if (algo == Algo::Pipe && (in.mode != Mode::AllReduce || in.host_memory)) algo = Algo::TwoShot;
  if (algo == Algo::Ring || algo == Algo::Auto || algo == Algo::Local) algo = Algo::TwoShot;
  p.spec.algo = algo;

  if (algo == Algo::LL) {
    const uint64_t units = ceil_div(wire_bytes, 8);
    p.spec.nthreads = units <= 128 ? 128 : 256;
    p.spec.nblocks = static_cast<int>(std::clamp<uint64_t>(ceil_div(units, p.spec.nthreads), 1, max_blocks ? max_blocks : 64));
    p.valid = true;
    return p;
  }
  if (algo == Algo::OneShot) {
    const uint64_t vecs = ceil_div(wire_bytes, 16);
    p.spec.nthreads = vecs <= 256 ? 256 : 512;
    // measured on 8 GPUs, 1 MiB on ordinary buffers: 29.4 us with 64 blocks, 27.7 us with 128 (NCCL: 30)
    const uint64_t cap = max_blocks ? max_blocks : (wire_bytes >= (768u << 10) ? 128 : 64);
    p.spec.nblocks = static_cast<int>(std::clamp<uint64_t>(ceil_div(vecs, p.spec.nthreads), 1, cap));
    p.valid = true;
    return p;
  }

  if (algo == Algo::Pipe) {
    // One block per chunk and role: chunks are small (512 KB by default: measured best on 8 GPUs,
    // 632 us for 256 MiB against 660 with 1 MB and 790 with 256 KB), bounded by one ring slot of
    // either staging area; a chunk is N shards of E elements, E a multiple of the vector width.
    const uint64_t stride = caps.stage_bytes / kPipeSlots;
    uint64_t target = cfg.pipe_chunk_bytes ? cfg.pipe_chunk_bytes : (512u << 10);
    uint64_t ce = std::min<uint64_t>(target / wsz, stride / std::max(wsz, osz));
    uint64_t E = ce / (uint64_t(N) * VW) * VW;
    if (E == 0) { p.reason = "staging buffer too small for the pipelined kernel"; return p; }
    // Ramp: four chunks of 1/16, 1/8, 1/4 and 1/2 of the regular size first, where the shard still divides
    // into whole vectors and the message is long enough for it to matter.
    const uint64_t unit = VW << 4;
    if (E >= 4 * unit && total_elems >= 8 * E * uint64_t(N)) {
      E = E / unit * unit;
      p.pipe_ramp = 4;
    }
    p.shard_elems = E;
    p.chunk_shard_vecs = E / VW;
    p.copy_in = p.copy_out = true;
    p.spec.pipe_nvls = caps.nvls && N > 2 && nvls_types;
    int want = p.spec.pipe_nvls ? 48 : 112;  // switch path: 14 + 20 + 14 blocks measured best (more only add contention)
    if (max_blocks) want = max_blocks;
    p.spec.nblocks = std::clamp(want, 3, std::max(3, caps.sm_count - 8));
    p.valid = true;
    return p;
  }

  // Two-shot / NVLS geometry.
  uint64_t E;  // elements per shard
  if (in.mode == Mode::AllReduce) E = ceil_div(ceil_div(in.count, VW), uint64_t(N)) * VW;
  else E = in.count;
  p.shard_elems = E;
  const uint64_t shard_vecs = ceil_div(E, VW);
  // Zero-copy needs 16-byte aligned shard starts inside the user buffers.
  const bool shard_al_in = (E * dtype_size(in.in)) % 16 == 0;
  const bool shard_al_out = (E * osz) % 16 == 0;
  bool zc_in = in.in_symmetric && in.in == in.wire && shard_al_in;
  bool zc_out = in.out_symmetric && shard_al_out;
  if (in.mode == Mode::AllGather) zc_in = true;         // AllGather reads its own send buffer only
  if (in.mode == Mode::ReduceScatter) zc_out = true;    // ReduceScatter writes its own recv buffer only
  p.copy_in = !zc_in;
  p.copy_out = !zc_out;
  const uint64_t out_vb = VW * osz;
  uint64_t sv = shard_vecs;
  if (p.copy_in) sv = std::min<uint64_t>(sv, caps.stage_bytes / (uint64_t(N) * 16));
  if (p.copy_out) sv = std::min<uint64_t>(sv, caps.stage_bytes / (uint64_t(N) * out_vb));
  if (sv == 0) { p.reason = "staging buffer too small"; return p; }
  p.chunk_shard_vecs = sv;
  p.spec.unroll = (algo == Algo::Nvls && in.mode == Mode::AllReduce && cfg.unroll == 8) ? 8 : 4;
  const uint64_t tiles = ceil_div(std::min(sv, shard_vecs), 512 * uint64_t(p.spec.unroll));
  // Measured: the switch path peaks with ~32 CTAs (more only add contention),
  // the P2P path wants ~96.
  int cap = max_blocks ? max_blocks : ((algo == Algo::Nvls && !p.copy_in && !p.copy_out) ? 32 : 96);
  p.spec.nblocks = static_cast<int>(std::clamp<uint64_t>(tiles, 1, cap));
  p.valid = true;
  return p;
}

std::vector<size_t> pipeline_chunks(size_t count, size_t elem_bytes, size_t uniform_elems, size_t cap_elems, bool taper) {
  std::vector<size_t> out;
  if (count == 0) return out;
  const size_t kAlign = 4096;
  if (uniform_elems < kAlign) uniform_elems = kAlign;
  uniform_elems &= ~(kAlign - 1);
  const size_t total_bytes = count * elem_bytes;
  if (!taper || total_bytes < (size_t(128) << 20) || cap_elems < 2 * kAlign) {
    for (size_t off = 0; off < count; off += uniform_elems) out.push_back(std::min(uniform_elems, count - off));
    return out;
  }
  size_t edge_bytes = std::min<size_t>(std::max<size_t>(total_bytes / 8, size_t(8) << 20), size_t(32) << 20);
  size_t edge = (edge_bytes / elem_bytes) & ~(kAlign - 1);
  const size_t cap = cap_elems & ~(kAlign - 1);
  if (edge > cap) edge = cap;
  if (edge == 0 || 2 * edge >= count) {
    for (size_t off = 0; off < count; off += uniform_elems) out.push_back(std::min(uniform_elems, count - off));
    return out;
  }
  out.push_back(edge);
  size_t left = count - 2 * edge;        // what the large chunks carry; the last small chunk takes the ragged end
  const size_t n_mid = (left + cap - 1) / cap;
  size_t mid = ((left + n_mid - 1) / n_mid + kAlign - 1) & ~(kAlign - 1);  // equal large chunks
  if (mid > cap) mid = cap;
  while (left > 0) {
    const size_t n = std::min(mid, left);
    if (n < mid && (n & (kAlign - 1)) != 0) {
      // a ragged piece in the middle would break the alignment of what follows: give it to the tail
      const size_t whole = n & ~(kAlign - 1);
      if (whole) out.push_back(whole);
      left -= whole;
      break;
    }
    out.push_back(n);
    left -= n;
  }
  out.push_back(edge + left);            // last chunk: small, plus the ragged remainder (< 4096 elements)
  if (out.back() > cap) {                // cannot happen with edge <= cap - 4096; keep the invariant anyway
    const size_t extra = out.back() - cap;
    out.back() = cap;
    out.push_back(extra);
  }
  return out;
}


}  // namespace mnccl
