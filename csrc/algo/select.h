// Algorithm choice and launch geometry: pure functions of the message and the
// communicator's capabilities, so they can be unit-tested without a GPU.  The
// reference has one algorithm (ring) for every size (reference:
// src/mini_nccl.cu:107-194); here the variant is picked per message size from
// a table of measured crossovers, with environment overrides
// (MINI_NCCL_ALGO, MINI_NCCL_LL_MAX_BYTES, MINI_NCCL_ONESHOT_MAX_BYTES,
// MINI_NCCL_NVLS_MIN_BYTES, MINI_NCCL_MAX_BLOCKS).
#pragma once
#include <vector>
#include <cstddef>
#include <cstdint>

#include "core/config.h"
#include "core/dtype.h"
#include "kernels/launch.h"

namespace mnccl {

struct CommCaps {
  int nranks = 1;
  bool nvls = false;              // multicast mapping exists for the control segment
  size_t ll_slot_bytes = 0;       // capacity of one LL inbox slot (payload is half of it)
  size_t inbox_slot_bytes = 0;    // capacity of one one-shot inbox slot
  size_t stage_bytes = 0;         // capacity of stage_a and of stage_b
  int sm_count = 148;
};

struct Thresholds {
  size_t ll_max = 0;       // wire bytes <= ll_max        -> LL
  size_t oneshot_max = 0;  // wire bytes <= oneshot_max   -> one-shot
  size_t nvls_min = 0;     // wire bytes >= nvls_min (and NVLS usable) -> NVLS, else two-shot
};

// Built-in crossovers for a rank count (measured on 8xB200 NVSwitch; see the
// benchmark sweep), adjusted by the config overrides.
Thresholds thresholds_for(int nranks, const Config& cfg, bool symmetric = true);
// Default capacities of the inbox slots for a rank count.
size_t default_ll_slot_bytes(int nranks, const Config& cfg);
size_t default_inbox_slot_bytes(int nranks, const Config& cfg);

struct PlanInput {
  Mode mode = Mode::AllReduce;
  uint64_t count = 0;  // AllReduce: total elements; RS / AG: elements per rank
  DType in = DType::Float32, wire = DType::Float32, out = DType::Float32;
  RedOp op = RedOp::Sum;
  bool in_symmetric = false;   // send buffer lies in symmetric memory (16-byte aligned)
  bool out_symmetric = false;  // recv buffer lies in symmetric memory (16-byte aligned)
  bool in_has_mc = false, out_has_mc = false;  // those segments have multicast mappings
  bool host_memory = false;     // a buffer is pinned host memory (never taken by the pipelined kernel)
  bool auto_eligible = false;  // both buffers are ordinary device memory of one type and lazy direct access is on:
                               // the two-shot kernel can run on them directly once every rank has mapped them
  Algo forced = Algo::Auto;
};

struct Plan {
  LaunchSpec spec;
  uint64_t shard_elems = 0;
  uint64_t chunk_shard_vecs = 0;
  bool copy_in = false, copy_out = false;
  int pipe_ramp = 0;           // pipelined kernel: small first chunks (shard_elems is divisible by vector width << pipe_ramp)
  bool valid = false;
  const char* reason = "";  // why the plan is invalid
};

// Throws nothing; returns plan.valid == false when no kernel can serve the
// request (caller falls back or reports InvalidArgument).
Plan make_plan(const PlanInput& in, const CommCaps& caps, const Config& cfg);

Algo parse_algo(const std::string& s);

// Element counts of the chunks the pipeline cuts a message of `count` elements into.
// `uniform_elems`: the regular chunk (a multiple of 4096 elements, > 0).  `taper`: the first and the
// last chunk are small (an eighth of the message, 8 to 32 MB) so that the copy-in nobody can hide
// and the copy-out after the last collective are short, and the chunks between them are as large as
// `cap_elems` allows (large collectives run closer to the link rate).  Every chunk but the last is a
// multiple of 4096 elements; the sum is `count`.
std::vector<size_t> pipeline_chunks(size_t count, size_t elem_bytes, size_t uniform_elems, size_t cap_elems, bool taper);


}  // namespace mnccl
