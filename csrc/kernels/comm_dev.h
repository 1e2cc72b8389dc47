// Device-visible description of a communicator, shared by the library's own
// kernels and by user kernels that fuse a collective (obtained through
// mncclCommDeviceHandle).  Plain C structs: no constructors, fixed layout.
//
// Every rank owns one "control segment" of symmetric memory that all peers map
// (NVLink P2P).  Its layout, at the byte offsets stored below:
//
//   sig      [kMaxBlocks][kMaxRanks] u32   barrier signals written by peers
//   local    LocalState                    this rank's private counters
//   ll       [2][nranks][ll_slot_bytes]    one-shot "LL" inboxes (flag+data)
//   inbox    [2][nranks][inbox_slot_bytes] one-shot inboxes (barrier flavour)
//   pipe     PipeCtl                       chunk flags of the pipelined AllReduce
//   auto     AutoCtl                       per-call buffer descriptors and votes (lazy direct access)
//   stage_a  [stage_bytes]                 staged inputs  (wire type)
//   stage_b  [stage_bytes]                 staged outputs (output type)
//
// The reference keeps its flags and scratch in host-pinned memory that the GPU
// polls across PCIe and relaunches a one-thread wait kernel per slice
// (reference: src/mini_nccl.cu:22-36, src/transport/RDMATransport.h:113-123);
// here flags live in device memory of the rank that waits on them and every
// wait happens inside the data kernel.
#pragma once
#include <stdint.h>

namespace mnccl {

constexpr int kMaxRanks = 16;
constexpr int kMaxBlocks = 512;

// Status codes a kernel can leave in LocalState::status / host_progress[2].
enum DevStatus : uint32_t {
  kDevOk = 0,
  kDevTimeout = 1,   // a bounded wait ran out
  kDevAborted = 2,   // the abort word was set while waiting
  kDevBadIndex = 3,  // checked build only (MNCCL_DEVICE_CHECKS): a staging access fell outside its area or off alignment
};

struct LocalState {
  uint32_t epoch[kMaxBlocks];    // per-block barrier epoch (monotonic)
  uint32_t ll_seq[kMaxBlocks];   // word 0: the communicator's LL sequence (flag value source); the rest is unused
  uint32_t ticket;               // blocks finished in the running kernel
  uint32_t started;              // collectives started on this rank
  uint32_t done;                 // collectives finished on this rank
  uint32_t status;               // first failure (DevStatus), sticky
  uint32_t detail;               // (block << 16) | peer of the first failure
  uint32_t pad[3];
};

// Flags of the pipelined AllReduce on ordinary buffers (coll_kernels.cuh, pipe_body).  The staging
// areas are rings of kPipeSlots slots; chunk number g (counted over ALL pipelined calls of the
// communicator, so nothing is ever reset) lives in slot g % kPipeSlots and its flags carry g + 1.
// in_ready / red_done / out_done are written by every rank into every rank's copy (index: slot,
// then source rank); the base is private to the owner.
constexpr int kPipeSlots = 64;
struct PipeCtl {
  uint32_t in_ready[kPipeSlots][kMaxRanks];   // source rank has staged its input chunk
  uint32_t red_done[kPipeSlots][kMaxRanks];   // source rank has reduced its shard of the chunk into every stage_b
  uint32_t out_done[kPipeSlots][kMaxRanks];   // source rank has copied the chunk out of its stage_b
  uint32_t base;                              // number of chunks handled by earlier calls
  uint32_t finished;                          // blocks that have left the running call
  uint32_t pad[2];
};

// Lazy direct access to ordinary device buffers (coll_kernels.cuh, twoshot_auto_body).  A rank exports
// the allocations its buffers live in (CUDA IPC; export slots 0..kAutoSlots-1, never reused) and maps
// what its peers have exported; row [peer][slot] of a table in device memory says where that peer's
// slot is mapped here.  With every launch the host passes, by value, which slots of which peer it had
// mapped when it launched (a bit mask per peer) and which of its own slots hold this call's buffers.
// Inside the kernel every rank pushes that, with the buffers' addresses, into every peer's AutoCtl
// before ONE barrier; afterwards every rank holds every rank's word and all of them evaluate the same
// condition: "every rank has the slots of every other rank's buffers mapped".  Only then the kernel
// reads and writes the user buffers directly, otherwise it stages as before.  Nothing is agreed on
// the host, a rank that has not mapped a peer's buffer yet merely delays the switch, and what the
// host maps while a kernel runs cannot split that kernel's blocks (the masks travel by value).
constexpr int kAutoSlots = 16;        // exported allocations per rank
constexpr int kAutoRanks = 8;         // ranks the masks of one descriptor cover
constexpr int kAutoBlocks = 128;      // grid cap of the kernel (rows of AutoCtl)
struct AutoMapEntry {
  uint64_t id;          // allocation id in the exporting process (informative)
  uint64_t peer_base;   // its address range in the exporting process
  uint64_t size;
  uint64_t local_base;  // where this process mapped it
};
// What a rank tells every peer about one call.
struct alignas(16) AutoDesc {
  uint64_t send_addr, recv_addr;   // in the sender's address space
  uint32_t slots;                  // send slot | recv slot << 8 | usable << 16 (exported, in range, 16-byte aligned)
  uint32_t pad;
  uint16_t mask[kAutoRanks];       // mask[r]: export slots of rank r that the sender has mapped
  uint64_t pad2;
};
struct AutoCtl {
  AutoDesc desc[kAutoBlocks][kMaxRanks];   // [block][source rank], written by the peers
};

struct CommDev {
  int32_t rank;
  int32_t nranks;
  char* ctrl[kMaxRanks];          // control segment of every rank, as mapped here
  char* ctrl_mc;                  // multicast mapping of the control segment (NVLS) or null
  const volatile uint32_t* abort_word;  // host-mapped, shared by all local ranks; may be null
  volatile uint32_t* host_progress;     // host-mapped {started, done, status, detail}; may be null
  uint64_t spin_timeout_ns;       // budget of every device-side wait
  uint64_t off_sig, off_local, off_ll, off_inbox, off_stage_a, off_stage_b;
  uint64_t off_pipe;              // PipeCtl
  uint64_t ll_slot_bytes, inbox_slot_bytes, stage_bytes;
  uint64_t off_auto;              // AutoCtl
  const AutoMapEntry* auto_map;   // [kMaxRanks][kAutoSlots] in device memory, or null
};

// Arguments of one AllReduce / ReduceScatter / AllGather launch.
struct CollArgs {
  const void* send;
  void* recv;
  uint64_t count;            // AllReduce: elements; RS: recv elements per rank; AG: send elements per rank
  uint64_t shard_elems;      // elements per rank-shard inside the kernel (AllReduce: multiple of the vector width)
  uint64_t chunk_shard_vecs; // staged paths: vectors of one shard handled per staging pass
  float scale_f;             // post-reduction factor for fp16 / bf16 / fp32 (includes 1/N for Avg)
  int32_t int_div;           // integer Avg divisor (0 = none)
  double scale_d;            // same for fp64
  char* in_peer[kMaxRanks];  // input view on every rank: stage_a, or a symmetric user buffer (zero-copy)
  char* out_peer[kMaxRanks]; // output view on every rank: stage_b, or a symmetric user buffer
  char* in_mc;               // multicast views (NVLS) or null
  char* out_mc;
  int32_t copy_in;           // 1: inputs are first staged from `send`
  int32_t copy_out;          // 1: outputs are copied from stage_b to `recv`
  int32_t pipe_ramp;         // pipelined kernel: number of small first chunks (CE / 2^R ... CE / 2), see pipe_chunk_geom
  int32_t pad0;
  AutoDesc auto_desc;        // twoshot_auto_body: what this rank tells its peers about the call
};

struct KParams {
  CommDev comm;
  CollArgs args;
};

}  // namespace mnccl
