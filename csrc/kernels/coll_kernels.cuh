// Collective kernels for one NVSwitch node, sm_100a.  Four AllReduce variants
// share one set of building blocks:
//
//   LL        one-shot push; every 8 bytes of payload travel with two copies of
//             a per-call flag in one 16-byte store, the receiver polls the data
//             itself.  No barrier, one NVLink traversal.  Tiny messages.
//   one-shot  push into per-source inboxes, one cross-rank barrier per block,
//             every rank reduces all N contributions itself.  Small messages.
//   two-shot  reduce-scatter by pulling a shard from every peer (128-bit P2P
//             loads), all-gather by pushing the reduced shard to every peer.
//   NVLS      the same split, but the switch does the work: multimem.ld_reduce
//             reads the sum of all ranks' copies, multimem.st writes all ranks.
//
// Inputs that are not in symmetric memory are staged (copy_in), outputs
// likewise (copy_out); symmetric buffers are used in place (zero-copy).
// Reductions accumulate in fp32 (fp64 / integer for those types) in rank order
// 0..N-1, except NVLS where the switch defines the order.  A conversion
// InT -> WireT -> OutT and a scale factor are fused in.
//
// These kernels replace the reference's per-slice trio of launches
// (wait_kernel, elementwise_reduce_kernel, cudaMemcpyAsync + set_flag_kernel;
// reference: src/mini_nccl.cu:108-194): one launch per collective, flags
// polled from device memory inside the kernel, every wait bounded.
//
// Work split.  Vectors (16 bytes of wire type) of a shard are grouped in tiles
// of blockDim.x * UNROLL; tile k belongs to block k % nblk on every rank, in
// every phase.  Hence block b of one rank only ever consumes data produced by
// block b of the other ranks, and the cross-rank barrier is per block index.
#pragma once
#include <cstddef>
#include <type_traits>

#include "kernels/dev_prims.cuh"

namespace mnccl {
namespace dev {

enum CollMode : int { kAllReduce = 0, kReduceScatter = 1, kAllGather = 2 };

// -------------------------------------------------------------------- N == 1
template <typename InT, typename OutT>
__device__ __forceinline__ void local_body(const KParams& P, int blk, int nblk) {
  const CollArgs& a = P.args;
  constexpr int VW = 16 / sizeof(typename Elem<InT>::Raw) < 16 / sizeof(typename Elem<OutT>::Raw)
                         ? 16 / sizeof(typename Elem<InT>::Raw)
                         : 16 / sizeof(typename Elem<OutT>::Raw);
  const bool in_al = vec_aligned<InT, VW>(a.send), out_al = vec_aligned<OutT, VW>(a.recv);
  const uint64_t nvec = (a.count + VW - 1) / VW;
  // Four vectors in flight per thread: a copy is bound by how many loads are outstanding.
  constexpr int U = 4;
  const uint64_t stride = uint64_t(nblk) * blockDim.x;
  for (uint64_t v0 = uint64_t(blk) * blockDim.x + threadIdx.x; v0 < nvec; v0 += U * stride) {
    typename Elem<InT>::Acc x[U][VW];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t v = v0 + u * stride;
      if (v < nvec) load_vec<InT, VW>(a.send, v * VW, a.count, in_al, x[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t v = v0 + u * stride;
      if (v >= nvec) continue;
      typename Elem<OutT>::Acc y[VW];
#pragma unroll
      for (int k = 0; k < VW; ++k) y[k] = finalize<OutT>(static_cast<typename Elem<OutT>::Acc>(x[u][k]), a);
      store_vec<OutT, VW>(a.recv, v * VW, a.count, out_al, y);
    }
  }
}

// -------------------------------------------------------------------- host-synchronised reduction
// out = scale * op over ranks of in_peer[r][0 .. count), in rank order, fp32 accumulation.  No flag, no
// wait, no control segment: the HOST orders the ranks (staging filled, barrier, this kernel, barrier).
// This is the data plane for ranks that share one GPU, where kernels of different processes can never
// be assumed to run at the same time and so must not wait for one another.
template <typename InT, typename WireT, typename OutT, int OP>
__device__ __forceinline__ void gather_reduce_body(const KParams& P, int blk, int nblk) {
  const CollArgs& a = P.args;
  const int N = P.comm.nranks;
  using Acc = typename Elem<WireT>::Acc;
  constexpr int VW = 16 / sizeof(typename Elem<WireT>::Raw);
  constexpr int U = 4;
  const bool out_al = vec_aligned<OutT, VW>(a.recv);
  const uint64_t nvec = (a.count + VW - 1) / VW;
  const uint64_t stride = uint64_t(nblk) * blockDim.x;
  for (uint64_t v0 = uint64_t(blk) * blockDim.x + threadIdx.x; v0 < nvec; v0 += U * stride) {
    Acc acc[U][VW];
    for (int r = 0; r < N; ++r) {
      uint4 got[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t v = v0 + u * stride;
        got[u] = make_uint4(0, 0, 0, 0);
        if (v < nvec) got[u] = ld_cg_v4(a.in_peer[r] + v * 16);  // staging is rewritten between calls by other processes
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        Packed<WireT, VW> in;
        in.vec.q[0] = got[u];
        Acc val[VW];
        in.to_acc(val);
#pragma unroll
        for (int k = 0; k < VW; ++k) acc[u][k] = (r == 0) ? val[k] : combine<OP>(acc[u][k], val[k]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t v = v0 + u * stride;
      if (v >= nvec) continue;
      typename Elem<OutT>::Acc y[VW];
#pragma unroll
      for (int k = 0; k < VW; ++k) y[k] = finalize<OutT>(static_cast<typename Elem<OutT>::Acc>(acc[u][k]), a);
      store_vec<OutT, VW>(a.recv, v * VW, a.count, out_al, y);
    }
  }
}

// -------------------------------------------------------------------- LL
template <typename InT, typename WireT, typename OutT, int OP>
__device__ __forceinline__ void ll_body(const KParams& P, int blk, int nblk, BlockCtl& ctl) {
  const CommDev& c = P.comm;
  const CollArgs& a = P.args;
  using Acc = typename Elem<WireT>::Acc;
  using WRaw = typename Elem<WireT>::Raw;
  constexpr int EPU = 8 / sizeof(WRaw);  // elements per 8-byte unit
  block_begin(c, blk, ctl);
  const int N = c.nranks, me = c.rank;
  uint32_t flag = ctl.ll_seq + 1;
  if (flag == 0) flag = 1;
  const uint32_t par = flag & 1u;
  const uint64_t units = (a.count + EPU - 1) / EPU;
  const bool in_al = vec_aligned<InT, EPU>(a.send);
  const bool out_al = vec_aligned<OutT, EPU>(a.recv);
  char* my_ll = c.ctrl[me] + c.off_ll;
  uint32_t fail = 0;
  for (uint64_t u = uint64_t(blk) * blockDim.x + threadIdx.x; u < units; u += uint64_t(nblk) * blockDim.x) {
    typename Elem<InT>::Acc x[EPU];
    load_vec<InT, EPU>(a.send, u * EPU, a.count, in_al, x);
    Acc mine[EPU];
#pragma unroll
    for (int k = 0; k < EPU; ++k) mine[k] = static_cast<Acc>(x[k]);
    Packed<WireT, EPU> pk;
    pk.from_acc(mine);
    pk.to_acc(mine);  // own contribution, rounded to the wire type like everyone else's
    const uint4 pkt = make_uint4(pk.w[0], flag, pk.w[1], flag);
    for (int k = 1; k < N; ++k) {
      const int p = (me + k) % N;
      char* dst = c.ctrl[p] + c.off_ll + (uint64_t(par) * N + me) * c.ll_slot_bytes + u * 16;
      st_volatile_v4(dst, pkt);
    }
    Acc acc[EPU];
    for (int r = 0; r < N; ++r) {
      Acc val[EPU];
      if (r == me) {
#pragma unroll
        for (int k = 0; k < EPU; ++k) val[k] = mine[k];
      } else {
        const char* src = my_ll + (uint64_t(par) * N + r) * c.ll_slot_bytes + u * 16;
        uint4 got = ld_volatile_v4(src);
        if (got.y != flag || got.w != flag) {
          const uint64_t t0 = globaltimer_ns();
          for (uint32_t it = 1;; ++it) {
            got = ld_volatile_v4(src);
            if (got.y == flag && got.w == flag) break;
            if ((it & 255u) == 0u) {
              if (c.abort_word != nullptr && ld_volatile_u32(c.abort_word) != 0u) { fail = kDevAborted; break; }
              if (globaltimer_ns() - t0 > c.spin_timeout_ns) { fail = kDevTimeout; break; }
            }
          }
          if (fail) {
            record_failure(c, fail, (uint32_t(blk) << 16) | uint32_t(r));
            break;
          }
        }
        Packed<WireT, EPU> in;
        in.w[0] = got.x;
        in.w[1] = got.z;
        in.to_acc(val);
      }
#pragma unroll
      for (int k = 0; k < EPU; ++k) acc[k] = (r == 0) ? val[k] : combine<OP>(acc[k], val[k]);
    }
    if (fail) break;
    typename Elem<OutT>::Acc y[EPU];
#pragma unroll
    for (int k = 0; k < EPU; ++k) y[k] = finalize<OutT>(static_cast<typename Elem<OutT>::Acc>(acc[k]), a);
    store_vec<OutT, EPU>(a.recv, u * EPU, a.count, out_al, y);
  }
  if (threadIdx.x == 0) ctl.ll_seq = flag;
  block_end(c, blk, nblk, ctl);
}

// -------------------------------------------------------------------- one-shot
template <typename InT, typename WireT, typename OutT, int OP>
__device__ __forceinline__ void oneshot_body(const KParams& P, int blk, int nblk, BlockCtl& ctl) {
  const CommDev& c = P.comm;
  const CollArgs& a = P.args;
  using Acc = typename Elem<WireT>::Acc;
  constexpr int VW = 16 / sizeof(typename Elem<WireT>::Raw);
  block_begin(c, blk, ctl);
  const int N = c.nranks, me = c.rank;
  const uint32_t par = (ctl.epoch + 1) & 1u;
  const uint64_t nvec = (a.count + VW - 1) / VW;
  const bool in_al = vec_aligned<InT, VW>(a.send), out_al = vec_aligned<OutT, VW>(a.recv);
  const uint64_t stride = uint64_t(nblk) * blockDim.x;
  const uint64_t first = uint64_t(blk) * blockDim.x + threadIdx.x;

  for (uint64_t v = first; v < nvec; v += stride) {
    typename Elem<InT>::Acc x[VW];
    load_vec<InT, VW>(a.send, v * VW, a.count, in_al, x);
    Acc w[VW];
#pragma unroll
    for (int k = 0; k < VW; ++k) w[k] = static_cast<Acc>(x[k]);
    Packed<WireT, VW> pk;
    pk.from_acc(w);
    for (int k = 0; k < N; ++k) {
      const int p = (me + k) % N;  // k == 0: own inbox, so that all N operands are read the same way
      char* dst = c.ctrl[p] + c.off_inbox + (uint64_t(par) * N + me) * c.inbox_slot_bytes + v * 16;
      *reinterpret_cast<uint4*>(dst) = pk.vec.q[0];
    }
  }
  if (block_barrier(c, blk, ctl)) {
    const char* inbox = c.ctrl[me] + c.off_inbox + uint64_t(par) * N * c.inbox_slot_bytes;
    for (uint64_t v = first; v < nvec; v += stride) {
      Acc acc[VW];
      for (int r = 0; r < N; ++r) {
        Packed<WireT, VW> in;
        in.vec.q[0] = *reinterpret_cast<const uint4*>(inbox + uint64_t(r) * c.inbox_slot_bytes + v * 16);
        Acc val[VW];
        in.to_acc(val);
#pragma unroll
        for (int k = 0; k < VW; ++k) acc[k] = (r == 0) ? val[k] : combine<OP>(acc[k], val[k]);
      }
      typename Elem<OutT>::Acc y[VW];
#pragma unroll
      for (int k = 0; k < VW; ++k) y[k] = finalize<OutT>(static_cast<typename Elem<OutT>::Acc>(acc[k]), a);
      store_vec<OutT, VW>(a.recv, v * VW, a.count, out_al, y);
    }
  }
  block_end(c, blk, nblk, ctl);
}

// -------------------------------------------------------------------- two-shot / NVLS
// One staging pass handles `sv` vectors of every shard, starting at vector
// `v0` of the shard.  Shard j covers elements [j*E, (j+1)*E) of the logical
// message; its vector i sits at element j*E + i*VW of user buffers and at
// vector (j*SV + i) of a staging buffer (SV = capacity per shard).
//
// twoshot_core is the body without the kernel prologue / epilogue: `sig_blk` is the block's index
// for the cross-rank barrier, (`blk`, `nblk`) its place among the blocks that share this message.
// They differ when one kernel serves two messages with two groups of blocks (the NVLS + peer-to-peer
// split of k_nvls.cu).
//
// `synced`: the caller has just passed a cross-rank barrier of its own and nothing is staged, so the
// first pass needs no barrier 1 (every rank's kernel has started: its inputs are in place; the previous
// call ended with a barrier).
template <typename InT, typename WireT, typename OutT, int OP, bool NVLS, int MODE, int kUnroll = 4>
__device__ __forceinline__ void twoshot_core(const CommDev& c, const CollArgs& a, int sig_blk, int blk, int nblk, BlockCtl& ctl,
                                             bool synced = false) {
  using Acc = typename Elem<WireT>::Acc;
  using OAcc = typename Elem<OutT>::Acc;
  constexpr int VW = 16 / sizeof(typename Elem<WireT>::Raw);
  constexpr int OUT_VB = VW * sizeof(typename Elem<OutT>::Raw);  // bytes of one output vector
  const int N = c.nranks, me = c.rank;
  const uint64_t E = a.shard_elems;
  const uint64_t total = (MODE == kAllReduce) ? a.count : E * uint64_t(N);  // logical message length
  const uint64_t shard_vecs = (E + VW - 1) / VW;
  const uint64_t SV = a.chunk_shard_vecs;  // vectors of a shard per pass (== shard_vecs when nothing is staged)
  const bool staged_in = a.copy_in != 0, staged_out = a.copy_out != 0;
  // Element-offset alignment of shard starts in user buffers.
  const bool shard_al_in = (E * sizeof(typename Elem<InT>::Raw)) % 16 == 0;
  const bool shard_al_out = (E * sizeof(typename Elem<OutT>::Raw)) % 16 == 0;
  const bool send_al = vec_aligned<InT, VW>(a.send) && shard_al_in;
  const bool recv_al = vec_aligned<OutT, VW>(a.recv) && shard_al_out;
  const uint64_t tile = uint64_t(blockDim.x) * kUnroll;
  bool ok = true;

  for (uint64_t v0 = 0; v0 < shard_vecs && ok; v0 += SV) {
    const uint64_t sv = (shard_vecs - v0 < SV) ? (shard_vecs - v0) : SV;
    const uint64_t ntiles = (sv + tile - 1) / tile;

    // ---- phase A: stage inputs (AllReduce / ReduceScatter)
    if (MODE != kAllGather && staged_in) {
      for (int j = 0; j < N; ++j) {
        for (uint64_t t = blk; t < ntiles; t += nblk) {
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const uint64_t i = t * tile + uint64_t(u) * blockDim.x + threadIdx.x;
            const uint64_t e0 = uint64_t(j) * E + (v0 + i) * VW;
            uint64_t lim = uint64_t(j) * E + E;
            if (lim > total) lim = total;
            if (i >= sv || e0 >= lim) continue;
            typename Elem<InT>::Acc x[VW];
            load_vec<InT, VW>(a.send, e0, lim, send_al, x);
            Acc w[VW];
#pragma unroll
            for (int k = 0; k < VW; ++k) w[k] = static_cast<Acc>(x[k]);
            Packed<WireT, VW> pk;
            pk.from_acc(w);
            if (!MNCCL_STAGE_OK(c, (uint64_t(j) * SV + i) * 16, 16)) continue;
            *reinterpret_cast<uint4*>(a.in_peer[me] + (uint64_t(j) * SV + i) * 16) = pk.vec.q[0];
          }
        }
      }
    }
    // Barrier 1: every rank's inputs are in place, and every rank has left the
    // previous pass (so its staging / receive buffers may be written again).
    if (!(synced && v0 == 0 && !staged_in)) {
      ok = block_barrier(c, sig_blk, ctl);
      if (!ok) break;
    }

    // ---- phase B: reduce my shard and hand the result out (AllGather: push my shard)
    if (MODE == kAllGather) {
      // `send` holds E elements; they become shard `me` of every rank's output.
      const bool src_al = vec_aligned<InT, VW>(a.send);
      for (uint64_t t = blk; t < ntiles; t += nblk) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const uint64_t i = t * tile + uint64_t(u) * blockDim.x + threadIdx.x;
          if (i >= sv) continue;
          const uint64_t e0 = (v0 + i) * VW;  // element inside the shard
          typename Elem<InT>::Acc x[VW];
          load_vec<InT, VW>(a.send, e0, E, src_al, x);
          OAcc y[VW];
#pragma unroll
          for (int k = 0; k < VW; ++k) y[k] = static_cast<OAcc>(x[k]);
          for (int k = 0; k < N; ++k) {
            const int p = (me + k) % N;
            if (staged_out) {
              if (!MNCCL_STAGE_OK(c, (uint64_t(me) * SV + i) * OUT_VB, OUT_VB)) continue;
              store_vec<OutT, VW>(a.out_peer[p] + (uint64_t(me) * SV + i) * OUT_VB, 0, VW, true, y);
            } else {
              store_vec<OutT, VW>(a.out_peer[p], uint64_t(me) * E + e0, uint64_t(me) * E + E, recv_al, y);
            }
          }
        }
      }
    } else {
      const uint64_t lim_me = (uint64_t(me) * E + E > total) ? total : uint64_t(me) * E + E;
      for (uint64_t t = blk; t < ntiles; t += nblk) {
        Acc acc[kUnroll][VW];
        bool valid[kUnroll];
        uint64_t off[kUnroll];  // byte offset of the input vector in every rank's input view
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const uint64_t i = t * tile + uint64_t(u) * blockDim.x + threadIdx.x;
          const uint64_t e0 = uint64_t(me) * E + (v0 + i) * VW;
          valid[u] = i < sv && e0 < lim_me;
          off[u] = staged_in ? (uint64_t(me) * SV + i) * 16 : e0 * sizeof(typename Elem<WireT>::Raw);
          if (staged_in && valid[u] && !MNCCL_STAGE_OK(c, off[u], 16)) valid[u] = false;
        }
        if constexpr (NVLS) {
          uint4 r[kUnroll];
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            r[u] = make_uint4(0, 0, 0, 0);
            if (valid[u]) r[u] = Nvls<WireT>::ld_reduce_add(a.in_mc + off[u]);
          }
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            Packed<WireT, VW> in;
            in.vec.q[0] = r[u];
            in.to_acc(acc[u]);
          }
        } else {
          for (int r = 0; r < N; ++r) {
            uint4 got[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
              got[u] = make_uint4(0, 0, 0, 0);
              if (valid[u]) got[u] = *reinterpret_cast<const uint4*>(a.in_peer[r] + off[u]);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
              Packed<WireT, VW> in;
              in.vec.q[0] = got[u];
              Acc val[VW];
              in.to_acc(val);
#pragma unroll
              for (int k = 0; k < VW; ++k) acc[u][k] = (r == 0) ? val[k] : combine<OP>(acc[u][k], val[k]);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (!valid[u]) continue;
          const uint64_t i = t * tile + uint64_t(u) * blockDim.x + threadIdx.x;
          OAcc y[VW];
#pragma unroll
          for (int k = 0; k < VW; ++k) y[k] = finalize<OutT>(static_cast<OAcc>(acc[u][k]), a);
          const uint64_t e0 = uint64_t(me) * E + (v0 + i) * VW;  // element in the logical message
          if (MODE == kReduceScatter) {
            // my reduced shard goes to my own recv buffer only
            store_vec<OutT, VW>(a.recv, (v0 + i) * VW, E, vec_aligned<OutT, VW>(a.recv), y);
          } else if (staged_out) {
            if constexpr (NVLS) {
              static_assert(OUT_VB % 16 == 0, "NVLS output vectors are whole 16-byte units");
              Packed<OutT, VW> pk;
              pk.from_acc(y);
              if (!MNCCL_STAGE_OK(c, (uint64_t(me) * SV + i) * OUT_VB, OUT_VB)) continue;
              char* dst = a.out_mc + (uint64_t(me) * SV + i) * OUT_VB;
#pragma unroll
              for (int q = 0; q < OUT_VB / 16; ++q) multimem_st_v4(dst + q * 16, pk.vec.q[q]);
            } else {
              if (!MNCCL_STAGE_OK(c, (uint64_t(me) * SV + i) * OUT_VB, OUT_VB)) continue;
              for (int k = 0; k < N; ++k) {
                const int p = (me + k) % N;
                store_vec<OutT, VW>(a.out_peer[p] + (uint64_t(me) * SV + i) * OUT_VB, 0, VW, true, y);
              }
            }
          } else {
            // zero-copy into every rank's recv buffer (16-byte aligned by contract)
            bool done = false;
            if constexpr (NVLS) {
              if (e0 + VW <= lim_me) {
                Packed<OutT, VW> pk;
                pk.from_acc(y);
                char* dst = a.out_mc + e0 * sizeof(typename Elem<OutT>::Raw);
#pragma unroll
                for (int q = 0; q < OUT_VB / 16; ++q) multimem_st_v4(dst + q * 16, pk.vec.q[q]);
                done = true;
              }
            }
            if (!done) {
              for (int k = 0; k < N; ++k) {
                const int p = (me + k) % N;
                store_vec<OutT, VW>(a.out_peer[p], e0, lim_me, true, y);
              }
            }
          }
        }
      }
    }
    ok = block_barrier(c, sig_blk, ctl);
    if (!ok) break;

    // ---- phase C: copy staged outputs to the user buffer
    if (MODE != kReduceScatter && staged_out) {
      for (int j = 0; j < N; ++j) {
        for (uint64_t t = blk; t < ntiles; t += nblk) {
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const uint64_t i = t * tile + uint64_t(u) * blockDim.x + threadIdx.x;
            const uint64_t e0 = uint64_t(j) * E + (v0 + i) * VW;
            uint64_t lim = uint64_t(j) * E + E;
            if (lim > total) lim = total;
            if (i >= sv || e0 >= lim) continue;
            if (!MNCCL_STAGE_OK(c, (uint64_t(j) * SV + i) * OUT_VB, OUT_VB)) continue;
            OAcc y[VW];
            load_vec<OutT, VW>(a.out_peer[me] + (uint64_t(j) * SV + i) * OUT_VB, 0, VW, true, y);
            store_vec<OutT, VW>(a.recv, e0, lim, recv_al, y);
          }
        }
      }
    }
  }
}

template <typename InT, typename WireT, typename OutT, int OP, bool NVLS, int MODE, int kUnroll = 4>
__device__ __forceinline__ void twoshot_body(const KParams& P, int blk, int nblk, BlockCtl& ctl) {
  block_begin(P.comm, blk, ctl);
  twoshot_core<InT, WireT, OutT, OP, NVLS, MODE, kUnroll>(P.comm, P.args, blk, blk, nblk, ctl);
  block_end(P.comm, blk, nblk, ctl);
}

// -------------------------------------------------------------------- two-shot with lazy direct access
// The peer-to-peer two-shot AllReduce on ORDINARY device buffers (one type, any operator).  Planned
// as the staged kernel (P.args: copy_in = copy_out = 1, staging views, passes of chunk_shard_vecs).
// Before the first pass the ranks find out, inside the kernel and with one extra barrier, whether
// every rank can reach every rank's buffers of this call directly (see AutoDesc); if so the same core
// runs once over the user buffers themselves: no copy-in, no copy-out, no passes.  All blocks of a
// rank decide alike, because everything the decision rests on travels by value with the launch.
template <typename T, int OP>
__device__ __forceinline__ void twoshot_auto_body(const KParams& P, int blk, int nblk, BlockCtl& ctl) {
  __shared__ CollArgs direct;
  __shared__ AutoDesc s_desc[kAutoRanks];
  const CommDev& c = P.comm;
  const CollArgs& a = P.args;
  const int t = threadIdx.x, N = c.nranks, me = c.rank;
  block_begin(c, blk, ctl);
  const AutoCtl* mine = reinterpret_cast<const AutoCtl*>(c.ctrl[me] + c.off_auto);
  if (t < N && t != me) {
    // 48 bytes as three 16-byte stores; the same thread releases this peer's barrier flag afterwards
    uint4* dst = reinterpret_cast<uint4*>(&reinterpret_cast<AutoCtl*>(c.ctrl[t] + c.off_auto)->desc[blk][me]);
    const uint4* src = reinterpret_cast<const uint4*>(&a.auto_desc);
    dst[0] = src[0];
    dst[1] = src[1];
    dst[2] = src[2];
  }
  if (t == 0) direct = a;
  bool ok = block_barrier(c, blk, ctl);
  bool agreed = false;
  if (ok && N <= kAutoRanks && c.auto_map != nullptr) {
    if (t < N) {
      if (t == me) {
        s_desc[t] = a.auto_desc;
      } else {
        const uint4* src = reinterpret_cast<const uint4*>(&mine->desc[blk][t]);
        uint4* dst = reinterpret_cast<uint4*>(&s_desc[t]);
        dst[0] = __ldcg(src);
        dst[1] = __ldcg(src + 1);
        dst[2] = __ldcg(src + 2);
      }
    }
    __syncthreads();
    // every rank evaluates the same words: rank q must have the slots of rank r's two buffers
    agreed = true;
    for (int r = 0; r < N; ++r) {
      const uint32_t sl = s_desc[r].slots;
      if (((sl >> 16) & 1u) == 0u) {
        agreed = false;
        break;
      }
      const uint32_t need = (1u << (sl & 15u)) | (1u << ((sl >> 8) & 15u));
      for (int q = 0; q < N; ++q)
        if (q != r && (s_desc[q].mask[r] & need) != need) agreed = false;
    }
    if (agreed) {
      // warp 0 resolves the peers' send buffers, warp 1 their recv buffers
      const int role = t >> 5, r = t & 31;
      if (role < 2 && r < N) {
        char* p = role == 0 ? static_cast<char*>(const_cast<void*>(a.send)) : static_cast<char*>(a.recv);
        if (r != me) {
          const uint32_t slot = (s_desc[r].slots >> (8 * role)) & 0xffu;
          const uint64_t addr = role == 0 ? s_desc[r].send_addr : s_desc[r].recv_addr;
          const uint4* e = reinterpret_cast<const uint4*>(c.auto_map + r * kAutoSlots + slot);
          const uint4 lo = __ldcg(e), hi = __ldcg(e + 1);
          const uint64_t base = (uint64_t(lo.w) << 32) | lo.z;
          const uint64_t local = (uint64_t(hi.w) << 32) | hi.z;
          p = reinterpret_cast<char*>(local + (addr - base));
        }
        if (role == 0) direct.in_peer[r] = p; else direct.out_peer[r] = p;
      }
      if (t == 64) {
        direct.copy_in = 0;
        direct.copy_out = 0;
        direct.in_mc = nullptr;
        direct.out_mc = nullptr;
        constexpr uint64_t VW = 16 / sizeof(typename Elem<T>::Raw);
        direct.chunk_shard_vecs = (a.shard_elems + VW - 1) / VW;
      }
      if (blk == 0 && t == 96) {   // calls that ran on the user buffers directly (statistics)
        const uint32_t n = atomicAdd(&local_state(c)->pad[0], 1u) + 1u;
        if (c.host_progress) c.host_progress[6] = n;
      }
      __syncthreads();
    }
  }
  // direct: the agreement's barrier stands in for the core's first one
  if (ok) twoshot_core<T, T, T, OP, false, kAllReduce>(c, agreed ? direct : a, blk, blk, nblk, ctl, agreed);
  block_end(c, blk, nblk, ctl);
}

// -------------------------------------------------------------------- pipelined (ordinary buffers)
// AllReduce of buffers that are NOT in symmetric memory, as ONE kernel whose blocks take three
// roles that run concurrently on different chunks of the message:
//
//   copy-in   user send buffer -> my stage_a slot (converted to the wire type)
//   reduce    my shard of the chunk: sum of all ranks' stage_a slots (multimem.ld_reduce through
//             the switch, or 128-bit peer loads in rank order) -> every rank's stage_b slot
//             (multimem.st, or peer stores), scale and output conversion fused in
//   copy-out  my stage_b slot -> user recv buffer
//
// The staging areas are rings of kPipeSlots slots.  Chunks are dealt round-robin to the blocks of a
// role: block b of a role with n blocks handles chunks b, b + n, b + 2n, ... ONE block per chunk, so
// every block streams through its own chunks with its loads in flight all the time and the blocks
// never meet.  (A first version let all blocks of a role share every chunk: each warp then touched
// every chunk, a chunk cost at least one load round trip of ~9 us whatever its size, and most lanes
// of a pass idled.)  The copies of later and earlier chunks overlap the reduction, so the NVLink
// transfer never waits for a local copy: a staged two-phase kernel idles the links during both
// copies, separate copy kernels on side streams pay a launch and a cross-rank barrier per chunk.
//
// Hand-over between roles and ranks is by monotonic chunk numbers (PipeCtl): chunk g, counted over
// ALL pipelined calls of the communicator, lives in slot g % kPipeSlots and its flags carry g + 1,
// so nothing is ever reset.  The block that finishes a chunk publishes "chunk g done by rank r" to
// every rank; waits are bounded like every other wait of the library.
//
//   copy-in  of chunk g waits for red_done[g - K] of all ranks   (the slot's last readers)
//   reduce   of chunk g waits for in_ready[g] of all ranks       (the data)
//                         and for out_done[g - K] of all ranks   (stage_b slots free everywhere)
//   copy-out of chunk g waits for red_done[g] of all ranks
//
// Inside a block, warp 0 publishes and warp 1 polls; the other warps work and never stall on either:
// a worker warp that has finished its part of a chunk bumps a counter in shared memory and goes on
// to the block's next chunk as soon as the poller has seen its inputs (at most kPipeAhead chunks
// ahead of the publisher).
//
// Chunk geometry: a chunk is N shards of E = a.shard_elems elements (a multiple of the vector
// width); rank r reduces shard r of every chunk.  Inside a slot the chunk is laid out like the
// user buffer, so both copies are straight copies.  On the peer-to-peer path a rank's OWN shard
// never touches the staging areas: the reduction reads it from the user's send buffer and writes the
// result straight into the user's recv buffer, and both copies skip it (with two ranks that halves
// the copy traffic).  The switch path cannot do that: multimem.ld_reduce reads the same offset of
// every rank's staging, the reader's own included.
constexpr int kPipeAhead = 4;  // chunks of one block whose completion may be outstanding; size of BlockCtl::pipe_done

// Chunk geometry with a ramp: the first R chunks are CE / 2^R, CE / 2^(R-1), ... CE / 2 elements, the
// rest CE each.  The first chunk's way through the three roles (copy, flags, reduce, flags, copy) is
// what the whole message waits for at the start; a small first chunk shortens it (measured: the
// pipelined kernel took a constant ~60 us more than the zero-copy one with uniform 512 KB chunks).
__host__ __device__ __forceinline__ void pipe_chunk_geom(uint32_t ch, uint64_t CE, uint32_t R, uint64_t* begin, uint64_t* size) {
  if (ch < R) {
    const uint64_t unit = CE >> R;
    *begin = unit * ((uint64_t(1) << ch) - 1);
    *size = unit << ch;
  } else {
    *begin = (CE >> R) * ((uint64_t(1) << R) - 1) + uint64_t(ch - R) * CE;
    *size = CE;
  }
}
__host__ __device__ __forceinline__ uint32_t pipe_chunk_count(uint64_t count, uint64_t CE, uint32_t R) {
  uint32_t n = 0;
  uint64_t begin = 0, size = 0;
  for (; n < R; ++n) {
    pipe_chunk_geom(n, CE, R, &begin, &size);
    if (begin >= count) return n;
  }
  pipe_chunk_geom(R, CE, R, &begin, &size);
  if (begin >= count) return R;
  return R + static_cast<uint32_t>((count - begin + CE - 1) / CE);
}

template <int NVLS>
__device__ __forceinline__ void pipe_roles(int nblk, int& n_in, int& n_red) {
  // switch path: the reduction needs fewer blocks than peer-to-peer loads and stores
  const int share = NVLS ? 3 : 2;
  n_in = (nblk * share + 5) / 10;
  if (n_in < 1) n_in = 1;
  n_red = nblk - 2 * n_in;
  if (n_red < 1) n_red = 1;
}

// Publisher: makes the block's writes visible (ONE system-scope fence: local, peer and multicast
// stores), then plain system-scope stores of the chunk number into flags[slot][me] of every rank.  (A
// release store per peer would wait for the previous peer's flag to be acknowledged across NVLink
// every time: measured ~30 us per chunk on 8 GPUs.)
__device__ __forceinline__ void pipe_publish(const CommDev& c, int slot, size_t flag_off, uint32_t value) {
  __threadfence_system();
  for (int k = 0; k < c.nranks; ++k) {
    const int p = (c.rank + k) % c.nranks;
    uint32_t* f = reinterpret_cast<uint32_t*>(c.ctrl[p] + c.off_pipe + flag_off) + slot * kMaxRanks + c.rank;
    st_volatile_u32(f, value);
  }
}

// Poller: lane t < nranks waits for flags[slot][t] >= target with the bounded system-scope wait.
// Worker warps never touch the flags (a thousand warps polling them, and the abort word in host
// memory behind them, was measured to slow the kernel a hundredfold).
__device__ __forceinline__ bool pipe_poll_all(const CommDev& c, BlockCtl& ctl, size_t flag_off, int slot, uint32_t target,
                                              int blk) {
  const int lane = threadIdx.x & 31;
  if (lane < c.nranks) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(c.ctrl[c.rank] + c.off_pipe + flag_off) + slot * kMaxRanks + lane;
    const uint32_t r = wait_ge(f, target, c);
    if (r != kDevOk) {
      ctl.fail = r;
      record_failure(c, r, (static_cast<uint32_t>(blk) << 16) | static_cast<uint32_t>(lane));
    }
  }
  __syncwarp();
  return ctl.fail == 0;
}

// Spin on a counter in shared memory until it exceeds `want_above` (bounded; ctl.fail ends it).
__device__ __forceinline__ bool pipe_spin(const CommDev& c, BlockCtl& ctl, const volatile uint32_t* counter, uint32_t want_above) {
  if (*counter <= want_above) {
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 1; *counter <= want_above; ++it) {
      if (ctl.fail != 0) return false;
      if ((it & 4095u) == 0u && globaltimer_ns() - t0 > 2 * c.spin_timeout_ns) {  // the poller gives up first
        ctl.fail = kDevTimeout;
        return false;
      }
    }
  }
  return true;
}

// A worker warp has issued all its loads and stores of the block's i-th chunk.
__device__ __forceinline__ void pipe_warp_done(BlockCtl& ctl, uint32_t i) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) {
    __threadfence_block();
    atomicAdd(const_cast<uint32_t*>(&ctl.pipe_done[i % kPipeAhead]), 1u);
  }
}

template <typename InT, typename WireT, typename OutT, int OP, bool NVLS>
__device__ __forceinline__ void pipe_body(const KParams& P, int blk, int nblk, BlockCtl& ctl) {
  const CommDev& c = P.comm;
  const CollArgs& a = P.args;
  using Acc = typename Elem<WireT>::Acc;
  using OAcc = typename Elem<OutT>::Acc;
  using WRaw = typename Elem<WireT>::Raw;
  using ORaw = typename Elem<OutT>::Raw;
  constexpr int VW = 16 / sizeof(WRaw);
  constexpr int OUT_VB = VW * sizeof(ORaw);
  static_assert(OUT_VB % 16 == 0, "output vectors are whole 16-byte units for every supported type triple");
  // Vectors in flight per thread in the reduction and in the two copies.  The switch form keeps its
  // arrays in registers (126 of the 128 a 512-thread block may use, no spills).
  constexpr int U = 4;
  constexpr int UC = (NVLS && OUT_VB == 16) ? 16 : 8;
  constexpr bool kSameIn = std::is_same<InT, WireT>::value;
  block_begin(c, blk, ctl);
  const int N = c.nranks, me = c.rank;
  const int nwork = static_cast<int>(blockDim.x) - 64;     // worker threads (warps 2..); warp 0 publishes, warp 1 polls
  const int wt = static_cast<int>(threadIdx.x) - 64;       // index among the workers; negative in the two control warps
  if (N > 0 && a.count > 0 && nwork >= 32) {
    PipeCtl* pc = reinterpret_cast<PipeCtl*>(c.ctrl[me] + c.off_pipe);
    const uint32_t base = pc->base;  // written only by the last block of a call, after everyone read it
    const uint64_t E = a.shard_elems;
    const uint64_t CE = E * uint64_t(N);              // elements per chunk
    const uint32_t ramp = static_cast<uint32_t>(a.pipe_ramp);
    const uint32_t nchunks = pipe_chunk_count(a.count, CE, ramp);
    const uint64_t stride = c.stage_bytes / kPipeSlots;  // bytes per slot in both staging areas
    constexpr size_t kOffIn = offsetof(PipeCtl, in_ready), kOffRed = offsetof(PipeCtl, red_done),
                     kOffOut = offsetof(PipeCtl, out_done);
    int n_in, n_red;
    pipe_roles<NVLS ? 1 : 0>(nblk, n_in, n_red);
    const int n_out = nblk - n_in - n_red;
    const int role = blk < n_in ? 0 : (blk < n_in + n_red ? 1 : 2);
    const uint32_t rb = static_cast<uint32_t>(role == 0 ? blk : (role == 1 ? blk - n_in : blk - n_in - n_red));
    const uint32_t nrb = static_cast<uint32_t>(role == 0 ? n_in : (role == 1 ? n_red : n_out));
    // this block's chunks: rb, rb + nrb, ...; `i` counts them
    const uint32_t mine_n = rb < nchunks ? (nchunks - rb + nrb - 1) / nrb : 0;
    const uint64_t tile = uint64_t(nwork) * U;
    const uint64_t ctile = uint64_t(nwork) * UC;
    char* my_a = c.ctrl[me] + c.off_stage_a;
    char* my_b = c.ctrl[me] + c.off_stage_b;

    if (wt < -32) {
      // ---------------------------------------------------------------- publisher (warp 0, lane 0)
      if (threadIdx.x == 0) {
        const uint32_t warps = static_cast<uint32_t>(nwork / 32);
        const size_t flag_off = role == 0 ? kOffIn : (role == 1 ? kOffRed : kOffOut);
        for (uint32_t i = 0; i < mine_n; ++i) {
          if (!pipe_spin(c, ctl, &ctl.pipe_done[i % kPipeAhead], warps - 1)) {
            if (ctl.fail == kDevTimeout) record_failure(c, kDevTimeout, (static_cast<uint32_t>(blk) << 16) | 0xffffu);
            break;
          }
          ctl.pipe_done[i % kPipeAhead] = 0;  // counted into again only by chunk i + kPipeAhead, which waits for pipe_pub
          const uint32_t g = base + rb + i * nrb;
          pipe_publish(c, static_cast<int>(g % kPipeSlots), flag_off, g + 1);
          ctl.pipe_pub = i + 1;
        }
      }
    } else if (wt < 0) {
      // ---------------------------------------------------------------- poller (warp 1)
      for (uint32_t i = 0; i < mine_n; ++i) {
        const uint32_t g = base + rb + i * nrb;
        const int slot = static_cast<int>(g % kPipeSlots);
        const bool reuse = g >= static_cast<uint32_t>(kPipeSlots);
        bool ok = true;
        if (role == 0) {
          if (reuse) ok = pipe_poll_all(c, ctl, kOffRed, slot, g - kPipeSlots + 1, blk);
        } else if (role == 1) {
          ok = pipe_poll_all(c, ctl, kOffIn, slot, g + 1, blk);
          if (ok && reuse) ok = pipe_poll_all(c, ctl, kOffOut, slot, g - kPipeSlots + 1, blk);
        } else {
          ok = pipe_poll_all(c, ctl, kOffRed, slot, g + 1, blk);
        }
        if (!ok) break;
        if ((threadIdx.x & 31) == 0) {
          __threadfence_block();
          ctl.pipe_ready = i + 1;
        }
      }
    } else {
      // ---------------------------------------------------------------- workers
      const bool in_al = vec_aligned<InT, VW>(a.send);
      const bool out_al = vec_aligned<OutT, VW>(a.recv);
      for (uint32_t i = 0; i < mine_n; ++i) {
        // inputs seen by the poller, and not more than kPipeAhead - 1 chunks ahead of the publisher
        if (!pipe_spin(c, ctl, &ctl.pipe_ready, i)) break;
        if (i >= static_cast<uint32_t>(kPipeAhead - 1) && !pipe_spin(c, ctl, &ctl.pipe_pub, i - (kPipeAhead - 1))) break;
        __threadfence_block();  // acquire side of the poller's hand-over
        const uint32_t ch = rb + i * nrb;
        const uint32_t g = base + ch;
        const int slot = static_cast<int>(g % kPipeSlots);
        uint64_t cb, cs;                 // first element and length of this chunk
        pipe_chunk_geom(ch, CE, ramp, &cb, &cs);
        const uint64_t Ec = cs / uint64_t(N);  // shard length inside this chunk (a multiple of the vector width)
        if (role == 0) {
          // -------------------------------------------------------------- copy-in
          const uint64_t e_begin = cb;
          const uint64_t e_end = (e_begin + cs < a.count) ? e_begin + cs : a.count;
          const uint64_t nvec = (e_end - e_begin + VW - 1) / VW;
          char* dst = my_a + uint64_t(slot) * stride;
          const uint64_t full = (e_end - e_begin) / VW;  // vectors that lie wholly inside the chunk
          // peer-to-peer path: vectors [own_lo, own_hi) are my own shard, which is not staged
          const uint64_t own_lo = NVLS ? nvec : uint64_t(me) * (Ec / VW);
          const uint64_t own_hi = NVLS ? nvec : own_lo + Ec / VW;
          for (uint64_t v0 = wt; v0 < nvec; v0 += ctile) {
            if (v0 >= own_lo && v0 + uint64_t(UC - 1) * nwork < own_hi) continue;  // the whole step lies in my shard
            if (NVLS && kSameIn && in_al && v0 + uint64_t(UC - 1) * nwork < full) {
              // same type, aligned, no ragged end: move the bits
              const uint4* src = reinterpret_cast<const uint4*>(static_cast<const WRaw*>(a.send) + e_begin);
              uint4 x[UC];
#pragma unroll
              for (int u = 0; u < UC; ++u) x[u] = src[v0 + uint64_t(u) * nwork];
#pragma unroll
              for (int u = 0; u < UC; ++u) *reinterpret_cast<uint4*>(dst + (v0 + uint64_t(u) * nwork) * 16) = x[u];
              continue;
            }
            if (!NVLS && kSameIn && in_al && v0 + uint64_t(UC - 1) * nwork < full) {
              const uint4* src = reinterpret_cast<const uint4*>(static_cast<const WRaw*>(a.send) + e_begin);
              uint4 x[UC];
#pragma unroll
              for (int u = 0; u < UC; ++u) {
                const uint64_t v = v0 + uint64_t(u) * nwork;
                if (v < own_lo || v >= own_hi) x[u] = src[v];
              }
#pragma unroll
              for (int u = 0; u < UC; ++u) {
                const uint64_t v = v0 + uint64_t(u) * nwork;
                if (v < own_lo || v >= own_hi) *reinterpret_cast<uint4*>(dst + v * 16) = x[u];
              }
              continue;
            }
#pragma unroll 2
            for (int u = 0; u < UC; ++u) {
              const uint64_t v = v0 + uint64_t(u) * nwork;
              if (v >= nvec || (v >= own_lo && v < own_hi)) continue;
              typename Elem<InT>::Acc x[VW];
              load_vec<InT, VW>(a.send, e_begin + v * VW, e_end, in_al, x);
              Acc w[VW];
#pragma unroll
              for (int k = 0; k < VW; ++k) w[k] = static_cast<Acc>(x[k]);
              Packed<WireT, VW> pk;
              pk.from_acc(w);
              *reinterpret_cast<uint4*>(dst + v * 16) = pk.vec.q[0];
            }
          }
        } else if (role == 1) {
          // -------------------------------------------------------------- reduce my shard
          const uint64_t e_begin = cb + uint64_t(me) * Ec;  // my shard of this chunk
          uint64_t e_end = e_begin + Ec;
          if (e_end > a.count) e_end = a.count;
          const uint64_t nvec = e_begin < e_end ? (e_end - e_begin + VW - 1) / VW : 0;
          const uint64_t in_off = uint64_t(slot) * stride + uint64_t(me) * Ec * sizeof(WRaw);
          const uint64_t out_off = uint64_t(slot) * stride + uint64_t(me) * Ec * sizeof(ORaw);
          for (uint64_t v0 = wt; v0 < nvec; v0 += tile) {
            Acc acc[U][VW];
            if constexpr (NVLS) {
              uint4 r[U];
#pragma unroll
              for (int u = 0; u < U; ++u) {
                const uint64_t v = v0 + uint64_t(u) * nwork;
                r[u] = make_uint4(0, 0, 0, 0);
                if (v < nvec) r[u] = Nvls<WireT>::ld_reduce_add(c.ctrl_mc + c.off_stage_a + in_off + v * 16);
              }
#pragma unroll
              for (int u = 0; u < U; ++u) {
                Packed<WireT, VW> in;
                in.vec.q[0] = r[u];
                in.to_acc(acc[u]);
              }
            } else {
              for (int r = 0; r < N; ++r) {
                uint4 got[U];
                if (r == me) {
                  // my own contribution comes from the user's buffer, rounded to the wire type like everyone's
#pragma unroll
                  for (int u = 0; u < U; ++u) {
                    const uint64_t v = v0 + uint64_t(u) * nwork;
                    got[u] = make_uint4(0, 0, 0, 0);
                    if (v < nvec) {
                      typename Elem<InT>::Acc x[VW];
                      load_vec<InT, VW>(a.send, e_begin + v * VW, e_end, in_al, x);
                      Acc w[VW];
#pragma unroll
                      for (int k = 0; k < VW; ++k) w[k] = static_cast<Acc>(x[k]);
                      Packed<WireT, VW> pk;
                      pk.from_acc(w);
                      got[u] = pk.vec.q[0];
                    }
                  }
                } else {
                  const char* src = c.ctrl[r] + c.off_stage_a + in_off;
#pragma unroll
                  for (int u = 0; u < U; ++u) {
                    const uint64_t v = v0 + uint64_t(u) * nwork;
                    got[u] = make_uint4(0, 0, 0, 0);
                    // L2-only loads: the slot held another chunk earlier in this kernel, a line of it
                    // must not be served from this SM's L1
                    if (v < nvec) got[u] = ld_cg_v4(src + v * 16);
                  }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                  Packed<WireT, VW> in;
                  in.vec.q[0] = got[u];
                  Acc val[VW];
                  in.to_acc(val);
#pragma unroll
                  for (int k = 0; k < VW; ++k) acc[u][k] = (r == 0) ? val[k] : combine<OP>(acc[u][k], val[k]);
                }
              }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const uint64_t v = v0 + uint64_t(u) * nwork;
              if (v >= nvec) continue;
              OAcc y[VW];
#pragma unroll
              for (int k = 0; k < VW; ++k) y[k] = finalize<OutT>(static_cast<OAcc>(acc[u][k]), a);
              Packed<OutT, VW> pk;
              pk.from_acc(y);
              if constexpr (NVLS) {
                char* dst = c.ctrl_mc + c.off_stage_b + out_off + v * OUT_VB;
#pragma unroll
                for (int q = 0; q < OUT_VB / 16; ++q) multimem_st_v4(dst + q * 16, pk.vec.q[q]);
              } else {
                store_vec<OutT, VW>(a.recv, e_begin + v * VW, e_end, out_al, y);  // mine: straight to the user's buffer
                for (int k = 1; k < N; ++k) {
                  const int p = (me + k) % N;
                  char* dst = c.ctrl[p] + c.off_stage_b + out_off + v * OUT_VB;
#pragma unroll
                  for (int q = 0; q < OUT_VB / 16; ++q) reinterpret_cast<uint4*>(dst)[q] = pk.vec.q[q];
                }
              }
            }
          }
        } else {
          // -------------------------------------------------------------- copy-out
          const uint64_t e_begin = cb;
          const uint64_t e_end = (e_begin + cs < a.count) ? e_begin + cs : a.count;
          const uint64_t nvec = (e_end - e_begin + VW - 1) / VW;
          const char* src = my_b + uint64_t(slot) * stride;
          const uint64_t full = (e_end - e_begin) / VW;
          const uint64_t own_lo = NVLS ? nvec : uint64_t(me) * (Ec / VW);  // my shard is already in recv (peer-to-peer path)
          const uint64_t own_hi = NVLS ? nvec : own_lo + Ec / VW;
          for (uint64_t v0 = wt; v0 < nvec; v0 += ctile) {
            if (v0 >= own_lo && v0 + uint64_t(UC - 1) * nwork < own_hi) continue;
            if (out_al && v0 + uint64_t(UC - 1) * nwork < full) {
              constexpr int Q = OUT_VB / 16;
              uint4* dstv = reinterpret_cast<uint4*>(static_cast<ORaw*>(a.recv) + e_begin);
              uint4 y[UC][Q];
#pragma unroll
              for (int u = 0; u < UC; ++u) {
                const uint64_t v = v0 + uint64_t(u) * nwork;
                if (v < own_lo || v >= own_hi) {
#pragma unroll
                  for (int q = 0; q < Q; ++q) y[u][q] = ld_cg_v4(src + (v * Q + q) * 16);
                }
              }
#pragma unroll
              for (int u = 0; u < UC; ++u) {
                const uint64_t v = v0 + uint64_t(u) * nwork;
                if (v < own_lo || v >= own_hi) {
#pragma unroll
                  for (int q = 0; q < Q; ++q) dstv[v * Q + q] = y[u][q];
                }
              }
              continue;
            }
#pragma unroll 2
            for (int u = 0; u < UC; ++u) {
              const uint64_t v = v0 + uint64_t(u) * nwork;
              if (v >= nvec || (v >= own_lo && v < own_hi)) continue;
              Packed<OutT, VW> pk;
#pragma unroll
              for (int q = 0; q < OUT_VB / 16; ++q) pk.vec.q[q] = ld_cg_v4(src + v * OUT_VB + q * 16);
              OAcc y[VW];
              pk.to_acc(y);
              store_vec<OutT, VW>(a.recv, e_begin + v * VW, e_end, out_al, y);
            }
          }
        }
        pipe_warp_done(ctl, i);
      }
    }
    // the last block to leave moves the base past this call's chunks
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(&pc->finished, 1u) == static_cast<uint32_t>(nblk - 1)) {
        pc->finished = 0;
        pc->base = base + nchunks;
      }
    }
  }
  block_end(c, blk, nblk, ctl);
}

}  // namespace dev
}  // namespace mnccl
