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
template <typename InT, typename WireT, typename OutT, int OP, bool NVLS, int MODE, int kUnroll = 4>
__device__ __forceinline__ void twoshot_body(const KParams& P, int blk, int nblk, BlockCtl& ctl) {
  const CommDev& c = P.comm;
  const CollArgs& a = P.args;
  using Acc = typename Elem<WireT>::Acc;
  using OAcc = typename Elem<OutT>::Acc;
  constexpr int VW = 16 / sizeof(typename Elem<WireT>::Raw);
  constexpr int OUT_VB = VW * sizeof(typename Elem<OutT>::Raw);  // bytes of one output vector
  block_begin(c, blk, ctl);
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
            *reinterpret_cast<uint4*>(a.in_peer[me] + (uint64_t(j) * SV + i) * 16) = pk.vec.q[0];
          }
        }
      }
    }
    // Barrier 1: every rank's inputs are in place, and every rank has left the
    // previous pass (so its staging / receive buffers may be written again).
    ok = block_barrier(c, blk, ctl);
    if (!ok) break;

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
              char* dst = a.out_mc + (uint64_t(me) * SV + i) * OUT_VB;
#pragma unroll
              for (int q = 0; q < OUT_VB / 16; ++q) multimem_st_v4(dst + q * 16, pk.vec.q[q]);
            } else {
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
    ok = block_barrier(c, blk, ctl);
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
            OAcc y[VW];
            load_vec<OutT, VW>(a.out_peer[me] + (uint64_t(j) * SV + i) * OUT_VB, 0, VW, true, y);
            store_vec<OutT, VW>(a.recv, e0, lim, recv_al, y);
          }
        }
      }
    }
  }
  block_end(c, blk, nblk, ctl);
}

}  // namespace dev
}  // namespace mnccl
