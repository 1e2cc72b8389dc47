"""Small single-GPU workloads for `ncu`: one kernel family per target, a few launches, inputs
larger than the L2 but far below a GB, so that a capture ends by itself within a minute or two.

  python benchmarks/profile_targets.py --target gemm        # tcgen05 GEMM, 4096 x 3584 x 4096, single-CTA tiles
  python benchmarks/profile_targets.py --target gemm_pair   # the same product on CTA pairs (cta_group::2)
  python benchmarks/profile_targets.py --target copy        # fused cast/scale copy kernel, 256 MiB
  python benchmarks/profile_targets.py --target twoshot     # emulated 4-rank two-shot AllReduce, 64 MiB per rank
  python benchmarks/profile_targets.py --target oneshot     # emulated 4-rank one-shot AllReduce, 256 KiB per rank
  python benchmarks/profile_targets.py --target gemm_rs     # fused GEMM->reduce-scatter kernel, one rank, 4096 x 4096 x 1792
  python benchmarks/profile_targets.py --target ag_gemm     # fused all-gather->GEMM kernel with the SwiGLU epilogue, one rank, 4096 x 3584 x 4096
  python benchmarks/profile_targets.py --target swiglu      # one-pass SwiGLU kernel, 4096 x 2 x 14336 bf16 in
  python benchmarks/profile_targets.py --target ll          # emulated 4-rank LL AllReduce, 32 KiB per rank
  python benchmarks/profile_targets.py --target pipe        # emulated 4-rank pipelined AllReduce (peer-to-peer form), 64 MiB per rank, ordinary buffers
  python benchmarks/profile_targets.py --target noalloc     # allocation-free one-shot AllReduce over 4 buffers of 64 KiB
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    import torch

    import mini_nccl_b200 as mn
    from mini_nccl_b200 import _lib

    ap = argparse.ArgumentParser()
    ap.add_argument("--target", required=True, choices=["gemm", "gemm_pair", "copy", "twoshot", "oneshot", "gemm_rs", "ag_gemm", "swiglu", "ll", "pipe", "noalloc", "auto_direct"])
    ap.add_argument("--launches", type=int, default=4)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    lib = mn.lib()
    if args.target in ("gemm", "gemm_pair"):
        from mini_nccl_b200.ops import gemm_bf16, gemm_status
        from mini_nccl_b200.ops.gemm import set_pair_mode

        set_pair_mode(1 if args.target == "gemm_pair" else 0)

        a = torch.randn(4096, 4096, device="cuda").to(torch.bfloat16)
        b = torch.randn(3584, 4096, device="cuda").to(torch.bfloat16)
        c = torch.empty(4096, 3584, device="cuda", dtype=torch.bfloat16)
        for _ in range(args.launches):
            gemm_bf16(a, b, out=c)
        torch.cuda.synchronize()
        assert gemm_status() == 0
    elif args.target == "gemm_rs":
        # single rank: the fused kernel's own code path (tile push into the staging slot, flags,
        # owner-side reduction) with local memory standing in for the peers
        from mini_nccl_b200.ops import GemmReduceScatter, gemm_status

        comm = mn.Communicator(1, 0)
        rs = GemmReduceScatter(comm, 4096, 4096)
        a = torch.randn(4096, 1792, device="cuda").to(torch.bfloat16)
        b = torch.randn(4096, 1792, device="cuda").to(torch.bfloat16)
        for _ in range(args.launches):
            rs(a, b)
        torch.cuda.synchronize()
        assert gemm_status() == 0
        comm.destroy()
    elif args.target == "ag_gemm":
        # single rank: the kernel's own code path (rows already local, no communication CTAs) with the
        # SwiGLU epilogue the tensor-parallel block uses: act [4096, 1792] out of a 4096 x 3584 x 4096 product
        from mini_nccl_b200.ops import AllGatherGemm, gemm_status, interleave_gate_up

        comm = mn.Communicator(1, 0)
        ag = AllGatherGemm(comm, 4096, 4096)
        ag.local_shard.copy_(torch.randn(4096, 4096, device="cuda").to(torch.bfloat16))
        w = interleave_gate_up((torch.randn(1792, 4096, device="cuda") * 0.02).to(torch.bfloat16),
                               (torch.randn(1792, 4096, device="cuda") * 0.02).to(torch.bfloat16))
        act = torch.empty(4096, 1792, device="cuda", dtype=torch.bfloat16)
        for _ in range(args.launches):
            ag(w, out=act, swiglu=True)
        torch.cuda.synchronize()
        assert gemm_status() == 0
        comm.destroy()
    elif args.target == "swiglu":
        from mini_nccl_b200.ops import swiglu_bf16

        h = torch.randn(4096, 2 * 14336, device="cuda").to(torch.bfloat16)      # 235 MB in, 117 MB out: larger than the L2
        out = torch.empty(4096, 14336, device="cuda", dtype=torch.bfloat16)
        for _ in range(args.launches):
            swiglu_bf16(h, out=out)
        torch.cuda.synchronize()
    elif args.target == "noalloc":
        n, count = 4, 16384
        ins = [torch.randn(count, device="cuda") for _ in range(n)]
        outs = [torch.empty_like(t) for t in ins]
        sp = (C.c_void_p * n)(*[t.data_ptr() for t in ins])
        rp = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
        lib.mncclLocalAllReduceNoAlloc.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
        for _ in range(args.launches):
            assert lib.mncclLocalAllReduceNoAlloc(sp, rp, n, count, _lib.FLOAT32, _lib.SUM, None) == 0
        torch.cuda.synchronize()
    elif args.target in ("ll", "pipe"):
        n = 4
        world = C.c_void_p()
        assert lib.mncclEmuCreate(n, 64 << 20, C.byref(world)) == 0
        count = (8 << 10) if args.target == "ll" else (16 << 20)
        algo = _lib.ALGO_LL if args.target == "ll" else 7
        ins = [torch.randn(count, device="cuda") for _ in range(n)]        # ordinary buffers
        outs = [torch.empty_like(t) for t in ins]
        sp = (C.c_void_p * n)(*[t.data_ptr() for t in ins])
        rp = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
        for _ in range(args.launches):
            rc = lib.mncclEmuCollective(world, 0, sp, rp, count, _lib.FLOAT32, _lib.FLOAT32, _lib.FLOAT32, _lib.SUM, 0.25, algo, 0, None)
            assert rc == 0, rc
        torch.cuda.synchronize()
        st = (C.c_uint32 * n)()
        assert lib.mncclEmuStatus(world, st, None) == 0 and list(st) == [0] * n
        lib.mncclEmuDestroy(world)
    elif args.target == "auto_direct":
        # four virtual ranks, ORDINARY buffers (plain device tensors), every rank's table complete: the
        # two-shot kernel with lazy direct access agrees inside the kernel and runs on the buffers directly
        n = 4
        world = C.c_void_p()
        assert lib.mncclEmuCreate(n, 8 << 20, C.byref(world)) == 0
        count = 16 << 20                                     # 64 MiB fp32 per rank, far above the 8 MiB staging
        bufs = [torch.randn(count, device="cuda") for _ in range(n)]
        ptrs = (C.c_void_p * n)(*[b.data_ptr() for b in bufs])
        assert lib.mncclEmuSetAutoMap(world, (C.c_int * (n * n))(*([1] * (n * n)))) == 0
        for _ in range(args.launches):
            rc = lib.mncclEmuCollective(world, 0, ptrs, ptrs, count, _lib.FLOAT32, _lib.FLOAT32, _lib.FLOAT32, _lib.SUM,
                                        0.25, _lib.ALGO_TWOSHOT, 0, None)
            assert rc == 0, rc
        torch.cuda.synchronize()
        st = (C.c_uint32 * n)()
        assert lib.mncclEmuStatus(world, st, None) == 0 and list(st) == [0] * n
        direct = (C.c_uint32 * n)()
        assert lib.mncclEmuDirectCalls(world, direct) == 0 and list(direct) == [args.launches] * n, list(direct)
        lib.mncclEmuDestroy(world)
    elif args.target == "copy":
        comm = mn.Communicator(1, 0)
        x = torch.randn(64 << 20, device="cuda")           # 256 MiB fp32
        y = torch.empty(64 << 20, device="cuda", dtype=torch.bfloat16)
        for _ in range(args.launches):
            comm.all_reduce(x, "sum", out=y, scale=0.125)   # cast + scale, one pass
        torch.cuda.synchronize()
        comm.destroy()
    else:
        n = 4
        world = C.c_void_p()
        assert lib.mncclEmuCreate(n, 64 << 20, C.byref(world)) == 0
        count = (16 << 20) if args.target == "twoshot" else (64 << 10)
        algo = _lib.ALGO_TWOSHOT if args.target == "twoshot" else _lib.ALGO_ONESHOT
        ptrs = (C.c_void_p * n)()
        assert lib.mncclEmuAlloc(world, count * 4, ptrs) == 0   # symmetric: zero-copy path
        for _ in range(args.launches):
            rc = lib.mncclEmuCollective(world, 0, ptrs, ptrs, count, _lib.FLOAT32, _lib.FLOAT32, _lib.FLOAT32, _lib.SUM,
                                        0.25, algo, 0, None)
            assert rc == 0, rc
        torch.cuda.synchronize()
        st = (C.c_uint32 * n)()
        assert lib.mncclEmuStatus(world, st, None) == 0 and list(st) == [0] * n
        lib.mncclEmuDestroy(world)
    print("done", args.target)


if __name__ == "__main__":
    main()
