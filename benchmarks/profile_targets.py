"""Small single-GPU workloads for `ncu`: one kernel family per target, a few launches, inputs
larger than the L2 but far below a GB, so that a capture ends by itself within a minute or two.

  python benchmarks/profile_targets.py --target gemm        # tcgen05 GEMM, 4096 x 3584 x 4096, single-CTA tiles
  python benchmarks/profile_targets.py --target gemm_pair   # the same product on CTA pairs (cta_group::2)
  python benchmarks/profile_targets.py --target copy        # fused cast/scale copy kernel, 256 MiB
  python benchmarks/profile_targets.py --target twoshot     # emulated 4-rank two-shot AllReduce, 64 MiB per rank
  python benchmarks/profile_targets.py --target oneshot     # emulated 4-rank one-shot AllReduce, 256 KiB per rank
  python benchmarks/profile_targets.py --target gemm_rs     # fused GEMM->reduce-scatter kernel, one rank, 4096 x 4096 x 1792
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
    ap.add_argument("--target", required=True, choices=["gemm", "gemm_pair", "copy", "twoshot", "oneshot", "gemm_rs"])
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
