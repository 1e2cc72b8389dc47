"""One tiny end-to-end pass on cuda:0: a GPT-2 shaped decoder steps through the DDP wrapper
(single rank: the fused scale / cast kernel reduces each bucket locally), then one emulated
four-rank AllReduce per algorithm runs through the communication kernels."""
from __future__ import annotations

import ctypes as C


def run() -> None:
    import numpy as np
    import torch

    import mini_nccl_b200 as mn
    from mini_nccl_b200 import _lib
    from mini_nccl_b200.models import GPT2Config, GPT2Model
    from mini_nccl_b200.parallel import DistributedDataParallel
    from mini_nccl_b200.utils import oracle as O

    if not torch.cuda.is_available():
        raise RuntimeError("smoke() needs a CUDA device")
    lib = mn.lib()
    cfg = GPT2Config.tiny()
    torch.manual_seed(0)
    model = GPT2Model(cfg).cuda().to(torch.bfloat16)
    comm = mn.Communicator(1, 0)
    ddp = DistributedDataParallel(model, comm, bucket_mb=0.25, main_grad_dtype=torch.float32)
    ids = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda")
    loss = ddp(ids, ids)
    loss.backward()
    torch.cuda.synchronize()
    assert torch.isfinite(loss).item(), "loss is not finite"
    assert ddp.launches == len(ddp.buckets) and ddp.launches > 0
    for b in ddp.buckets:  # fused cast: fp32 main grads equal the bf16 grads
        assert torch.equal(b.main, b.flat.float()), "fused cast kernel produced wrong main gradients"
    stats = comm.stats()
    assert stats["algo"]["local"] == ddp.launches, stats
    comm.destroy()

    # Emulated 4-rank AllReduce through the LL, one-shot and two-shot kernels.
    world = C.c_void_p()
    assert lib.mncclEmuCreate(4, 0, C.byref(world)) == 0
    try:
        count = 4096 + 7
        ins = [O.make_input(_lib.FLOAT32, count, r) for r in range(4)]
        want = O.oracle_allreduce(ins, _lib.FLOAT32, _lib.SUM)
        for algo in (_lib.ALGO_LL, _lib.ALGO_ONESHOT, _lib.ALGO_TWOSHOT):
            bufs = [torch.from_numpy(a).cuda() for a in ins]
            ptrs = (C.c_void_p * 4)(*[b.data_ptr() for b in bufs])
            rc = lib.mncclEmuCollective(world, 0, ptrs, ptrs, count, _lib.FLOAT32, _lib.FLOAT32, _lib.FLOAT32, _lib.SUM,
                                        1.0, algo, 0, None)
            assert rc == 0, rc
            torch.cuda.synchronize()
            for b in bufs:
                assert np.array_equal(b.cpu().numpy(), want), f"algorithm {algo} mismatch"
    finally:
        lib.mncclEmuDestroy(world)
    # tcgen05 GEMM on single-CTA tiles and on CTA pairs, and the two fused tensor-parallel kernels
    # with one rank, against an fp32 matmul.
    from mini_nccl_b200.ops import gemm_bf16, gemm_status
    from mini_nccl_b200.ops.fused import AllGatherGemm, GemmReduceScatter
    from mini_nccl_b200.ops.gemm import set_pair_mode

    a = (torch.randn(512, 256, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(512, 256, device="cuda") * 0.5).to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    for mode in (0, 1):
        set_pair_mode(mode)
        c = gemm_bf16(a, b)
        torch.cuda.synchronize()
        assert (c.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item(), f"GEMM (pair mode {mode}) mismatch"
    set_pair_mode(-1)
    solo = mn.Communicator(1, 0)
    rs = GemmReduceScatter(solo, 512, 512)
    out = rs(a, b)
    ag = AllGatherGemm(solo, 512, 256)
    ag.local_shard.copy_(a)
    c2 = ag(b)
    torch.cuda.synchronize()
    for got, name in ((out, "GEMM->reduce-scatter"), (c2, "all-gather->GEMM")):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item(), name + " mismatch"
    assert gemm_status() == 0
    solo.destroy()
    print(f"smoke ok: loss={loss.item():.4f} buckets={len(ddp.buckets)} kernels=local,ll,oneshot,twoshot,gemm,gemm_pair,gemm_rs,ag_gemm")
